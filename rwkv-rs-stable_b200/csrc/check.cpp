#include "check.h"

#include <cstdint>

#include <cstdio>

namespace rwkv7 {

namespace {
thread_local std::string g_last_error;
}

int fail(int status, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return status;
}

void clear_error() { g_last_error.clear(); }
const char *last_error() { return g_last_error.c_str(); }

std::string shape_string(const int64_t *shape, int ndim) {
    std::string s = "[";
    for (int i = 0; i < ndim; ++i) {
        if (i) s += ", ";
        s += std::to_string(shape[i]);
    }
    return s + "]";
}

const char *dtype_name(int32_t dtype) {
    switch (dtype) {
        case RWKV7_F32: return "F32";
        case RWKV7_BF16: return "BF16";
        case RWKV7_F16: return "F16";
        case RWKV7_I32: return "I32";
        case RWKV7_I64: return "I64";
        case RWKV7_U32: return "U32";
        default: return "?";
    }
}

size_t dtype_size(int32_t dtype) {
    switch (dtype) {
        case RWKV7_F32: case RWKV7_I32: case RWKV7_U32: return 4;
        case RWKV7_BF16: case RWKV7_F16: return 2;
        case RWKV7_I64: return 8;
        default: return 0;
    }
}

int64_t num_elements(const rwkv7_tensor *t) {
    int64_t n = 1;
    for (int i = 0; i < t->ndim; ++i) n *= t->shape[i];
    return n;
}

int check_present(const TensorInfo &x, int ndim) {
    if (x.t == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: tensor descriptor %s is null", x.name);
    if (x.t->ndim != ndim)
        return fail(RWKV7_ERR_SHAPE_MISMATCH,
                    "ShapeMismatch: kernel input rank mismatch for %s: expected rank %d, actual rank %d",
                    x.name, ndim, x.t->ndim);
    if (dtype_size(x.t->dtype) == 0)
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: %s has unknown dtype code %d", x.name, x.t->dtype);
    for (int i = 0; i < ndim; ++i)
        if (x.t->shape[i] < 0)
            return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: %s has negative dimension %d", x.name, i);
    if (x.t->data == nullptr && num_elements(x.t) != 0)
        return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: %s has a null data pointer", x.name);
    return RWKV7_OK;
}

int check_axis_non_empty(const TensorInfo &x, int axis) {
    if (x.dim(axis) == 0)
        return fail(RWKV7_ERR_EMPTY_AXIS, "EmptyAxis: kernel input axis must be non-empty: %s[%d]", x.name, axis);
    return RWKV7_OK;
}

int check_axes_equal(const std::vector<std::pair<TensorInfo, int>> &axes) {
    if (axes.empty()) return RWKV7_OK;
    const auto &ref = axes[0];
    const int64_t ref_dim = ref.first.dim(ref.second);
    for (size_t i = 1; i < axes.size(); ++i) {
        const int64_t d = axes[i].first.dim(axes[i].second);
        if (d != ref_dim)
            return fail(RWKV7_ERR_AXIS_MISMATCH,
                        "AxisMismatch: kernel input axis mismatch: %s[%d]=%lld != %s[%d]=%lld",
                        ref.first.name, ref.second, (long long)ref_dim, axes[i].first.name,
                        axes[i].second, (long long)d);
    }
    return RWKV7_OK;
}

int check_shape(const TensorInfo &x, const std::vector<int64_t> &expected) {
    bool same = (int)expected.size() == x.t->ndim;
    for (int i = 0; same && i < x.t->ndim; ++i) same = x.t->shape[i] == expected[i];
    if (!same)
        return fail(RWKV7_ERR_SHAPE_MISMATCH,
                    "ShapeMismatch: kernel input shape mismatch for %s: expected=%s, actual=%s", x.name,
                    shape_string(expected.data(), (int)expected.size()).c_str(),
                    shape_string(x.t->shape, x.t->ndim).c_str());
    return RWKV7_OK;
}

int check_same_shape(const std::vector<TensorInfo> &xs) {
    if (xs.empty()) return RWKV7_OK;
    std::vector<int64_t> expected(xs[0].t->shape, xs[0].t->shape + xs[0].t->ndim);
    for (size_t i = 1; i < xs.size(); ++i)
        if (int st = check_shape(xs[i], expected)) return st;
    return RWKV7_OK;
}

int check_same_dtype(const std::vector<TensorInfo> &xs) {
    for (size_t i = 1; i < xs.size(); ++i)
        if (xs[i].t->dtype != xs[0].t->dtype)
            return fail(RWKV7_ERR_DTYPE_MISMATCH,
                        "DTypeMismatch: kernel input dtype mismatch: %s=%s, %s=%s", xs[0].name,
                        dtype_name(xs[0].t->dtype), xs[i].name, dtype_name(xs[i].t->dtype));
    return RWKV7_OK;
}

int check_same_device(const std::vector<TensorInfo> &xs) {
    for (size_t i = 1; i < xs.size(); ++i)
        if (xs[i].t->device != xs[0].t->device)
            return fail(RWKV7_ERR_DEVICE_MISMATCH,
                        "DeviceMismatch: kernel input device mismatch: %s=Cuda(%d), %s=Cuda(%d)",
                        xs[0].name, xs[0].t->device, xs[i].name, xs[i].t->device);
    return RWKV7_OK;
}

int check_contiguous(const TensorInfo &x) {
    if (num_elements(x.t) == 0) return RWKV7_OK;  // no element, no observable stride
    int64_t expect = 1;
    for (int i = x.t->ndim - 1; i >= 0; --i) {
        // A stride is only observable on an axis longer than 1.
        if (x.t->shape[i] > 1 && x.t->stride[i] != expect)
            return fail(RWKV7_ERR_NOT_CONTIGUOUS, "NotContiguous: %s must be contiguous", x.name);
        expect *= x.t->shape[i];
    }
    // Every kernel moves tensor data with 16-byte vector accesses or TMA; a view that starts at an odd
    // element of its storage would fault on the device, so it is refused here, on the host.
    if ((reinterpret_cast<uintptr_t>(x.t->data) & 15u) != 0)
        return fail(RWKV7_ERR_UNSUPPORTED,
                    "Unsupported: the data pointer of %s is not 16-byte aligned (the kernels use 16-byte "
                    "vector accesses); pass a tensor whose storage offset is a multiple of 16 bytes", x.name);
    return RWKV7_OK;
}

}  // namespace rwkv7
