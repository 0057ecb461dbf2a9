// extern "C" entry points: input contracts in the reference's order, then
// dispatch to the CUDA launchers.  There is no CPU fallback: every entry point
// either enqueues sm_100a kernels or returns an error status.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <mutex>
#include <vector>

#include "check.h"
#include "kernels.h"
#include "rwkv7_b200.h"
#include "trace.h"

using namespace rwkv7;

namespace {

std::atomic<int> g_wkv7_path{RWKV7_WKV7_AUTO};

constexpr int kMaxDevices = 64;
std::mutex g_props_mu;
int g_num_sms[kMaxDevices] = {};

// Makes `device` current for the duration of a call and restores the caller's.
class DeviceGuard {
   public:
    explicit DeviceGuard(int device) {
        err_ = cudaGetDevice(&prev_);
        if (err_ == cudaSuccess && prev_ != device) {
            err_ = cudaSetDevice(device);
            switched_ = err_ == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (switched_) cudaSetDevice(prev_);
    }
    cudaError_t error() const { return err_; }

   private:
    int prev_ = 0;
    bool switched_ = false;
    cudaError_t err_ = cudaSuccess;
};

int cuda_fail(const char *what, int err) {
    return fail(RWKV7_ERR_CUDA, "CudaError: %s: %s", what, cudaGetErrorString((cudaError_t)err));
}

int num_sms(int device, int *out) {
    if (device < 0 || device >= kMaxDevices)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(g_props_mu);
    if (g_num_sms[device] == 0) {
        int v = 0;
        cudaError_t e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return cuda_fail("cudaDeviceGetAttribute", (int)e);
        g_num_sms[device] = v;
    }
    *out = g_num_sms[device];
    return RWKV7_OK;
}

bool float_dtype_supported(int32_t dt) { return dt == RWKV7_F32 || dt == RWKV7_BF16; }

// Shortest sequence the automatic choice gives to the two-kernel prefill.
constexpr int64_t kSplitMinTokens = 512;

#define RWKV7_TRY(expr)                 \
    do {                                \
        if (int st_ = (expr)) return st_; \
    } while (0)

// check_wkv7_sequence_inputs (wkv7/io.rs:175-241) + the contiguity assertions of
// the CubeBackend impl (wkv7/mod.rs:56-76).  `chunk_len == 16` and
// `T % chunk_len == 0` (io.rs:187,198-201) are properties of the reference's
// backward snapshots, not of the forward arithmetic, and are not required here.
int check_wkv7_sequence(const TensorInfo six[6], int64_t chunk_len) {
    for (int i = 0; i < 6; ++i) RWKV7_TRY(check_present(six[i], 4));
    if (chunk_len <= 0)
        return fail(RWKV7_ERR_BAD_CHUNK, "BadChunk: chunk_len must be positive, got %lld", (long long)chunk_len);
    const TensorInfo &r = six[0];
    RWKV7_TRY(check_axis_non_empty(r, 1));
    RWKV7_TRY(check_axis_non_empty(r, 3));
    RWKV7_TRY(check_axes_equal({{six[0], 0}, {six[1], 0}, {six[2], 0}, {six[3], 0}, {six[4], 0}, {six[5], 0}}));
    const std::vector<int64_t> expected(r.t->shape, r.t->shape + 4);
    for (int i = 1; i < 6; ++i) RWKV7_TRY(check_shape(six[i], expected));
    RWKV7_TRY(check_same_dtype({six[0], six[1], six[2], six[3], six[4], six[5]}));
    RWKV7_TRY(check_same_device({six[0], six[1], six[2], six[3], six[4], six[5]}));
    for (int i = 0; i < 6; ++i) RWKV7_TRY(check_contiguous(six[i]));
    if (!float_dtype_supported(r.t->dtype))
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: wkv7 computes F32 or BF16 inputs, got %s",
                    dtype_name(r.t->dtype));
    return RWKV7_OK;
}

// check_initial_state (wkv7/io.rs:243-258).  The reference keeps the state in the
// sequence dtype; this ABI carries it in F32 for every sequence dtype.
int check_wkv7_state(const TensorInfo &state, const TensorInfo &r) {
    RWKV7_TRY(check_present(state, 4));
    RWKV7_TRY(check_shape(state, {r.dim(0), r.dim(2), r.dim(3), r.dim(3)}));
    if (state.t->dtype != RWKV7_F32)
        return fail(RWKV7_ERR_DTYPE_MISMATCH,
                    "DTypeMismatch: kernel input dtype mismatch: %s=%s, expected F32 state", state.name,
                    dtype_name(state.t->dtype));
    RWKV7_TRY(check_same_device({state, r}));
    RWKV7_TRY(check_contiguous(state));
    return RWKV7_OK;
}

// Contract checks of a WKV7 forward call in the reference's order; fills `p` on success.
int wkv7_validate(const rwkv7_tensor *s0, const rwkv7_tensor *const six_t[6], int64_t chunk_len,
                  rwkv7_tensor *y, rwkv7_tensor *s_out, bool want_state, bool has_s0, Wkv7Args &p) {
    clear_error();
    static const char *names[6] = {"receptance", "weight_decay", "replacement_key",
                                   "value", "removal_key_normalized", "replacement"};
    TensorInfo six[6];
    for (int i = 0; i < 6; ++i) six[i] = TensorInfo{names[i], six_t[i]};
    // Reference order (io.rs:95-106,131-141): sequence inputs first, then the state.
    RWKV7_TRY(check_wkv7_sequence(six, chunk_len));
    const TensorInfo &r = six[0];
    if (has_s0) RWKV7_TRY(check_wkv7_state(TensorInfo{"initial_state", s0}, r));
    const TensorInfo out{"output", y};
    RWKV7_TRY(check_present(out, 4));
    RWKV7_TRY(check_shape(out, std::vector<int64_t>(r.t->shape, r.t->shape + 4)));
    RWKV7_TRY(check_same_dtype({r, out}));
    RWKV7_TRY(check_same_device({r, out}));
    RWKV7_TRY(check_contiguous(out));
    if (want_state) RWKV7_TRY(check_wkv7_state(TensorInfo{"next_state", s_out}, r));

    p = Wkv7Args{};
    p.r = six_t[0]->data; p.w = six_t[1]->data; p.k = six_t[2]->data;
    p.v = six_t[3]->data; p.a = six_t[4]->data; p.b = six_t[5]->data;
    p.s0 = has_s0 ? static_cast<const float *>(s0->data) : nullptr;
    p.y = y->data;
    p.s_out = want_state ? static_cast<float *>(s_out->data) : nullptr;
    p.B = r.dim(0); p.T = r.dim(1); p.H = r.dim(2); p.N = r.dim(3);
    p.bf16 = r.t->dtype == RWKV7_BF16;
    p.device = r.t->device;
    return RWKV7_OK;
}

// Picks the kernel for validated arguments and enqueues it.
int wkv7_dispatch(Wkv7Args &p, void *workspace, size_t workspace_bytes, rwkv7_stream stream) {
    if (p.B == 0 || p.H == 0) return RWKV7_OK;  // nothing to compute

    DeviceGuard guard(p.device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(p.device, &p.num_sms));

    const int path = g_wkv7_path.load();
    bool chunked = false;
    // The two-kernel prefill first, where it applies and the workspace holds at least one segment of
    // operators; chains it leaves flagged (decay beyond what fp16 operands resolve, non-finite values)
    // go to the tf32 chunked kernel, and from there to the sequential scan.
    const bool split_fits = wkv7_split_supported(p) && workspace != nullptr &&
                            workspace_bytes >= wkv7_split_min_workspace_bytes(p.B, p.T, p.H, p.N);
    if (path == RWKV7_WKV7_SPLIT && !split_fits) {
        if (!wkv7_split_supported(p))
            return fail(RWKV7_ERR_UNSUPPORTED,
                        "Unsupported: the two-kernel WKV7 prefill needs N == 64 and 16-byte aligned tensors (got N=%lld)", (long long)p.N);
        return fail(RWKV7_ERR_WORKSPACE_TOO_SMALL, "WorkspaceTooSmall: wkv7 needs %zu workspace bytes, got %zu",
                    wkv7_split_min_workspace_bytes(p.B, p.T, p.H, p.N), workspace == nullptr ? (size_t)0 : workspace_bytes);
    }
    if (path == RWKV7_WKV7_SPLIT || (path == RWKV7_WKV7_AUTO && split_fits && p.T >= kSplitMinTokens)) {
        if (int e = launch_wkv7_split(p, workspace, workspace_bytes, (cudaStream_t)stream))
            return cuda_fail("wkv7 split launch", e);
        // (the tf32 chunked kernel reads bf16 tiles: flagged chains of fp32 tensors go straight to the sequential scan)
        if (int e = p.bf16 ? launch_wkv7_chunked_flagged(p, workspace, (cudaStream_t)stream)
                           : launch_wkv7_sequential_flagged(p, static_cast<const int *>(workspace), (cudaStream_t)stream))
            return cuda_fail("wkv7 flagged-chain launch", e);
        return RWKV7_OK;
    }
    if (path == RWKV7_WKV7_CHUNKED) {
        if (!wkv7_chunked_supported(p))
            return fail(RWKV7_ERR_UNSUPPORTED,
                        "Unsupported: the chunked WKV7 kernel needs N == 64 (got N=%lld)", (long long)p.N);
        chunked = true;
    } else if (path == RWKV7_WKV7_AUTO) {
        chunked = wkv7_chunked_supported(p) && p.T >= 64;
    }
    if (chunked) {
        const size_t need = wkv7_chunked_workspace_bytes(p.B, p.T, p.H, p.N);
        if (need > 0 && (workspace == nullptr || workspace_bytes < need))
            return fail(RWKV7_ERR_WORKSPACE_TOO_SMALL,
                        "WorkspaceTooSmall: wkv7 needs %zu workspace bytes, got %zu", need,
                        workspace == nullptr ? (size_t)0 : workspace_bytes);
        if (int e = launch_wkv7_chunked(p, workspace, workspace_bytes, (cudaStream_t)stream))
            return cuda_fail("wkv7 chunked launch", e);
        return RWKV7_OK;
    }
    if (p.N > 128)
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: head size N=%lld exceeds 128", (long long)p.N);
    if (int e = launch_wkv7_sequential(p, (cudaStream_t)stream)) return cuda_fail("wkv7 sequential launch", e);
    return RWKV7_OK;
}

int wkv7_run(const rwkv7_tensor *s0, const rwkv7_tensor *const six_t[6], int64_t chunk_len,
             rwkv7_tensor *y, rwkv7_tensor *s_out, bool want_state, void *workspace,
             size_t workspace_bytes, rwkv7_stream stream, bool has_s0) {
    Wkv7Args p{};
    RWKV7_TRY(wkv7_validate(s0, six_t, chunk_len, y, s_out, want_state, has_s0, p));
    return wkv7_dispatch(p, workspace, workspace_bytes, stream);
}

// Shared contract of the [1,1,C] scale tensors (mix6/io.rs:48-86, addcmul/io.rs:42-54).
int check_scales(const TensorInfo &x, const rwkv7_tensor *const *scales, const char *const *names, int n) {
    const int64_t C = x.dim(2);
    std::vector<TensorInfo> all{x};
    for (int s = 0; s < n; ++s) {
        TensorInfo info{names[s], scales[s]};
        RWKV7_TRY(check_present(info, 3));
        RWKV7_TRY(check_shape(info, {1, 1, C}));
        all.push_back(info);
    }
    RWKV7_TRY(check_same_dtype(all));
    RWKV7_TRY(check_same_device(all));
    for (auto &t : all) RWKV7_TRY(check_contiguous(t));
    return RWKV7_OK;
}

int check_output_like(const TensorInfo &x, const TensorInfo &out) {
    RWKV7_TRY(check_present(out, x.t->ndim));
    RWKV7_TRY(check_shape(out, std::vector<int64_t>(x.t->shape, x.t->shape + x.t->ndim)));
    RWKV7_TRY(check_same_dtype({x, out}));
    RWKV7_TRY(check_same_device({x, out}));
    RWKV7_TRY(check_contiguous(out));
    return RWKV7_OK;
}

const char *kMixScaleNames[6] = {"receptance_scale", "weight_decay_scale", "key_scale",
                                 "value_scale", "learning_rate_scale", "gate_scale"};
const char *kMixOutNames[6] = {"receptance_input", "weight_decay_input", "key_input",
                               "value_input", "learning_rate_input", "gate_input"};

int mix6_common(const rwkv7_tensor *x_t, const rwkv7_tensor *const scales[6], MixArgs *p) {
    const TensorInfo x{"embedded_context", x_t};
    RWKV7_TRY(check_present(x, 3));
    if (scales == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: scales array is null");
    // Mix6ForwardInputs::check (mix6/io.rs:48-86)
    RWKV7_TRY(check_axis_non_empty(x, 2));
    RWKV7_TRY(check_scales(x, scales, kMixScaleNames, 6));
    if (!float_dtype_supported(x_t->dtype))
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: mix6 computes F32 or BF16, got %s", dtype_name(x_t->dtype));
    p->x = x_t->data;
    for (int s = 0; s < 6; ++s) p->mu[s] = scales[s]->data;
    p->B = x.dim(0); p->T = x.dim(1); p->C = x.dim(2);
    p->bf16 = x_t->dtype == RWKV7_BF16;
    return RWKV7_OK;
}

}  // namespace

extern "C" {

int rwkv7_abi_version(void) { return RWKV7_ABI_VERSION; }

int rwkv7_build_features(void) { return (RWKV7_TRACE_ENABLED ? 1 : 0) | (RWKV7_CHECKED_ENABLED ? 2 : 0); }

const char *rwkv7_status_string(int status) {
    switch (status) {
        case RWKV7_OK: return "Ok";
        case RWKV7_ERR_AXIS_MISMATCH: return "AxisMismatch";
        case RWKV7_ERR_SHAPE_MISMATCH: return "ShapeMismatch";
        case RWKV7_ERR_DTYPE_MISMATCH: return "DTypeMismatch";
        case RWKV7_ERR_DEVICE_MISMATCH: return "DeviceMismatch";
        case RWKV7_ERR_EMPTY_AXIS: return "EmptyAxis";
        case RWKV7_ERR_NOT_CONTIGUOUS: return "NotContiguous";
        case RWKV7_ERR_BAD_CHUNK: return "BadChunk";
        case RWKV7_ERR_UNSUPPORTED: return "Unsupported";
        case RWKV7_ERR_NULL_POINTER: return "NullPointer";
        case RWKV7_ERR_WORKSPACE_TOO_SMALL: return "WorkspaceTooSmall";
        case RWKV7_ERR_CUDA: return "CudaError";
        case RWKV7_ERR_TIMEOUT: return "Timeout";
        case RWKV7_ERR_BAD_INDEX: return "BadIndex";
        case RWKV7_ERR_BAD_ARGUMENT: return "BadArgument";
        default: return "Unknown";
    }
}

const char *rwkv7_last_error_message(void) { return last_error(); }

int rwkv7_set_wkv7_path(int path) {
    if (path < RWKV7_WKV7_AUTO || path > RWKV7_WKV7_SPLIT)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: unknown wkv7 path %d", path);
    g_wkv7_path.store(path);
    return RWKV7_OK;
}

int rwkv7_get_wkv7_path(void) { return g_wkv7_path.load(); }

int rwkv7_set_wkv7_cluster(int cluster_size) {
    if (cluster_size != 0 && cluster_size != 1 && cluster_size != 2 && cluster_size != 4)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: cluster size must be 0 (automatic), 1, 2 or 4, got %d", cluster_size);
    wkv7_set_cluster_override(cluster_size);
    return RWKV7_OK;
}

int rwkv7_set_wkv7_overlap(int on) {
    wkv7_set_split_overlap(on);
    return RWKV7_OK;
}

int64_t rwkv7_kernel_launch_count(void) { return launch_count(); }

int rwkv7_read_device_status(int device, rwkv7_stream stream) {
    clear_error();
    DeviceGuard guard(device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    int *word = nullptr;
    if (int e = device_status_ptr(device, &word)) return cuda_fail("device status word", e);
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(word, 0, sizeof(int), (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail("reading the device status word", (int)e);
    if (host == kDevTimeout) return fail(RWKV7_ERR_TIMEOUT, "Timeout: a bounded device-side wait expired");
    if (host == kDevBadIndex) return fail(RWKV7_ERR_BAD_INDEX, "BadIndex: a device-side index was out of range");
    if (host == kDevInternal) return fail(RWKV7_ERR_CUDA, "CudaError: a kernel's own precondition check failed (shared memory alignment)");
    return RWKV7_OK;
}

int rwkv7_selftest_bounded_wait(int device, int64_t max_polls, rwkv7_stream stream) {
    clear_error();
    if (max_polls < 1 || max_polls > 1000000)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: max_polls must be in [1, 1000000], got %lld", (long long)max_polls);
    DeviceGuard guard(device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    if (int e = launch_bounded_wait_selftest(device, (unsigned)max_polls, (cudaStream_t)stream))
        return cuda_fail("bounded-wait self-test launch", e);
    return RWKV7_OK;
}

size_t rwkv7_wkv7_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N, int32_t dtype) {
    const int path = g_wkv7_path.load();
    if (path == RWKV7_WKV7_SEQUENTIAL) return 0;
    if ((path == RWKV7_WKV7_SPLIT || (path == RWKV7_WKV7_AUTO && T >= kSplitMinTokens)) &&
        (dtype == RWKV7_BF16 || dtype == RWKV7_F32) && N == 64)
    {
        // (the size depends on whether the scan will overlap the operator kernel, i.e. on the SM count of
        // the device the call will run on: the calling thread's current device is taken)
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || num_sms(dev, &sms) != RWKV7_OK) sms = 0;
        (void)cudaGetLastError();
        return wkv7_split_workspace_bytes(B, T, H, N, sms);
    }
    return wkv7_chunked_workspace_bytes(B, T, H, N);
}

int rwkv7_fused_wkv7_pretrain(const rwkv7_tensor *r, const rwkv7_tensor *w, const rwkv7_tensor *k,
                              const rwkv7_tensor *v, const rwkv7_tensor *a, const rwkv7_tensor *b,
                              int64_t chunk_len, rwkv7_tensor *output, void *workspace,
                              size_t workspace_bytes, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer.wkv7_pretrain");
    const rwkv7_tensor *six[6] = {r, w, k, v, a, b};
    return wkv7_run(nullptr, six, chunk_len, output, nullptr, false, workspace, workspace_bytes, stream, false);
}

int rwkv7_fused_wkv7_statetune(const rwkv7_tensor *s0, const rwkv7_tensor *r, const rwkv7_tensor *w,
                               const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                               const rwkv7_tensor *b, int64_t chunk_len, rwkv7_tensor *output,
                               void *workspace, size_t workspace_bytes, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer_statetune.wkv7");
    const rwkv7_tensor *six[6] = {r, w, k, v, a, b};
    return wkv7_run(s0, six, chunk_len, output, nullptr, false, workspace, workspace_bytes, stream, true);
}

int rwkv7_fused_wkv7_statepass(const rwkv7_tensor *s0, const rwkv7_tensor *r, const rwkv7_tensor *w,
                               const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                               const rwkv7_tensor *b, int64_t chunk_len, rwkv7_tensor *output,
                               rwkv7_tensor *next_state, void *workspace, size_t workspace_bytes,
                               rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer.wkv7");
    const rwkv7_tensor *six[6] = {r, w, k, v, a, b};
    return wkv7_run(s0, six, chunk_len, output, next_state, true, workspace, workspace_bytes, stream, true);
}

int rwkv7_fused_wkv7_statepass_noalloc(const rwkv7_tensor *s0, const rwkv7_tensor *r, const rwkv7_tensor *w,
                                       const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                                       const rwkv7_tensor *b, int64_t chunk_len, rwkv7_tensor *output,
                                       rwkv7_tensor *next_state, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer.wkv7");
    // The reference-ordered contract checks come first, so that a malformed call reports the same
    // error here as through rwkv7_fused_wkv7_statepass; only then the capacity of the fixed array.
    const rwkv7_tensor *six[6] = {r, w, k, v, a, b};
    Wkv7Args p{};
    RWKV7_TRY(wkv7_validate(s0, six, chunk_len, output, next_state, true, true, p));
    const int64_t cap = wkv7_static_scratch_max_chains();
    if (p.B > cap || p.H > cap || p.B * p.H > cap)
        return fail(RWKV7_ERR_UNSUPPORTED,
                    "Unsupported: B*H = %lld chains exceed the %lld-chain capacity of the allocation-free "
                    "entry point; use rwkv7_fused_wkv7_statepass with a workspace",
                    (long long)(p.B * p.H), (long long)cap);
    if (p.B == 0 || p.H == 0) return RWKV7_OK;
    DeviceGuard guard(p.device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    if (int e = wkv7_static_scratch(p.device, &scratch, &scratch_bytes)) return cuda_fail("static scratch address", e);
    return wkv7_dispatch(p, scratch, scratch_bytes, stream);
}

// ---- wkv7 from pinned host buffers ---------------------------------------------------------

namespace {

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// Device memory of one slice set: six sequence tensors, y, state in, state out, workspace.
struct HostSliceLayout {
    size_t seq, state, ws, total;
};

HostSliceLayout host_slice_layout(int64_t rows, int64_t T, int64_t H, int64_t N, int32_t dtype) {
    HostSliceLayout l{};
    l.seq = align256((size_t)(rows * T * H * N) * dtype_size(dtype));
    l.state = align256((size_t)(rows * H * N * N) * sizeof(float));
    l.ws = align256(rwkv7_wkv7_workspace_bytes(rows, T, H, N, dtype));
    l.total = 7 * l.seq + 2 * l.state + l.ws;
    return l;
}

}  // namespace

size_t rwkv7_wkv7_host_staging_bytes(int64_t B, int64_t T, int64_t H, int64_t N, int32_t dtype, int32_t slices,
                                     int32_t n_streams) {
    if (slices < 1 || n_streams < 1 || B < 0 || T < 0 || H < 0 || N < 0 || B % slices != 0 || dtype_size(dtype) == 0)
        return 0;
    const int32_t sets = n_streams < slices ? n_streams : slices;
    return (size_t)sets * host_slice_layout(B / slices, T, H, N, dtype).total;
}

int rwkv7_wkv7_host_join(int32_t device, const rwkv7_stream *streams, int32_t n_streams, rwkv7_stream caller_stream) {
    clear_error();
    if (streams == nullptr || n_streams < 1)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: at least one worker stream is required");
    DeviceGuard guard(device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    for (int32_t i = 0; i < n_streams; ++i) {
        cudaEvent_t ev;
        cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventRecord(ev, (cudaStream_t)streams[i]);
        if (e == cudaSuccess) e = cudaStreamWaitEvent((cudaStream_t)caller_stream, ev, 0);
        cudaEventDestroy(ev);   // (released once the recorded work has completed)
        if (e != cudaSuccess) return cuda_fail("joining the worker streams", (int)e);
    }
    return RWKV7_OK;
}

int rwkv7_wkv7_statepass_host(const rwkv7_tensor *host_s0, const rwkv7_tensor *const host_six[6], int64_t chunk_len,
                              rwkv7_tensor *host_y, rwkv7_tensor *host_s_out, int32_t device, int32_t slices,
                              void *device_staging, size_t staging_bytes, const rwkv7_stream *streams,
                              int32_t n_streams, rwkv7_stream caller_stream, int32_t flags) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer.wkv7_host");
    clear_error();
    if (host_six == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: the array of sequence tensors is null");
    if (streams == nullptr || n_streams < 1)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: at least one worker stream is required");
    // The contract of the device-resident statepass, applied to the host descriptors.
    Wkv7Args whole{};
    RWKV7_TRY(wkv7_validate(host_s0, host_six, chunk_len, host_y, host_s_out, true, host_s0 != nullptr, whole));
    if (host_six[0]->device != RWKV7_HOST)
        return fail(RWKV7_ERR_DEVICE_MISMATCH, "DeviceMismatch: host tensors must carry device = RWKV7_HOST (-1), got %d",
                    host_six[0]->device);
    const int64_t B = whole.B, T = whole.T, H = whole.H, N = whole.N;
    if (slices < 1 || B % slices != 0)
        return fail(RWKV7_ERR_SHAPE_MISMATCH, "ShapeMismatch: %d slices do not divide B=%lld", slices, (long long)B);
    if (B == 0 || H == 0) return RWKV7_OK;
    const int32_t dtype = host_six[0]->dtype;
    const int64_t rows = B / slices;
    const int32_t sets = n_streams < slices ? n_streams : slices;
    const HostSliceLayout lay = host_slice_layout(rows, T, H, N, dtype);
    if (device_staging == nullptr || staging_bytes < (size_t)sets * lay.total)
        return fail(RWKV7_ERR_WORKSPACE_TOO_SMALL, "WorkspaceTooSmall: the host statepass needs %zu bytes of device staging, got %zu",
                    (size_t)sets * lay.total, device_staging == nullptr ? (size_t)0 : staging_bytes);
    if ((reinterpret_cast<uintptr_t>(device_staging) & 255u) != 0)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: device staging must be 256-byte aligned");
    DeviceGuard guard(device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());

    // fork: every worker stream starts after what the caller has enqueued so far
    {
        cudaEvent_t ev;
        cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventRecord(ev, (cudaStream_t)caller_stream);
        for (int32_t i = 0; e == cudaSuccess && i < sets; ++i) e = cudaStreamWaitEvent((cudaStream_t)streams[i], ev, 0);
        cudaEventDestroy(ev);
        if (e != cudaSuccess) return cuda_fail("ordering the worker streams after the caller's stream", (int)e);
    }
    const size_t seq_bytes = (size_t)(rows * T * H * N) * dtype_size(dtype);
    const size_t state_bytes = (size_t)(rows * H * N * N) * sizeof(float);
    for (int32_t i = 0; i < slices; ++i) {
        const int32_t set = i % sets;
        cudaStream_t st = (cudaStream_t)streams[set];
        unsigned char *base = static_cast<unsigned char *>(device_staging) + (size_t)set * lay.total;
        unsigned char *dev_six[6];
        for (int k = 0; k < 6; ++k) dev_six[k] = base + (size_t)k * lay.seq;
        unsigned char *dev_y = base + 6 * lay.seq;
        unsigned char *dev_s_in = base + 7 * lay.seq, *dev_s_out = dev_s_in + lay.state, *dev_ws = dev_s_out + lay.state;
        cudaError_t e = cudaSuccess;
        for (int k = 0; e == cudaSuccess && k < 6; ++k)
            e = cudaMemcpyAsync(dev_six[k], static_cast<const unsigned char *>(host_six[k]->data) + (size_t)i * seq_bytes,
                                seq_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) {
            if (host_s0 != nullptr)
                e = cudaMemcpyAsync(dev_s_in, static_cast<const unsigned char *>(host_s0->data) + (size_t)i * state_bytes,
                                    state_bytes, cudaMemcpyHostToDevice, st);
            else
                e = cudaMemsetAsync(dev_s_in, 0, state_bytes, st);
        }
        if (e != cudaSuccess) return cuda_fail("copying a batch slice to the device", (int)e);
        Wkv7Args p = whole;
        p.r = dev_six[0]; p.w = dev_six[1]; p.k = dev_six[2]; p.v = dev_six[3]; p.a = dev_six[4]; p.b = dev_six[5];
        p.s0 = reinterpret_cast<const float *>(dev_s_in);
        p.y = dev_y;
        p.s_out = reinterpret_cast<float *>(dev_s_out);
        p.B = rows;
        p.device = device;
        RWKV7_TRY(wkv7_dispatch(p, dev_ws, lay.ws, (rwkv7_stream)st));
        e = cudaMemcpyAsync(static_cast<unsigned char *>(host_y->data) + (size_t)i * seq_bytes, dev_y, seq_bytes,
                            cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(static_cast<unsigned char *>(host_s_out->data) + (size_t)i * state_bytes, dev_s_out,
                                state_bytes, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) return cuda_fail("copying a batch slice back to the host", (int)e);
    }
    if (flags & RWKV7_HOST_NO_JOIN) return RWKV7_OK;
    return rwkv7_wkv7_host_join(device, streams, sets, caller_stream);
}

namespace {

const char *kSixNames[6] = {"receptance", "weight_decay", "replacement_key",
                            "value", "removal_key_normalized", "replacement"};

// The reference's training contract (wkv7/io.rs:187,198-201): positive chunk_len dividing T.
int check_training_chunks(const TensorInfo &r, int64_t chunk_len) {
    if (r.dim(1) % chunk_len != 0)
        return fail(RWKV7_ERR_BAD_CHUNK, "BadChunk: context_len must be a multiple of chunk_len");
    return RWKV7_OK;
}

int check_snapshots(const TensorInfo &snap, const TensorInfo &r, int64_t chunk_len) {
    RWKV7_TRY(check_present(snap, 5));
    RWKV7_TRY(check_shape(snap, {r.dim(0), r.dim(2), r.dim(1) / chunk_len, r.dim(3), r.dim(3)}));
    if (snap.t->dtype != RWKV7_F32)
        return fail(RWKV7_ERR_DTYPE_MISMATCH, "DTypeMismatch: kernel input dtype mismatch: %s=%s, expected F32",
                    snap.name, dtype_name(snap.t->dtype));
    RWKV7_TRY(check_same_device({snap, r}));
    return check_contiguous(snap);
}

}  // namespace

int rwkv7_fused_wkv7_forward_saved(const rwkv7_tensor *s0, const rwkv7_tensor *r_t, const rwkv7_tensor *w,
                                   const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                                   const rwkv7_tensor *b, int64_t chunk_len, rwkv7_tensor *output,
                                   rwkv7_tensor *next_state, rwkv7_tensor *snapshots,
                                   rwkv7_tensor *state_replacement, void *workspace, size_t workspace_bytes,
                                   rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.train.model.time_mixer.wkv7_forward");
    clear_error();
    const rwkv7_tensor *six_t[6] = {r_t, w, k, v, a, b};
    TensorInfo six[6];
    for (int i = 0; i < 6; ++i) six[i] = TensorInfo{kSixNames[i], six_t[i]};
    RWKV7_TRY(check_wkv7_sequence(six, chunk_len));
    const TensorInfo &r = six[0];
    RWKV7_TRY(check_training_chunks(r, chunk_len));
    if (s0 != nullptr) RWKV7_TRY(check_wkv7_state(TensorInfo{"initial_state", s0}, r));
    RWKV7_TRY(check_output_like(r, TensorInfo{"output", output}));
    if (next_state != nullptr) RWKV7_TRY(check_wkv7_state(TensorInfo{"next_state", next_state}, r));
    RWKV7_TRY(check_snapshots(TensorInfo{"snapshots", snapshots}, r, chunk_len));
    RWKV7_TRY(check_output_like(r, TensorInfo{"state_replacement", state_replacement}));
    Wkv7Args p{};
    p.r = r_t->data; p.w = w->data; p.k = k->data; p.v = v->data; p.a = a->data; p.b = b->data;
    p.s0 = s0 ? static_cast<const float *>(s0->data) : nullptr;
    p.y = output->data;
    p.s_out = next_state ? static_cast<float *>(next_state->data) : nullptr;
    p.B = r.dim(0); p.T = r.dim(1); p.H = r.dim(2); p.N = r.dim(3);
    p.bf16 = r_t->dtype == RWKV7_BF16;
    p.device = r_t->device;
    if (p.B == 0 || p.H == 0) return RWKV7_OK;
    if (p.N > 128) return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: head size N=%lld exceeds 128", (long long)p.N);
    DeviceGuard guard(p.device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(p.device, &p.num_sms));
    // The tensor-core kernel writes snapshots every 16 tokens; other chunk lengths, head sizes and
    // fp32 tensors take the sequential scan.
    const int path = g_wkv7_path.load();
    if (path != RWKV7_WKV7_SEQUENTIAL && chunk_len == 16 && p.T >= 64 && wkv7_chunked_supported(p) &&
        (reinterpret_cast<uintptr_t>(state_replacement->data) & 15u) == 0) {
        const size_t need = wkv7_chunked_workspace_bytes(p.B, p.T, p.H, p.N);
        if (workspace == nullptr || workspace_bytes < need)
            return fail(RWKV7_ERR_WORKSPACE_TOO_SMALL, "WorkspaceTooSmall: wkv7 needs %zu workspace bytes, got %zu", need,
                        workspace == nullptr ? (size_t)0 : workspace_bytes);
        if (int e = launch_wkv7_chunked_saved(p, workspace, static_cast<float *>(snapshots->data),
                                              state_replacement->data, (cudaStream_t)stream))
            return cuda_fail("wkv7 training forward launch", e);
        return RWKV7_OK;
    }
    if (int e = launch_wkv7_forward_saved(p, static_cast<float *>(snapshots->data), state_replacement->data,
                                          (int)chunk_len, (cudaStream_t)stream))
        return cuda_fail("wkv7 training forward launch", e);
    return RWKV7_OK;
}

size_t rwkv7_wkv7_backward_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N) {
    if (B <= 0 || T <= 0 || H <= 0) return 0;
    return wkv7_backward_parallel_workspace_bytes(B, T, H, N);
}

static int wkv7_backward_impl(const rwkv7_tensor *s0, const rwkv7_tensor *r_t, const rwkv7_tensor *w,
                              const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                              const rwkv7_tensor *b, const rwkv7_tensor *snapshots, const rwkv7_tensor *state_replacement,
                              int64_t chunk_len, const rwkv7_tensor *output_grad,
                              const rwkv7_tensor *next_state_grad, rwkv7_tensor *const sequence_grads[6],
                              rwkv7_tensor *initial_state_grad, bool parallel, void *workspace, size_t workspace_bytes,
                              rwkv7_stream stream);

int rwkv7_fused_wkv7_backward(const rwkv7_tensor *s0, const rwkv7_tensor *r_t, const rwkv7_tensor *w,
                              const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                              const rwkv7_tensor *b, const rwkv7_tensor *snapshots, const rwkv7_tensor *state_replacement,
                              int64_t chunk_len, const rwkv7_tensor *output_grad,
                              const rwkv7_tensor *next_state_grad, rwkv7_tensor *const sequence_grads[6],
                              rwkv7_tensor *initial_state_grad, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.train.model.time_mixer.wkv7_backward");
    return wkv7_backward_impl(s0, r_t, w, k, v, a, b, snapshots, state_replacement, chunk_len, output_grad,
                              next_state_grad, sequence_grads, initial_state_grad, false, nullptr, 0, stream);
}

int rwkv7_fused_wkv7_backward_parallel(const rwkv7_tensor *s0, const rwkv7_tensor *r_t, const rwkv7_tensor *w,
                                       const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                                       const rwkv7_tensor *b, const rwkv7_tensor *snapshots,
                                       const rwkv7_tensor *state_replacement, int64_t chunk_len,
                                       const rwkv7_tensor *output_grad, const rwkv7_tensor *next_state_grad,
                                       rwkv7_tensor *const sequence_grads[6], rwkv7_tensor *initial_state_grad,
                                       void *workspace, size_t workspace_bytes, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.train.model.time_mixer.wkv7_backward");
    return wkv7_backward_impl(s0, r_t, w, k, v, a, b, snapshots, state_replacement, chunk_len, output_grad,
                              next_state_grad, sequence_grads, initial_state_grad, true, workspace, workspace_bytes,
                              stream);
}

static int wkv7_backward_impl(const rwkv7_tensor *s0, const rwkv7_tensor *r_t, const rwkv7_tensor *w,
                              const rwkv7_tensor *k, const rwkv7_tensor *v, const rwkv7_tensor *a,
                              const rwkv7_tensor *b, const rwkv7_tensor *snapshots, const rwkv7_tensor *state_replacement,
                              int64_t chunk_len, const rwkv7_tensor *output_grad,
                              const rwkv7_tensor *next_state_grad, rwkv7_tensor *const sequence_grads[6],
                              rwkv7_tensor *initial_state_grad, bool parallel, void *workspace, size_t workspace_bytes,
                              rwkv7_stream stream) {
    clear_error();
    const rwkv7_tensor *six_t[6] = {r_t, w, k, v, a, b};
    TensorInfo six[6];
    for (int i = 0; i < 6; ++i) six[i] = TensorInfo{kSixNames[i], six_t[i]};
    RWKV7_TRY(check_wkv7_sequence(six, chunk_len));
    const TensorInfo &r = six[0];
    RWKV7_TRY(check_training_chunks(r, chunk_len));
    if (chunk_len > 16 || chunk_len % 4 != 0)
        return fail(RWKV7_ERR_BAD_CHUNK, "BadChunk: the backward pass supports chunk_len 4, 8, 12 or 16, got %lld",
                    (long long)chunk_len);
    if (s0 != nullptr) RWKV7_TRY(check_wkv7_state(TensorInfo{"initial_state", s0}, r));
    RWKV7_TRY(check_snapshots(TensorInfo{"snapshots", snapshots}, r, chunk_len));
    RWKV7_TRY(check_output_like(r, TensorInfo{"state_replacement", state_replacement}));
    RWKV7_TRY(check_output_like(r, TensorInfo{"output_grad", output_grad}));
    if (next_state_grad != nullptr) RWKV7_TRY(check_wkv7_state(TensorInfo{"next_state_grad", next_state_grad}, r));
    if (sequence_grads == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: sequence_grads array is null");
    static const char *grad_names[6] = {"receptance_grad", "weight_decay_grad", "replacement_key_grad",
                                        "value_grad", "removal_key_normalized_grad", "replacement_grad"};
    for (int i = 0; i < 6; ++i) RWKV7_TRY(check_output_like(r, TensorInfo{grad_names[i], sequence_grads[i]}));
    if (initial_state_grad != nullptr)
        RWKV7_TRY(check_wkv7_state(TensorInfo{"initial_state_grad", initial_state_grad}, r));
    Wkv7BackwardArgs p{};
    p.r = r_t->data; p.w = w->data; p.k = k->data; p.v = v->data; p.a = a->data; p.b = b->data;
    p.snapshots = static_cast<const float *>(snapshots->data);
    p.state_replacement = state_replacement->data;
    p.output_grad = output_grad->data;
    p.initial_state = s0 ? static_cast<const float *>(s0->data) : nullptr;
    p.next_state_grad = next_state_grad ? static_cast<const float *>(next_state_grad->data) : nullptr;
    p.receptance_grad = sequence_grads[0]->data; p.weight_decay_grad = sequence_grads[1]->data;
    p.replacement_key_grad = sequence_grads[2]->data; p.value_grad = sequence_grads[3]->data;
    p.removal_key_normalized_grad = sequence_grads[4]->data; p.replacement_grad = sequence_grads[5]->data;
    p.initial_state_grad = initial_state_grad ? static_cast<float *>(initial_state_grad->data) : nullptr;
    p.B = r.dim(0); p.T = r.dim(1); p.H = r.dim(2); p.N = r.dim(3); p.chunk_len = chunk_len;
    p.bf16 = r_t->dtype == RWKV7_BF16;
    if (p.B == 0 || p.H == 0) return RWKV7_OK;
    if (p.N > 64)
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: the backward pass keeps its work matrices in shared memory, "
                                           "head size N=%lld exceeds 64", (long long)p.N);
    DeviceGuard guard(r_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    if (parallel && wkv7_backward_parallel_supported(p)) {
        // (shapes outside the time-parallel form take the token-by-token kernel below)
        const size_t need = wkv7_backward_parallel_workspace_bytes(p.B, p.T, p.H, p.N);
        if (workspace == nullptr || workspace_bytes < need)
            return fail(RWKV7_ERR_WORKSPACE_TOO_SMALL, "WorkspaceTooSmall: wkv7 backward needs %zu workspace bytes, got %zu",
                        need, workspace == nullptr ? (size_t)0 : workspace_bytes);
        if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
            return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: the backward workspace must be 256-byte aligned");
        int sms = 0;
        RWKV7_TRY(num_sms(r_t->device, &sms));
        if (int e = launch_wkv7_backward_parallel(p, workspace, r_t->device, sms, (cudaStream_t)stream))
            return cuda_fail("wkv7 backward (time-parallel) launch", e);
        return RWKV7_OK;
    }
    if (int e = launch_wkv7_backward(p, (cudaStream_t)stream)) return cuda_fail("wkv7 backward launch", e);
    return RWKV7_OK;
}

int rwkv7_fused_mix6(const rwkv7_tensor *x_t, const rwkv7_tensor *const scales[6],
                     rwkv7_tensor *const outputs[6], rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer.mix6");
    clear_error();
    MixArgs p{};
    RWKV7_TRY(mix6_common(x_t, scales, &p));
    if (outputs == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: outputs array is null");
    const TensorInfo x{"embedded_context", x_t};
    for (int s = 0; s < 6; ++s) {
        RWKV7_TRY(check_output_like(x, TensorInfo{kMixOutNames[s], outputs[s]}));
        p.out[s] = outputs[s]->data;
    }
    DeviceGuard guard(x_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(x_t->device, &p.num_sms));
    if (int e = launch_mix6(p, (cudaStream_t)stream)) return cuda_fail("mix6 launch", e);
    return RWKV7_OK;
}

int rwkv7_fused_mix6_stacked(const rwkv7_tensor *x_t, const rwkv7_tensor *const scales[6],
                             rwkv7_tensor *stacked, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer.mix6");
    clear_error();
    MixArgs p{};
    RWKV7_TRY(mix6_common(x_t, scales, &p));
    const TensorInfo x{"embedded_context", x_t};
    const TensorInfo out{"stacked_output", stacked};
    RWKV7_TRY(check_present(out, 4));
    RWKV7_TRY(check_shape(out, {6, p.B, p.T, p.C}));
    RWKV7_TRY(check_same_dtype({x, out}));
    RWKV7_TRY(check_same_device({x, out}));
    RWKV7_TRY(check_contiguous(out));
    const size_t plane = (size_t)(p.B * p.T * p.C) * dtype_size(x_t->dtype);
    for (int s = 0; s < 6; ++s) p.out[s] = static_cast<char *>(stacked->data) + plane * s;
    DeviceGuard guard(x_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(x_t->device, &p.num_sms));
    if (int e = launch_mix6(p, (cudaStream_t)stream)) return cuda_fail("mix6 launch", e);
    return RWKV7_OK;
}

static int addcmul_run(const rwkv7_tensor *base_t, const rwkv7_tensor *diff_t,
                       const rwkv7_tensor *const *scales, rwkv7_tensor *const *outputs, int n,
                       const char *const *scale_names, const char *const *out_names,
                       rwkv7_stream stream) {
    clear_error();
    const TensorInfo base{"base", base_t}, diff{"diff", diff_t};
    RWKV7_TRY(check_present(base, 3));
    RWKV7_TRY(check_present(diff, 3));
    if (scales == nullptr || outputs == nullptr)
        return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: scales or outputs array is null");
    // AddcmulForwardInputs::check / Addcmul5ForwardInputs::check (addcmul/io.rs:42-54,108-150)
    RWKV7_TRY(check_axis_non_empty(base, 2));
    RWKV7_TRY(check_same_shape({base, diff}));
    const int64_t C = base.dim(2);
    std::vector<TensorInfo> all{base, diff};
    for (int s = 0; s < n; ++s) {
        TensorInfo info{scale_names[s], scales[s]};
        RWKV7_TRY(check_present(info, 3));
        RWKV7_TRY(check_shape(info, {1, 1, C}));
        all.push_back(info);
    }
    RWKV7_TRY(check_same_dtype(all));
    RWKV7_TRY(check_same_device(all));
    for (auto &t : all) RWKV7_TRY(check_contiguous(t));
    if (!float_dtype_supported(base_t->dtype))
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: addcmul computes F32 or BF16, got %s", dtype_name(base_t->dtype));
    AddcmulArgs p{};
    p.base = base_t->data; p.diff = diff_t->data; p.nscale = n;
    p.rows = base.dim(0) * base.dim(1); p.C = C; p.bf16 = base_t->dtype == RWKV7_BF16;
    for (int s = 0; s < n; ++s) {
        RWKV7_TRY(check_output_like(base, TensorInfo{out_names[s], outputs[s]}));
        p.scale[s] = scales[s]->data;
        p.out[s] = outputs[s]->data;
    }
    DeviceGuard guard(base_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(base_t->device, &p.num_sms));
    if (int e = launch_addcmul(p, (cudaStream_t)stream)) return cuda_fail("addcmul launch", e);
    return RWKV7_OK;
}

int rwkv7_fused_addcmul(const rwkv7_tensor *base, const rwkv7_tensor *diff, const rwkv7_tensor *scale,
                        rwkv7_tensor *output, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.addcmul");
    static const char *sn[1] = {"scale"};
    static const char *on[1] = {"output"};
    const rwkv7_tensor *scales[1] = {scale};
    rwkv7_tensor *outs[1] = {output};
    return addcmul_run(base, diff, scales, outs, 1, sn, on, stream);
}

int rwkv7_fused_addcmul5(const rwkv7_tensor *base, const rwkv7_tensor *diff,
                         const rwkv7_tensor *const scales[5], rwkv7_tensor *const outputs[5],
                         rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.addcmul5");
    return addcmul_run(base, diff, scales, outputs, 5, kMixScaleNames, kMixOutNames, stream);
}

int rwkv7_fused_token_shift_diff(const rwkv7_tensor *x_t, rwkv7_tensor *state_t,
                                 const rwkv7_tensor *ids_t, rwkv7_tensor *diff_t, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.time_mixer.token_shift_diff");
    clear_error();
    const TensorInfo x{"embedded_context", x_t}, state{"embedded_token_shift", state_t},
        ids{"batch_ids", ids_t};
    RWKV7_TRY(check_present(x, 3));
    RWKV7_TRY(check_present(state, 2));
    RWKV7_TRY(check_present(ids, 1));
    // TokenShiftDiffForwardInputs::check (token_shift_diff/io.rs:50-66)
    RWKV7_TRY(check_axis_non_empty(x, 2));
    RWKV7_TRY(check_shape(state, {state.dim(0), x.dim(2)}));
    RWKV7_TRY(check_shape(ids, {x.dim(0)}));
    RWKV7_TRY(check_same_dtype({x, state}));
    RWKV7_TRY(check_same_device({x, state, ids}));
    RWKV7_TRY(check_contiguous(x));
    RWKV7_TRY(check_contiguous(state));
    RWKV7_TRY(check_contiguous(ids));
    if (!float_dtype_supported(x_t->dtype))
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: token_shift_diff computes F32 or BF16, got %s", dtype_name(x_t->dtype));
    if (ids_t->dtype != RWKV7_I32 && ids_t->dtype != RWKV7_I64 && ids_t->dtype != RWKV7_U32)
        return fail(RWKV7_ERR_DTYPE_MISMATCH, "DTypeMismatch: batch_ids must be I32, I64 or U32, got %s", dtype_name(ids_t->dtype));
    RWKV7_TRY(check_output_like(x, TensorInfo{"token_shifted_diff", diff_t}));
    TokenShiftArgs p{};
    p.x = x_t->data; p.state = state_t->data; p.ids = ids_t->data; p.ids_dtype = ids_t->dtype;
    p.diff = diff_t->data;
    p.B = x.dim(0); p.T = x.dim(1); p.C = x.dim(2); p.S = state.dim(0);
    p.bf16 = x_t->dtype == RWKV7_BF16;
    if (p.B == 0 || p.T == 0) return RWKV7_OK;  // token_shift_diff/mod.rs:88-97: T == 0 is a no-op
    DeviceGuard guard(x_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(x_t->device, &p.num_sms));
    if (int e = device_status_ptr(x_t->device, &p.status)) return cuda_fail("device status word", e);
    if (int e = launch_token_shift_diff(p, (cudaStream_t)stream)) return cuda_fail("token_shift_diff launch", e);
    return RWKV7_OK;
}

namespace {

// A [B,T,C] or [B,T,H,N] tensor (the same memory): non-null, 3 or 4 axes, contiguous.
int check_sequence_tensor(const TensorInfo &x) {
    if (x.t == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: %s descriptor is null", x.name);
    if (x.t->ndim != 3 && x.t->ndim != 4)
        return fail(RWKV7_ERR_AXIS_MISMATCH, "AxisMismatch: %s has %d axes, expected [B,T,C] or [B,T,H,N]", x.name,
                    x.t->ndim);
    RWKV7_TRY(check_present(x, x.t->ndim));
    return check_contiguous(x);
}

int64_t channels_of(const rwkv7_tensor *t) { return t->ndim == 4 ? t->shape[2] * t->shape[3] : t->shape[2]; }

// Same batch, context length, channel count, dtype and device as `ref` (either axis form).
int check_sequence_like(const TensorInfo &ref, const TensorInfo &x) {
    RWKV7_TRY(check_sequence_tensor(x));
    if (x.dim(0) != ref.dim(0) || x.dim(1) != ref.dim(1) || channels_of(x.t) != channels_of(ref.t))
        return fail(RWKV7_ERR_SHAPE_MISMATCH, "ShapeMismatch: %s is %s, expected the extent of %s %s", x.name,
                    shape_string(x.t->shape, x.t->ndim).c_str(), ref.name,
                    shape_string(ref.t->shape, ref.t->ndim).c_str());
    RWKV7_TRY(check_same_dtype({ref, x}));
    return check_same_device({ref, x});
}

// A per-channel parameter: any contiguous shape with C elements.
int check_channel_param(const TensorInfo &ref, const TensorInfo &x, int64_t C) {
    if (x.t == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: %s descriptor is null", x.name);
    RWKV7_TRY(check_present(x, x.t->ndim));
    if (num_elements(x.t) != C)
        return fail(RWKV7_ERR_SHAPE_MISMATCH, "ShapeMismatch: %s is %s, expected %lld elements", x.name,
                    shape_string(x.t->shape, x.t->ndim).c_str(), (long long)C);
    RWKV7_TRY(check_same_dtype({ref, x}));
    RWKV7_TRY(check_same_device({ref, x}));
    return check_contiguous(x);
}

int check_heads(int64_t C, int64_t num_heads, const rwkv7_tensor *ref) {
    if (num_heads <= 0 || C % num_heads != 0)
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: num_heads %lld does not divide %lld channels",
                    (long long)num_heads, (long long)C);
    if (ref->ndim == 4 && ref->shape[2] != num_heads)
        return fail(RWKV7_ERR_SHAPE_MISMATCH, "ShapeMismatch: tensor has %lld heads, num_heads is %lld",
                    (long long)ref->shape[2], (long long)num_heads);
    return RWKV7_OK;
}

}  // namespace

int rwkv7_fused_weight_prepare(const rwkv7_tensor *k_t, const rwkv7_tensor *lr_t, const rwkv7_tensor *wd_t,
                               const rwkv7_tensor *xi_t, const rwkv7_tensor *alpha_t,
                               const rwkv7_tensor *vp_t, const rwkv7_tensor *vf_t, const rwkv7_tensor *nu_t,
                               int64_t num_heads, rwkv7_tensor *w_t, rwkv7_tensor *kt_t, rwkv7_tensor *a_t,
                               rwkv7_tensor *b_t, rwkv7_tensor *v_t, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.weight_prepare");
    clear_error();
    const TensorInfo k{"key_precursor", k_t};
    RWKV7_TRY(check_sequence_tensor(k));
    RWKV7_TRY(check_axis_non_empty(k, 2));
    const int64_t C = channels_of(k_t);
    RWKV7_TRY(check_heads(C, num_heads, k_t));
    RWKV7_TRY(check_sequence_like(k, TensorInfo{"learning_rate_lora", lr_t}));
    RWKV7_TRY(check_sequence_like(k, TensorInfo{"weight_decay_lora", wd_t}));
    RWKV7_TRY(check_channel_param(k, TensorInfo{"key_removal", xi_t}, C));
    RWKV7_TRY(check_channel_param(k, TensorInfo{"key_replacement", alpha_t}, C));
    const int n_value = (vp_t != nullptr) + (vf_t != nullptr) + (nu_t != nullptr) + (v_t != nullptr);
    if (n_value != 0 && n_value != 4)
        return fail(RWKV7_ERR_NULL_POINTER,
                    "NullPointer: value_precursor, value_from_first_cell, value_residual_lora and value "
                    "must be all given or all null");
    if (n_value == 4) {
        RWKV7_TRY(check_sequence_like(k, TensorInfo{"value_precursor", vp_t}));
        RWKV7_TRY(check_sequence_like(k, TensorInfo{"value_from_first_cell", vf_t}));
        RWKV7_TRY(check_sequence_like(k, TensorInfo{"value_residual_lora", nu_t}));
        RWKV7_TRY(check_sequence_like(k, TensorInfo{"value", v_t}));
    }
    if (!float_dtype_supported(k_t->dtype))
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: weight_prepare computes F32 or BF16, got %s", dtype_name(k_t->dtype));
    RWKV7_TRY(check_sequence_like(k, TensorInfo{"weight_decay", w_t}));
    RWKV7_TRY(check_sequence_like(k, TensorInfo{"replacement_key", kt_t}));
    RWKV7_TRY(check_sequence_like(k, TensorInfo{"removal_key_normalized", a_t}));
    RWKV7_TRY(check_sequence_like(k, TensorInfo{"replacement", b_t}));
    WeightPrepareArgs p{};
    p.key_precursor = k_t->data; p.learning_rate_lora = lr_t->data; p.weight_decay_lora = wd_t->data;
    p.key_removal = xi_t->data; p.key_replacement = alpha_t->data;
    if (n_value == 4) {
        p.value_precursor = vp_t->data; p.value_from_first_cell = vf_t->data; p.value_residual_lora = nu_t->data;
        p.value = v_t->data;
    }
    p.weight_decay = w_t->data; p.replacement_key = kt_t->data; p.removal_key_normalized = a_t->data;
    p.replacement = b_t->data;
    p.H = num_heads; p.N = C / num_heads; p.rows = k.dim(0) * k.dim(1) * num_heads;
    p.bf16 = k_t->dtype == RWKV7_BF16;
    if (p.rows == 0) return RWKV7_OK;
    DeviceGuard guard(k_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(k_t->device, &p.num_sms));
    if (int e = launch_weight_prepare(p, (cudaStream_t)stream)) return cuda_fail("weight_prepare launch", e);
    return RWKV7_OK;
}

int rwkv7_fused_gated_readout(const rwkv7_tensor *y_t, const rwkv7_tensor *r_t, const rwkv7_tensor *kt_t,
                              const rwkv7_tensor *v_t, const rwkv7_tensor *gate_t, const rwkv7_tensor *gamma_t,
                              const rwkv7_tensor *beta_t, const rwkv7_tensor *bonus_t, double epsilon,
                              int64_t num_heads, rwkv7_tensor *out_t, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.gated_readout");
    clear_error();
    const TensorInfo y{"wkv7_output", y_t};
    RWKV7_TRY(check_sequence_tensor(y));
    RWKV7_TRY(check_axis_non_empty(y, 2));
    const int64_t C = channels_of(y_t);
    RWKV7_TRY(check_heads(C, num_heads, y_t));
    RWKV7_TRY(check_sequence_like(y, TensorInfo{"receptance", r_t}));
    RWKV7_TRY(check_sequence_like(y, TensorInfo{"replacement_key", kt_t}));
    RWKV7_TRY(check_sequence_like(y, TensorInfo{"value", v_t}));
    RWKV7_TRY(check_sequence_like(y, TensorInfo{"gate", gate_t}));
    RWKV7_TRY(check_channel_param(y, TensorInfo{"group_norm_gamma", gamma_t}, C));
    RWKV7_TRY(check_channel_param(y, TensorInfo{"group_norm_beta", beta_t}, C));
    RWKV7_TRY(check_channel_param(y, TensorInfo{"receptance_key_bonus", bonus_t}, C));
    if (!(epsilon >= 0.0))
        return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: epsilon must be non-negative, got %g", epsilon);
    if (!float_dtype_supported(y_t->dtype))
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: gated_readout computes F32 or BF16, got %s", dtype_name(y_t->dtype));
    RWKV7_TRY(check_sequence_like(y, TensorInfo{"output", out_t}));
    GatedReadoutArgs p{};
    p.wkv7_output = y_t->data; p.receptance = r_t->data; p.replacement_key = kt_t->data; p.value = v_t->data;
    p.gate = gate_t->data; p.gamma = gamma_t->data; p.beta = beta_t->data; p.bonus = bonus_t->data;
    p.output = out_t->data; p.epsilon = (float)epsilon;
    p.H = num_heads; p.N = C / num_heads; p.rows = y.dim(0) * y.dim(1) * num_heads;
    p.bf16 = y_t->dtype == RWKV7_BF16;
    if (p.rows == 0) return RWKV7_OK;
    DeviceGuard guard(y_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(y_t->device, &p.num_sms));
    if (int e = launch_gated_readout(p, (cudaStream_t)stream)) return cuda_fail("gated_readout launch", e);
    return RWKV7_OK;
}

size_t rwkv7_channel_mixer_workspace_bytes(int64_t B, int64_t T, int64_t C, int64_t F) {
    if (B <= 0 || T <= 0) return 0;
    return channel_mixer_workspace_bytes(B * T, C, F);
}

int rwkv7_fused_channel_mixer(const rwkv7_tensor *x_t, const rwkv7_tensor *scale_t, const rwkv7_tensor *kw_t,
                              const rwkv7_tensor *vw_t, rwkv7_tensor *out_t, void *workspace,
                              size_t workspace_bytes, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.infer.model.channel_mixer");
    clear_error();
    const TensorInfo x{"embedded_context", x_t}, scale{"key_scale", scale_t}, kw{"key_weight", kw_t},
        vw{"value_weight", vw_t};
    RWKV7_TRY(check_present(x, 3));
    RWKV7_TRY(check_present(scale, 1));
    RWKV7_TRY(check_present(kw, 2));
    RWKV7_TRY(check_present(vw, 2));
    // ChannelMixerForwardInputs::check (channel_mixer/io.rs:40-62)
    RWKV7_TRY(check_axis_non_empty(x, 2));
    RWKV7_TRY(check_axis_non_empty(kw, 0));
    RWKV7_TRY(check_shape(scale, {x.dim(2)}));
    RWKV7_TRY(check_axes_equal({{x, 2}, {kw, 1}, {vw, 0}}));
    RWKV7_TRY(check_axes_equal({{kw, 0}, {vw, 1}}));
    RWKV7_TRY(check_shape(vw, {x.dim(2), kw.dim(0)}));
    RWKV7_TRY(check_same_dtype({x, scale, kw, vw}));
    RWKV7_TRY(check_same_device({x, scale, kw, vw}));
    RWKV7_TRY(check_contiguous(x));
    RWKV7_TRY(check_contiguous(scale));
    RWKV7_TRY(check_contiguous(kw));
    RWKV7_TRY(check_contiguous(vw));
    if (x_t->dtype != RWKV7_BF16)
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: channel_mixer computes BF16 tensors, got %s", dtype_name(x_t->dtype));
    RWKV7_TRY(check_output_like(x, TensorInfo{"output", out_t}));
    ChannelMixerArgs p{};
    p.x = x_t->data; p.key_scale = scale_t->data; p.key_weight = kw_t->data; p.value_weight = vw_t->data;
    p.out = out_t->data;
    p.B = x.dim(0); p.T = x.dim(1); p.C = x.dim(2); p.F = kw.dim(0);
    if (p.C % 8 != 0 || p.F % 8 != 0)
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: channel_mixer needs C and F to be multiples of 8, got %lld and %lld",
                    (long long)p.C, (long long)p.F);
    if (p.B == 0 || p.T == 0) return RWKV7_OK;   // channel_mixer/mod.rs:102-104: an empty context gives an empty output
    for (const void *ptr : {p.x, p.key_scale, p.key_weight, p.value_weight, (const void *)p.out, (const void *)workspace})
        if (reinterpret_cast<uintptr_t>(ptr) & 15u)
            return fail(RWKV7_ERR_BAD_ARGUMENT, "BadArgument: channel_mixer tensors and workspace must be 16-byte aligned");
    const size_t need = channel_mixer_workspace_bytes(p.B * p.T, p.C, p.F);
    if (workspace == nullptr) return fail(RWKV7_ERR_NULL_POINTER, "NullPointer: channel_mixer needs a workspace of %zu bytes", need);
    if (workspace_bytes < need)
        return fail(RWKV7_ERR_WORKSPACE_TOO_SMALL, "WorkspaceTooSmall: channel_mixer needs %zu workspace bytes, got %zu", need,
                    workspace_bytes);
    DeviceGuard guard(x_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(x_t->device, &p.num_sms));
    if (int e = device_status_ptr(x_t->device, &p.status)) return cuda_fail("device status word", e);
    if (int e = launch_channel_mixer(p, workspace, workspace_bytes, (cudaStream_t)stream))
        return cuda_fail("channel_mixer launch", e);
    return RWKV7_OK;
}

size_t rwkv7_lm_head_ce_workspace_bytes(int64_t R, int64_t C, int64_t V_shard) {
    return lm_head_ce_workspace_bytes(R, C, V_shard);
}

int rwkv7_fused_lm_head_ce_partial(const rwkv7_tensor *x_t, const rwkv7_tensor *w_t,
                                   const rwkv7_tensor *targets_t, int64_t vocab_offset,
                                   rwkv7_tensor *partials_t, void *workspace, size_t workspace_bytes,
                                   rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.train.lm_head_ce.partial");
    clear_error();
    const TensorInfo x{"x", x_t}, w{"weight_shard", w_t}, tg{"targets", targets_t},
        pt{"partials", partials_t};
    RWKV7_TRY(check_present(x, 2));
    RWKV7_TRY(check_present(w, 2));
    RWKV7_TRY(check_present(tg, 1));
    RWKV7_TRY(check_present(pt, 2));
    RWKV7_TRY(check_axis_non_empty(x, 1));
    RWKV7_TRY(check_axis_non_empty(w, 0));
    RWKV7_TRY(check_axes_equal({{x, 1}, {w, 1}}));
    RWKV7_TRY(check_shape(tg, {x.dim(0)}));
    RWKV7_TRY(check_shape(pt, {x.dim(0), 3}));
    RWKV7_TRY(check_same_dtype({x, w}));
    RWKV7_TRY(check_same_device({x, w, tg, pt}));
    RWKV7_TRY(check_contiguous(x));
    RWKV7_TRY(check_contiguous(w));
    RWKV7_TRY(check_contiguous(tg));
    RWKV7_TRY(check_contiguous(pt));
    if (x_t->dtype != RWKV7_BF16)
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: lm_head_ce computes BF16 inputs, got %s", dtype_name(x_t->dtype));
    if (targets_t->dtype != RWKV7_I32 && targets_t->dtype != RWKV7_I64)
        return fail(RWKV7_ERR_DTYPE_MISMATCH, "DTypeMismatch: targets must be I32 or I64, got %s", dtype_name(targets_t->dtype));
    if (partials_t->dtype != RWKV7_F32)
        return fail(RWKV7_ERR_DTYPE_MISMATCH, "DTypeMismatch: partials must be F32, got %s", dtype_name(partials_t->dtype));
    LmHeadArgs p{};
    p.x = x_t->data; p.w = w_t->data; p.targets = targets_t->data; p.targets_dtype = targets_t->dtype;
    p.vocab_offset = vocab_offset; p.partials = static_cast<float *>(partials_t->data);
    p.R = x.dim(0); p.C = x.dim(1); p.V = w.dim(0); p.device = x_t->device;
    if (p.R == 0) return RWKV7_OK;
    if (p.C % 64 != 0)
        return fail(RWKV7_ERR_UNSUPPORTED, "Unsupported: lm_head_ce needs C %% 64 == 0 (got C=%lld)", (long long)p.C);
    const size_t need = lm_head_ce_workspace_bytes(p.R, p.C, p.V);
    if (need > 0 && (workspace == nullptr || workspace_bytes < need))
        return fail(RWKV7_ERR_WORKSPACE_TOO_SMALL, "WorkspaceTooSmall: lm_head_ce needs %zu workspace bytes, got %zu",
                    need, workspace == nullptr ? (size_t)0 : workspace_bytes);
    DeviceGuard guard(p.device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    RWKV7_TRY(num_sms(p.device, &p.num_sms));
    if (int e = device_status_ptr(p.device, &p.status)) return cuda_fail("device status word", e);
    if (int e = launch_lm_head_ce_partial(p, workspace, workspace_bytes, (cudaStream_t)stream))
        return cuda_fail("lm_head_ce launch", e);
    return RWKV7_OK;
}

int rwkv7_lm_head_ce_finalize(const rwkv7_tensor *partials_all_t, const rwkv7_tensor *targets_t,
                              rwkv7_tensor *lse_t, rwkv7_tensor *loss_t, rwkv7_stream stream) {
    RWKV7_TRACE("rwkv.train.lm_head_ce.finalize");
    clear_error();
    const TensorInfo pa{"partials_all", partials_all_t}, tg{"targets", targets_t}, lse{"lse", lse_t},
        loss{"loss", loss_t};
    RWKV7_TRY(check_present(pa, 3));
    RWKV7_TRY(check_present(tg, 1));
    RWKV7_TRY(check_present(lse, 1));
    RWKV7_TRY(check_present(loss, 1));
    RWKV7_TRY(check_axis_non_empty(pa, 0));
    const int64_t R = pa.dim(1);
    RWKV7_TRY(check_shape(pa, {pa.dim(0), R, 3}));
    RWKV7_TRY(check_shape(tg, {R}));
    RWKV7_TRY(check_shape(lse, {R}));
    RWKV7_TRY(check_shape(loss, {R}));
    RWKV7_TRY(check_same_dtype({pa, lse, loss}));
    RWKV7_TRY(check_same_device({pa, tg, lse, loss}));
    RWKV7_TRY(check_contiguous(pa));
    RWKV7_TRY(check_contiguous(tg));
    RWKV7_TRY(check_contiguous(lse));
    RWKV7_TRY(check_contiguous(loss));
    if (partials_all_t->dtype != RWKV7_F32)
        return fail(RWKV7_ERR_DTYPE_MISMATCH, "DTypeMismatch: partials_all must be F32, got %s", dtype_name(partials_all_t->dtype));
    if (targets_t->dtype != RWKV7_I32 && targets_t->dtype != RWKV7_I64)
        return fail(RWKV7_ERR_DTYPE_MISMATCH, "DTypeMismatch: targets must be I32 or I64, got %s", dtype_name(targets_t->dtype));
    if (R == 0) return RWKV7_OK;
    DeviceGuard guard(partials_all_t->device);
    if (guard.error() != cudaSuccess) return cuda_fail("cudaSetDevice", (int)guard.error());
    if (int e = launch_lm_head_ce_finalize(static_cast<const float *>(partials_all_t->data), (int)pa.dim(0),
                                           targets_t->data, targets_t->dtype, static_cast<float *>(lse_t->data),
                                           static_cast<float *>(loss_t->data), R, (cudaStream_t)stream))
        return cuda_fail("lm_head_ce finalize launch", e);
    return RWKV7_OK;
}

}  // extern "C"
