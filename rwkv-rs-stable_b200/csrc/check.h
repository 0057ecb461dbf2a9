// Host-side input contracts of the C ABI.  Mirrors the reference's
// crates/rwkv-nn/src/kernels/check.rs (KernelInputsError :34-73 and the check_*
// helpers :91-217): same checks, same order at each call site, same message text.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <string>
#include <vector>

#include "rwkv7_b200.h"

namespace rwkv7 {

// Records `status` with a printf-formatted message for rwkv7_last_error_message().
int fail(int status, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();
const char *last_error();

struct TensorInfo {
    const char *name;
    const rwkv7_tensor *t;
    int64_t dim(int axis) const { return t->shape[axis]; }
};

std::string shape_string(const int64_t *shape, int ndim);
const char *dtype_name(int32_t dtype);
size_t dtype_size(int32_t dtype);
int64_t num_elements(const rwkv7_tensor *t);

// Non-null descriptor, sane ndim; data may be null only for zero-element tensors.
int check_present(const TensorInfo &x, int ndim);
// check.rs:166-178
int check_axis_non_empty(const TensorInfo &x, int axis);
// check.rs:115-138: every listed (tensor, axis) must equal the first.
int check_axes_equal(const std::vector<std::pair<TensorInfo, int>> &axes);
// check.rs:140-164
int check_shape(const TensorInfo &x, const std::vector<int64_t> &expected);
// check.rs:180-200 (expected = the first tensor's shape)
int check_same_shape(const std::vector<TensorInfo> &xs);
// check.rs:202-222
int check_same_dtype(const std::vector<TensorInfo> &xs);
// check.rs:224-244
int check_same_device(const std::vector<TensorInfo> &xs);
// The CubeBackend impls assert is_contiguous() (wkv7/mod.rs:56-76).
int check_contiguous(const TensorInfo &x);

}  // namespace rwkv7
