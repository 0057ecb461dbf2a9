// Optional instrumentation, both off in the product build.
//
// RWKV7_NVTX: every compute entry point of the C ABI opens an NVTX range for the duration of the call
// (host side: validation and the enqueueing of its kernels), named after the tracing span of the reference
// module that makes the call (`tracing::instrument(name = "rwkv.infer.model.*")`,
// crates/rwkv-nn/src/modules/time_mixer/mod.rs:153-156, modules/time_mixer/weight_prepare.rs:207,
// modules/time_mixer/gated_readout.rs:108, modules/channel_mixer/mod.rs:78, cells/causal.rs:72-75), with the
// operator appended, so that a timeline shows the same hierarchy as the reference's trace.
//
// RWKV7_CHECKED: device code verifies the indices it is about to use (rows of shared-memory tiles, rows of
// the output, slots of the workspace) and, when one is out of range, records kDevBadIndex in the device
// status word and skips the access instead of performing it.  Nothing traps; the host reads the word with
// rwkv7_read_device_status.
#pragma once

#ifdef RWKV7_NVTX
#include <nvtx3/nvToolsExt.h>
namespace rwkv7 {
struct TraceRange {
    explicit TraceRange(const char *name) { nvtxRangePushA(name); }
    ~TraceRange() { nvtxRangePop(); }
    TraceRange(const TraceRange &) = delete;
    TraceRange &operator=(const TraceRange &) = delete;
};
}  // namespace rwkv7
#define RWKV7_TRACE(name) ::rwkv7::TraceRange rwkv7_trace_range_(name)
#define RWKV7_TRACE_ENABLED 1
#else
#define RWKV7_TRACE(name) do {} while (0)
#define RWKV7_TRACE_ENABLED 0
#endif

#ifdef RWKV7_CHECKED
// True when `cond` holds; otherwise records the bad index and yields false so that the caller skips the access.
#define RWKV7_IN_RANGE(cond, status_ptr) ((cond) ? true : (atomicExch((status_ptr), (int)::rwkv7::kDevBadIndex), false))
#define RWKV7_CHECKED_ENABLED 1
#else
#define RWKV7_IN_RANGE(cond, status_ptr) (true)
#define RWKV7_CHECKED_ENABLED 0
#endif
