// Placeholder translation unit: replaced by the tcgen05 chunked prefill kernel.
#include "kernels.h"
namespace rwkv7 {
size_t wkv7_chunked_workspace_bytes(int64_t, int64_t, int64_t, int64_t) { return 0; }
bool wkv7_chunked_supported(const Wkv7Args &) { return false; }
int launch_wkv7_chunked(const Wkv7Args &, void *, size_t, cudaStream_t) { return (int)cudaErrorNotSupported; }
size_t lm_head_ce_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }
int launch_lm_head_ce_partial(const LmHeadArgs &, void *, size_t, cudaStream_t) { return (int)cudaErrorNotSupported; }
int launch_lm_head_ce_finalize(const float *, int, const void *, int, float *, float *, int64_t, cudaStream_t) { return (int)cudaErrorNotSupported; }
}
