// Placeholder translation unit: replaced by the tcgen05 LM-head kernel.
#include "kernels.h"
namespace rwkv7 {
size_t lm_head_ce_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }
int launch_lm_head_ce_partial(const LmHeadArgs &, void *, size_t, cudaStream_t) { return (int)cudaErrorNotSupported; }
int launch_lm_head_ce_finalize(const float *, int, const void *, int, float *, float *, int64_t, cudaStream_t) { return (int)cudaErrorNotSupported; }
}
