// Fused LM-head cross entropy for sm_100a: z = x W^T on the tcgen05 tensor cores
// with an online log-sum-exp epilogue, so the [R, V] logits are never written.
//
// The reference reserves this operator but ships no implementation
// (crates/rwkv-nn/src/kernels/train/lm_head_l2wrap_ce/mod.rs is empty; the config
// switch is crates/rwkv-config/src/raw/train.rs:59-60), so the definition is the
// one stated in rwkv7_b200.h: per row the triple (max_v z_v, sum_v exp(z_v - max),
// z_target) over a vocabulary shard, then a combine over shards.
//
// One CTA owns a block of 128 rows and a contiguous range of 256-wide vocabulary
// tiles.  Warp roles: warp 0 requests the x and W tiles (TMA, 128-byte swizzle, K
// slices of 64 bf16, 4-stage ring); warp 1 issues the UMMAs (M=128, N=256, bf16 in,
// fp32 accumulators, two 256-column TMEM buffers); warps 2..5 are the epilogue:
// thread = row, it reads its accumulator row 32 columns at a time and keeps the
// running (max, sum-exp, target logit) in registers while the next tile is being
// multiplied.  CTAs that run together walk the vocabulary in the same order, so a
// W tile is fetched from HBM once per wave and served to the others from L2.
// Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"
#include "rwkv7_b200.h"
#include "sm100_umma.cuh"

namespace rwkv7 {
namespace {

using namespace sm100;

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4;
constexpr int kThreads = 192;  // TMA warp, MMA warp, four epilogue warps
constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = kBN * kBK * 2;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*alignment slack*/;
constexpr float kLog2e = 1.4426950408889634f;

struct LmMaps {
    CUtensorMap x;  // [R, C] bf16, box 128 x 64
    CUtensorMap w;  // [V, C] bf16, box 256 x 64
};

__device__ __forceinline__ int64_t load_target(const void *t, int dtype, int64_t row) {
    return dtype == RWKV7_I64 ? reinterpret_cast<const int64_t *>(t)[row]
                              : (int64_t) reinterpret_cast<const int32_t *>(t)[row];
}

__global__ void __launch_bounds__(kThreads, 1)
lm_head_ce_kernel(const __grid_constant__ LmMaps maps, const void *__restrict__ targets, int targets_dtype,
                  int64_t vocab_offset, float *__restrict__ out /* [splits][R][3] */, int64_t R, int C, int V,
                  int row_blocks, int tiles_per_split, int *status) {
    extern __shared__ __align__(1024) unsigned char smem[];   // swizzled TMA tiles need 1024-byte alignment
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(status, (int)kDevInternal);
        return;
    }
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
    uint64_t *empty = full + kStages;
    uint64_t *tmem_full = empty + kStages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // consecutive CTAs share a vocabulary split and differ in the row block
    const int rb = blockIdx.x % row_blocks, split = blockIdx.x / row_blocks;
    const int total_tiles = (V + kBN - 1) / kBN;
    const int tile0 = split * tiles_per_split;
    const int ntiles = min(tiles_per_split, total_tiles - tile0);
    const int ksteps = C / kBK;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
        mbar_fence_init();
        tma_prefetch_desc(&maps.x);
        tma_prefetch_desc(&maps.w);
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = 0; t < ntiles && !timed_out; ++t) {
                for (int ks = 0; ks < ksteps; ++ks, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1)) { timed_out = true; break; }
                    unsigned char *a = smem + s * kStageBytes, *b = a + kABytes;
                    mbar_expect_tx(&full[s], kStageBytes);
                    tma_load_2d(a, &maps.x, ks * kBK, rb * kBM, &full[s]);
                    tma_load_2d(b, &maps.w, ks * kBK, (tile0 + t) * kBN, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kFmtBF16, kBM, kBN, false, false);
            uint32_t it = 0;
            for (int t = 0; t < ntiles && !timed_out; ++t) {
                const uint32_t buf = t & 1, bph = (t >> 1) & 1;
                if (!mbar_wait(&tmem_empty[buf], bph ^ 1)) { timed_out = true; break; }
                tc_fence_after();
                for (int ks = 0; ks < ksteps; ++ks, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                    if (!mbar_wait(&full[s], ph)) { timed_out = true; break; }
                    tc_fence_after();
                    const uint32_t a = smem_u32(smem + s * kStageBytes), b = a + kABytes;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        umma_f16(tmem + buf * kBN, make_smem_desc(a + k * 32, 16, 1024),
                                 make_smem_desc(b + k * 32, 16, 1024), idesc, ks > 0 || k > 0);
                    umma_commit(&empty[s]);   // the stage may be refilled once these MMAs have read it
                }
                if (timed_out) break;
                umma_commit(&tmem_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row_local = quarter * 32 + lane;
        const int64_t row = (int64_t)rb * kBM + row_local;
        const bool row_ok = row < R;
        int64_t tgt = -1;
        if (row_ok) tgt = load_target(targets, targets_dtype, row);
        const int64_t tgt_local = (tgt >= 0) ? tgt - vocab_offset : -1;   // column inside this shard
        float m = -INFINITY, ssum = 0.f, zt = 0.f;
        for (int t = 0; t < ntiles && !timed_out; ++t) {
            const uint32_t buf = t & 1, bph = (t >> 1) & 1;
            if (!mbar_wait(&tmem_full[buf], bph)) { timed_out = true; break; }
            tc_fence_after();
            const int col0 = (tile0 + t) * kBN;
#pragma unroll 1
            for (int ch = 0; ch < kBN / 32; ++ch) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * kBN + ch * 32, v);
                tmem_ld_wait();
                const int c0 = col0 + ch * 32;
                if (c0 >= V) continue;                       // padding columns of the last tile
                const int ncol = min(32, V - c0);
                float cm = -INFINITY;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    if (e >= ncol) v[e] = __float_as_uint(-INFINITY);
                    cm = fmaxf(cm, __uint_as_float(v[e]));
                }
                const float m_new = fmaxf(m, cm);
                const float mb = m_new * kLog2e;
                ssum *= exp2f(m * kLog2e - mb);               // exp2(-inf) = 0 on the first chunk
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    acc0 += exp2f(fmaf(__uint_as_float(v[e]), kLog2e, -mb));
                    acc1 += exp2f(fmaf(__uint_as_float(v[e + 1]), kLog2e, -mb));
                }
                ssum += acc0 + acc1;
                m = m_new;
                if (tgt_local >= c0 && tgt_local < c0 + ncol) {
                    const int off = (int)(tgt_local - c0);
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (e == off) zt = __uint_as_float(v[e]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
        if (row_ok && !timed_out) {
            float *o = out + ((size_t)split * R + row) * 3;
            o[0] = m;
            o[1] = ssum;
            o[2] = zt;
        }
    }
    if (timed_out) atomicExch(status, (int)kDevTimeout);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// Combines `nparts` partial triples per row: out[row] = (M, sum_g s_g exp(m_g - M), sum_g zt_g).
__global__ void lm_head_combine_kernel(const float *__restrict__ parts, int nparts, float *__restrict__ out,
                                       int64_t R) {
    const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= R) return;
    float M = -INFINITY;
    for (int g = 0; g < nparts; ++g) M = fmaxf(M, parts[((size_t)g * R + row) * 3]);
    float s = 0.f, zt = 0.f;
    for (int g = 0; g < nparts; ++g) {
        const float *p = parts + ((size_t)g * R + row) * 3;
        if (p[0] > -INFINITY) s += p[1] * expf(p[0] - M);
        zt += p[2];
    }
    out[row * 3 + 0] = M;
    out[row * 3 + 1] = s;
    out[row * 3 + 2] = zt;
}

__global__ void lm_head_finalize_kernel(const float *__restrict__ parts, int nparts, const void *__restrict__ targets,
                                        int targets_dtype, float *__restrict__ lse, float *__restrict__ loss,
                                        int64_t R) {
    const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= R) return;
    float M = -INFINITY;
    for (int g = 0; g < nparts; ++g) M = fmaxf(M, parts[((size_t)g * R + row) * 3]);
    float s = 0.f, zt = 0.f;
    for (int g = 0; g < nparts; ++g) {
        const float *p = parts + ((size_t)g * R + row) * 3;
        if (p[0] > -INFINITY) s += p[1] * expf(p[0] - M);
        zt += p[2];
    }
    const float l = M + logf(s);
    lse[row] = l;
    loss[row] = load_target(targets, targets_dtype, row) >= 0 ? l - zt : 0.f;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn lm_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Vocabulary splits per row block.  A CTA takes one block of 128 rows and a run of column tiles, one CTA fits an
// SM, so a launch runs in waves of `num_sms` CTAs and its time goes with waves x (tiles per CTA): the split count
// that minimises that product is taken (half a tile is charged per CTA for filling its pipeline, which favours fewer
// splits on a tie).  Example, 148 SMs, 256 row blocks x 32 column tiles: one or two splits take 2 x 32 = 4 x 16 = 64
// tile times, four splits 7 x 8 = 56 (the ideal is 55.4): 1140 -> 1195 TFLOP/s on that shape.  (Persistent CTAs that
// walk the work items themselves measured no better: 1167.)
constexpr int kMaxSplits = 16;
void plan(int64_t R, int64_t V, int num_sms, int *row_blocks, int *splits, int *tiles_per_split) {
    const int rbs = (int)((R + kBM - 1) / kBM);
    const int tiles = (int)((V + kBN - 1) / kBN);
    const int sms = num_sms > 0 ? num_sms : 1;
    int best_sp = 1, best_tps = tiles;
    double best_cost = 0.0;
    for (int want = 1; want <= kMaxSplits && want <= tiles; ++want) {
        const int tps = (tiles + want - 1) / want;
        const int sp = (tiles + tps - 1) / tps;
        const long long ctas = (long long)rbs * sp;
        const long long waves = (ctas + sms - 1) / sms;
        const double cost = (double)waves * (tps + 0.5);
        if (want == 1 || cost < best_cost - 1e-9) {
            best_cost = cost;
            best_sp = sp;
            best_tps = tps;
        }
    }
    *row_blocks = rbs;
    *splits = best_sp;
    *tiles_per_split = best_tps;
}

}  // namespace

size_t lm_head_ce_workspace_bytes(int64_t R, int64_t C, int64_t V) {
    (void)C;
    // Upper bound for any device: one triple per row per vocabulary split, at most kMaxSplits of them.
    const int64_t tiles = (V + kBN - 1) / kBN;
    const int64_t sp = tiles < kMaxSplits ? tiles : kMaxSplits;
    return sp > 1 ? (size_t)sp * (size_t)R * 3 * sizeof(float) : 0;
}

int launch_lm_head_ce_partial(const LmHeadArgs &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    EncodeTiledFn encode = lm_encode_fn();
    if (encode == nullptr) return (int)cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(p.x) & 15u) || (reinterpret_cast<uintptr_t>(p.w) & 15u))
        return (int)cudaErrorMisalignedAddress;
    LmMaps maps;
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {(cuuint64_t)p.C, (cuuint64_t)p.R};
        const cuuint64_t strides[1] = {(cuuint64_t)p.C * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
        if (encode(&maps.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(p.x), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)p.C, (cuuint64_t)p.V};
        const cuuint64_t strides[1] = {(cuuint64_t)p.C * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBN};
        if (encode(&maps.w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(p.w), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    int row_blocks, splits, tps;
    plan(p.R, p.V, p.num_sms, &row_blocks, &splits, &tps);
    float *parts = splits == 1 ? p.partials : static_cast<float *>(workspace);
    if (splits > 1 && workspace_bytes < (size_t)splits * p.R * 3 * sizeof(float)) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(lm_head_ce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    lm_head_ce_kernel<<<(unsigned)(row_blocks * splits), kThreads, kSmemBytes, stream>>>(
        maps, p.targets, p.targets_dtype, p.vocab_offset, parts, p.R, (int)p.C, (int)p.V, row_blocks, tps, p.status);
    count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (splits > 1) {
        lm_head_combine_kernel<<<(unsigned)((p.R + 255) / 256), 256, 0, stream>>>(parts, splits, p.partials, p.R);
        count_launch();
        e = cudaGetLastError();
    }
    return (int)e;
}

int launch_lm_head_ce_finalize(const float *partials_all, int num_shards, const void *targets, int targets_dtype,
                               float *lse, float *loss, int64_t R, cudaStream_t stream) {
    lm_head_finalize_kernel<<<(unsigned)((R + 255) / 256), 256, 0, stream>>>(partials_all, num_shards, targets,
                                                                            targets_dtype, lse, loss, R);
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace rwkv7
