// Channel mixer for sm_100a: token-shift mix -> key projection -> relu^2 -> value
// projection, the two projections on the tcgen05 tensor cores with the activation
// applied in the first one's epilogue.
//
// Replaces ChannelMixerBackend::fused_channel_mixer
// (crates/rwkv-nn/src/kernels/train/channel_mixer/forward.rs:52-88; semantic definition
// channel_mixer_reference, mod.rs:96-128; elementwise kernels kernel.rs:4-45):
//     shifted[b,t,:] = x[b,t-1,:] (zero at t == 0)
//     key_input = x + (shifted - x) * key_scale
//     hidden    = relu(key_input . key_weight^T)^2        key_weight   [F, C]
//     output    = hidden . value_weight^T                 value_weight [C, F]
// The reference runs two elementwise kernels around two library matmuls; here the
// hidden activation never exists unactivated: the first GEMM's epilogue squares the
// rectified accumulator before it is rounded to bf16.
//
// GEMM kernel: out[M,N] = act(A[M,K] . B[N,K]^T), A and B row-major bf16 (both "K-major"),
// fp32 accumulation in TMEM, bf16 output.  Persistent CTAs, one per SM; a tile is 128 x 256;
// tiles are walked with the column block fastest, so that the CTAs running together share a
// few row blocks of A and sweep all of B, and both stay in L2.  Warp roles as in the LM-head
// kernel: warp 0 requests A and B tiles by TMA (128-byte swizzle, K slices of 64, 4-stage
// ring), warp 1 issues tcgen05.mma (M=128, N=256, kind::f16) into one of two 256-column
// TMEM buffers, warps 2..5 read the finished buffer back (thread = row, 32 columns at a
// time), apply the activation and store 64 contiguous bytes per thread while the next tile
// multiplies.  Every mbarrier wait is bounded.
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

struct GemmMaps {
    CUtensorMap a;  // [M, K] bf16, box 128 x 64
    CUtensorMap b;  // [N, K] bf16, box 256 x 64
};

enum { kEpiNone = 0, kEpiReluSquare = 1 };

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_bf16_kernel(const __grid_constant__ GemmMaps maps, __nv_bfloat16 *__restrict__ out, int64_t M, int N,
                    int K, int n_tiles, int total_tiles, int *status) {
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
    const int ksteps = (K + kBK - 1) / kBK;   // the K tail is zero-filled by TMA

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
        mbar_fence_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b);
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
            for (int tile = blockIdx.x; tile < total_tiles && !timed_out; tile += gridDim.x) {
                const int nt = tile % n_tiles, mt = tile / n_tiles;
                for (int ks = 0; ks < ksteps; ++ks, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1)) { timed_out = true; break; }
                    unsigned char *a = smem + s * kStageBytes, *b = a + kABytes;
                    mbar_expect_tx(&full[s], kStageBytes);
                    tma_load_2d(a, &maps.a, ks * kBK, mt * kBM, &full[s]);
                    tma_load_2d(b, &maps.b, ks * kBK, nt * kBN, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kFmtBF16, kBM, kBN, false, false);
            uint32_t it = 0, local = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !timed_out; tile += gridDim.x, ++local) {
                const uint32_t buf = local & 1, bph = (local >> 1) & 1;
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
        uint32_t local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !timed_out; tile += gridDim.x, ++local) {
            const int nt = tile % n_tiles, mt = tile / n_tiles;
            const uint32_t buf = local & 1, bph = (local >> 1) & 1;
            if (!mbar_wait(&tmem_full[buf], bph)) { timed_out = true; break; }
            tc_fence_after();
            const int64_t row = (int64_t)mt * kBM + quarter * 32 + lane;
            __nv_bfloat16 *orow = out + row * N + (int64_t)nt * kBN;
#pragma unroll 1
            for (int ch = 0; ch < kBN / 32; ++ch) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * kBN + ch * 32, v);
                tmem_ld_wait();
                const int c0 = nt * kBN + ch * 32;
                if (row >= M || c0 >= N) continue;            // padding rows / columns of edge tiles
                const int nvec = min(32, N - c0) / 8;          // N is a multiple of 8
                uint4 pk[4];
                unsigned *pw = &pk[0].x;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float x0 = __uint_as_float(v[e]), x1 = __uint_as_float(v[e + 1]);
                    if constexpr (EPI == kEpiReluSquare) {
                        x0 = fmaxf(x0, 0.f); x0 *= x0;
                        x1 = fmaxf(x1, 0.f); x1 *= x1;
                    }
                    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
                    pw[e >> 1] = *reinterpret_cast<const unsigned *>(&h);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (q < nvec) *reinterpret_cast<uint4 *>(orow + ch * 32 + q * 8) = pk[q];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
    }
    if (timed_out) atomicExch(status, (int)kDevTimeout);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// key_input = x + (shifted - x) * key_scale, shifted = previous token (zero at t == 0)
// (channel_mixer/kernel.rs:4-25).  A CTA owns 16 consecutive token rows, a thread one
// 16-byte channel vector; the previous row is carried in registers.
constexpr int kMixRows = 16;
__global__ void __launch_bounds__(256)
channel_mixer_mix_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ scale,
                         __nv_bfloat16 *__restrict__ out, int64_t rows, int64_t Tlen, int64_t C) {
    const int64_t CV = C / 8;
    const int64_t row_begin = (int64_t)blockIdx.x * kMixRows;
    const int64_t row_end = row_begin + kMixRows < rows ? row_begin + kMixRows : rows;
    auto unpack = [](const uint4 &u, float (&f)[8]) {
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    };
    for (int64_t cv = threadIdx.x; cv < CV; cv += blockDim.x) {
        const int64_t c = cv * 8;
        float mu[8], prev[8], cur[8];
        unpack(*reinterpret_cast<const uint4 *>(scale + c), mu);
        if (row_begin % Tlen == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) prev[e] = 0.f;
        } else {
            unpack(*reinterpret_cast<const uint4 *>(x + (row_begin - 1) * C + c), prev);
        }
#pragma unroll 4
        for (int64_t row = row_begin; row < row_end; ++row) {
            unpack(__ldcs(reinterpret_cast<const uint4 *>(x + row * C + c)), cur);
            if (row % Tlen == 0) {
#pragma unroll
                for (int e = 0; e < 8; ++e) prev[e] = 0.f;   // first token of a sequence
            }
            uint4 o;
            unsigned *ow = &o.x;
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(fmaf(prev[e] - cur[e], mu[e], cur[e]),
                                                               fmaf(prev[e + 1] - cur[e + 1], mu[e + 1], cur[e + 1]));
                ow[e >> 1] = *reinterpret_cast<const unsigned *>(&h);
            }
            *reinterpret_cast<uint4 *>(out + row * C + c) = o;
#pragma unroll
            for (int e = 0; e < 8; ++e) prev[e] = cur[e];
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn gemm_encode_fn() {
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

int encode_rows_by_k(EncodeTiledFn encode, CUtensorMap *map, const void *base, int64_t rows, int64_t K, int box_rows) {
    const cuuint32_t estr[2] = {1, 1};
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? 0
               : (int)cudaErrorInvalidValue;
}

// out[M,N] = act(A[M,K] . B[N,K]^T); K and N multiples of 8, all pointers 16-byte aligned.
int launch_gemm(const void *a, const void *b, void *out, int64_t M, int64_t N, int64_t K, int epi, int num_sms,
                int *status, cudaStream_t stream) {
    EncodeTiledFn encode = gemm_encode_fn();
    if (encode == nullptr) return (int)cudaErrorNotSupported;
    GemmMaps maps;
    if (int e = encode_rows_by_k(encode, &maps.a, a, M, K, kBM)) return e;
    if (int e = encode_rows_by_k(encode, &maps.b, b, N, K, kBN)) return e;
    const int m_tiles = (int)((M + kBM - 1) / kBM), n_tiles = (int)((N + kBN - 1) / kBN);
    const int total = m_tiles * n_tiles;
    const unsigned grid = (unsigned)(total < num_sms ? total : num_sms);
    cudaError_t e;
    if (epi == kEpiReluSquare) {
        e = cudaFuncSetAttribute(gemm_tn_bf16_kernel<kEpiReluSquare>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        gemm_tn_bf16_kernel<kEpiReluSquare><<<grid, kThreads, kSmemBytes, stream>>>(
            maps, (__nv_bfloat16 *)out, M, (int)N, (int)K, n_tiles, total, status);
    } else {
        e = cudaFuncSetAttribute(gemm_tn_bf16_kernel<kEpiNone>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        gemm_tn_bf16_kernel<kEpiNone><<<grid, kThreads, kSmemBytes, stream>>>(
            maps, (__nv_bfloat16 *)out, M, (int)N, (int)K, n_tiles, total, status);
    }
    count_launch();
    return (int)cudaGetLastError();
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

size_t channel_mixer_workspace_bytes(int64_t rows, int64_t C, int64_t F) {
    if (rows <= 0 || C <= 0 || F <= 0) return 0;
    return align256((size_t)rows * C * 2) + align256((size_t)rows * F * 2);   // key_input, hidden
}

int launch_channel_mixer(const ChannelMixerArgs &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    const int64_t rows = p.B * p.T;
    if (rows == 0) return 0;
    if (workspace_bytes < channel_mixer_workspace_bytes(rows, p.C, p.F)) return (int)cudaErrorInvalidValue;
    __nv_bfloat16 *key_input = static_cast<__nv_bfloat16 *>(workspace);
    __nv_bfloat16 *hidden = reinterpret_cast<__nv_bfloat16 *>(static_cast<unsigned char *>(workspace) +
                                                              align256((size_t)rows * p.C * 2));
    int threads = 32;
    while (threads < 256 && threads < p.C / 8) threads <<= 1;
    channel_mixer_mix_kernel<<<(unsigned)((rows + kMixRows - 1) / kMixRows), threads, 0, stream>>>(
        (const __nv_bfloat16 *)p.x, (const __nv_bfloat16 *)p.key_scale, key_input, rows, p.T, p.C);
    count_launch();
    if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return (int)e;
    if (int e = launch_gemm(key_input, p.key_weight, hidden, rows, p.F, p.C, kEpiReluSquare, p.num_sms, p.status, stream))
        return e;
    return launch_gemm(hidden, p.value_weight, p.out, rows, p.C, p.F, kEpiNone, p.num_sms, p.status, stream);
}

}  // namespace rwkv7
