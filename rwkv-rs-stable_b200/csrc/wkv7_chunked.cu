// Chunked WKV7 prefill for sm_100a: tcgen05 (UMMA) tensor-core tiles with TMEM
// accumulators, inputs staged by TMA, fp32 state carried across chunks in
// registers.  N == 64, bf16 inputs/outputs, chunk length L = 64.
//
// Reference semantics: crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:179-242
// (token recurrence).  The reference kernel (kernel.rs:82-195) scans token by
// token; here one chunk of 64 tokens is advanced with dense products.
//
// Per (b,h), with Z = S^T (key index j rows, value index i columns), log-decay
// l_t = -exp(w_t), c_t = sum_{s<=t} l_s inside the chunk (c_{-1} = 0):
//     At = a_t * exp(c_{t-1})      Rt = r_t * exp(c_t)
//     Bh = b_t * exp(-c_t)         Kh = k_t * exp(-c_t)
//     G  = [At;Rt] [Bh;Kh]^T                     (128 x 128, one MMA group)
//     A_ab = strict_lower(At Bh^T)  A_ak = strict_lower(At Kh^T)
//     A_rb = lower(Rt Bh^T)         A_rk = lower(Rt Kh^T)
//     T  = (I - A_ab)^-1                         (unit lower triangular, CUDA cores)
//     X  = At Z0 + A_ak V           U = T X      (u_t = S_{t-1} a_t)
//     Y  = Rt Z0 + A_rb U + A_rk V
//     Z1 = diag(exp(c_L)) (Z0 + Bh^T U + Kh^T V)
// Every MMA operand is fp32 rounded to tf32 (round-to-nearest) in shared memory;
// accumulation is fp32 in TMEM; the state itself never leaves fp32 registers
// except as a tf32-rounded MMA operand.  exp(-c_t) stays finite because the
// kernel requires |c_L| <= 80 per chunk (the model's decay range gives <= 38.9);
// a chain that violates this is flagged and recomputed by the sequential kernel.
//
// All MMAs are M = 128.  Where only 64 rows are meaningful the other 64 rows of
// the A operand alias neighbouring shared memory and the matching accumulator
// lanes are never read.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"
#include "sm100_umma.cuh"

namespace rwkv7 {

// Sequential recomputation of flagged chains (wkv7_seq.cu).
int launch_wkv7_sequential_flagged(const Wkv7Args &p, const int *flags, cudaStream_t stream);

namespace {

using namespace sm100;

constexpr int kN = 64;   // head size
constexpr int kL = 64;   // chunk length
constexpr int kThreads = 128;
constexpr float kMaxLogDecay = 80.f;

// Shared-memory map (bytes from a 1024-aligned base).
constexpr uint32_t kRawBytes = 6 * kL * kN * 2;        // six bf16 tiles
constexpr uint32_t kOffRaw = 0;
constexpr uint32_t kOffAR = kOffRaw + kRawBytes;        // [At;Rt]        128 x 64 fp32
constexpr uint32_t kOffBK = kOffAR + 32768;             // [Bh;Kh]        128 x 64, later [T;A_rb]
constexpr uint32_t kOffZT = kOffBK + 32768;             // [Bh^T;Kh^T]    128 x 64
constexpr uint32_t kOffS = kOffZT + 32768;              // S [i][j]       64 x 64
constexpr uint32_t kOffVT = kOffS + 16384;              // V^T [i][s]     64 x 64
constexpr uint32_t kOffAKRK = kOffVT + 16384;           // [A_ak;A_rk]    128 x 64
constexpr uint32_t kOffXU = kOffAKRK + 32768;           // A_ab, then X^T, then U^T   64 x 64
constexpr uint32_t kOffMisc = kOffXU + 16384;
constexpr uint32_t kMiscBytes = 1024;
constexpr uint32_t kSmemBytes = kOffMisc + kMiscBytes + 1024;  // + alignment slack
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of an sm_100 CTA");

// TMEM columns.
constexpr uint32_t kColG = 0, kColXY = 128, kColU = 192, kColZ = 256, kTmemCols = 512;

struct TmaMaps {
    CUtensorMap m[6];  // r, w, k, v, a, b as [B*T, H*N] bf16, box 64 x 64
};

enum { TR = 0, TW = 1, TK = 2, TV = 3, TA = 4, TB = 5 };

__device__ __forceinline__ float bf16_at(const unsigned char *raw, int tensor, int t, int j) {
    const unsigned short u = *reinterpret_cast<const unsigned short *>(raw + tensor * (kL * kN * 2) + (t * kN + j) * 2);
    return __uint_as_float((unsigned)u << 16);
}

__device__ __forceinline__ void st_tile(unsigned char *tile, int rows, int row, int col, float v) {
    *reinterpret_cast<float *>(tile + tile_off_f32(rows, row, col)) = v;
}

// Issues the 8 K-steps of one 128 x N x 64 tf32 product, both operands K-major.
__device__ __forceinline__ void mma_k64(uint32_t d_tmem, uint32_t a_addr, int a_rows, uint32_t b_addr, int b_rows,
                                        int N, bool accumulate) {
    const uint32_t idesc = make_idesc(kFmtTF32, 128, N, false, false);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
        umma_tf32(d_tmem, desc_kmajor(a_addr, a_rows, ks), desc_kmajor(b_addr, b_rows, ks), idesc,
                  accumulate || ks > 0);
}

__global__ void __launch_bounds__(kThreads, 1)
wkv7_chunked_kernel(const __grid_constant__ TmaMaps maps, const float *__restrict__ s0,
                    __nv_bfloat16 *__restrict__ y, float *__restrict__ s_out, int *__restrict__ flags,
                    int Tlen, int H, int *status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *raw = smem + kOffRaw, *tAR = smem + kOffAR, *tBK = smem + kOffBK, *tZT = smem + kOffZT,
                  *tS = smem + kOffS, *tVT = smem + kOffVT, *tAKRK = smem + kOffAKRK, *tXU = smem + kOffXU;
    uint64_t *bar_tma = reinterpret_cast<uint64_t *>(smem + kOffMisc);
    uint64_t *bar_mma = bar_tma + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kOffMisc + 16);
    float *exp_cl = reinterpret_cast<float *>(smem + kOffMisc + 64);   // [64] exp(c_L)
    float *tot0 = exp_cl + 64;                                         // [64] sum of l over the first half
    int *unsafe = reinterpret_cast<int *>(tot0 + 64);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int bh = blockIdx.x;
    const int bi = bh / H, h = bh % H;
    const int nchunks = (Tlen + kL - 1) / kL;

    if (tid == 0) {
        mbar_init(bar_tma, 1);
        mbar_init(bar_mma, 1);
        mbar_fence_init();
        *unsafe = 0;
#pragma unroll
        for (int i = 0; i < 6; ++i) tma_prefetch_desc(&maps.m[i]);
    }
    if (warp == 0) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;

    auto issue_tma = [&](int chunk) {
        mbar_expect_tx(bar_tma, kRawBytes);
        const int row = bi * Tlen + chunk * kL;
#pragma unroll
        for (int i = 0; i < 6; ++i) tma_load_2d(raw + i * (kL * kN * 2), &maps.m[i], h * kN, row, bar_tma);
    };
    if (tid == 0) issue_tma(0);

    // fp32 state: thread j (< 64) holds Z[j][i] = S[i][j] for all i.
    float Z[kN];
    if (tid < kN) {
#pragma unroll
        for (int i = 0; i < kN; ++i) Z[i] = s0 ? s0[((size_t)bh * kN + i) * kN + tid] : 0.f;
    }

    uint32_t mma_phase = 0;
    bool failed = false;
    int tma_issued = 1, tma_consumed = 0;  // tile batches requested / received

    for (int chunk = 0; chunk < nchunks; ++chunk) {
        const int valid = min(kL, Tlen - chunk * kL);
        // ---------------- wait for this chunk's six input tiles
        {
            const bool ok = mbar_wait(bar_tma, (uint32_t)(chunk & 1));
            if (__syncthreads_or(!ok)) { failed = true; break; }
            ++tma_consumed;
        }
        // ---------------- phase A: decay prefix sums and scaled operands
        {
            const int j = tid & 63, half = tid >> 6;
            const int t0 = half * 32;
            float l[32];
            float sum = 0.f;
#pragma unroll
            for (int u = 0; u < 32; ++u) {
                const int t = t0 + u;
                const float lw = (t < valid) ? -__expf(bf16_at(raw, TW, t, j)) : 0.f;
                sum += lw;
                l[u] = sum;  // inclusive prefix inside this half
            }
            if (half == 0) tot0[j] = sum;
            __syncthreads();
            const float base = half ? tot0[j] : 0.f;
            const float c_last = base + sum;
            if (half == 1) {
                exp_cl[j] = __expf(c_last);
                if (c_last < -kMaxLogDecay) *unsafe = 1;
            }
            float e_prev = __expf(base);  // exp(c_{t0-1})
#pragma unroll
            for (int u = 0; u < 32; ++u) {
                const int t = t0 + u;
                const bool live = t < valid;
                const float e = __expf(base + l[u]);   // exp(c_t)
                const float einv = __frcp_rn(e);        // exp(-c_t)
                const float a = live ? bf16_at(raw, TA, t, j) : 0.f;
                const float r = live ? bf16_at(raw, TR, t, j) : 0.f;
                const float b = live ? bf16_at(raw, TB, t, j) : 0.f;
                const float k = live ? bf16_at(raw, TK, t, j) : 0.f;
                const float v = live ? bf16_at(raw, TV, t, j) : 0.f;
                const float bh_ = round_tf32(b * einv), kh_ = round_tf32(k * einv);
                st_tile(tAR, 128, t, j, round_tf32(a * e_prev));
                st_tile(tAR, 128, 64 + t, j, round_tf32(r * e));
                st_tile(tBK, 128, t, j, bh_);
                st_tile(tBK, 128, 64 + t, j, kh_);
                st_tile(tZT, 128, j, t, bh_);        // Bh^T [j][t]
                st_tile(tZT, 128, 64 + j, t, kh_);   // Kh^T [j][t]
                st_tile(tVT, 64, j, t, v);           // V^T [i][s]  (bf16 values are tf32-exact)
                e_prev = e;
            }
        }
        __syncthreads();  // every read of the raw tiles is done
        if (*unsafe) { failed = true; break; }
        if (chunk + 1 < nchunks) {
            if (tid == 0) issue_tma(chunk + 1);
            ++tma_issued;
        }
        // state -> S operand tile [i][j], tf32-rounded
        if (tid < kN) {
#pragma unroll
            for (int i = 0; i < kN; ++i) st_tile(tS, 64, i, tid, round_tf32(Z[i]));
        }
        fence_proxy_async();
        __syncthreads();
        // ---------------- M1: G = [At;Rt] [Bh;Kh]^T ; state-independent part of Z
        if (tid == 0) {
            tc_fence_after();
            mma_k64(tmem + kColG, smem_u32(tAR), 128, smem_u32(tBK), 128, 128, false);
            // Z = Kh^T V : A = rows 64..127 of the [Bh^T;Kh^T] stack
            mma_k64(tmem + kColZ, smem_u32(tZT) + 64 * 128, 128, smem_u32(tVT), 64, 64, false);
            umma_commit(bar_mma);
        }
        {
            const bool ok = mbar_wait(bar_mma, mma_phase);
            mma_phase ^= 1;
            if (__syncthreads_or(!ok)) { failed = true; break; }
        }
        tc_fence_after();
        // ---------------- hop 1: G -> masked A_ab (fp32), A_ak, A_rb, A_rk (tf32)
        {
            const bool upper = tid >= 64;         // Rt rows: inclusive lower triangle
            const int t = tid & 63;
            const int lim = upper ? t : t - 1;    // keep s <= lim
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + kColG + q * 32, v);
                tmem_ld_wait();
                const int s0c = (q & 1) * 32;     // column offset inside the 64-wide quadrant
                // q = 0,1: against Bh (A_ab / A_rb) ; q = 2,3: against Kh (A_ak / A_rk)
                unsigned char *dst;
                int rows, row;
                bool exact = false;
                if (q < 2) {
                    if (!upper) { dst = tXU; rows = 64; row = t; exact = true; }       // A_ab plain fp32
                    else        { dst = tBK; rows = 128; row = 64 + t; }               // A_rb under T
                } else {
                    dst = tAKRK; rows = 128; row = upper ? 64 + t : t;                 // A_ak / A_rk
                }
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    float4 o;
                    float *of = &o.x;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int s = s0c + e4 * 4 + e;
                        float x = __uint_as_float(v[e4 * 4 + e]);
                        x = (s <= lim) ? x : 0.f;
                        of[e] = exact ? x : round_tf32(x);
                    }
                    *reinterpret_cast<float4 *>(dst + tile_off_f32(rows, row, s0c + e4 * 4)) = o;
                }
            }
        }
        tc_fence_before();
        __syncthreads();
        // ---------------- T = (I - A_ab)^-1 by forward substitution, two threads per column
        {
            // Thread (c, p) keeps T[s][c] for s % 4 in {2p, 2p+1} and sums its half of
            // every dot product; A_ab is strictly lower triangular, so entries with
            // s >= t are zero in shared memory and need no predicate.
            const int c = tid >> 1, p = tid & 1;
            float Tc[32];  // T[4*q + 2*p + e][c] at index 2*q + e
#pragma unroll
            for (int q = 0; q < 32; ++q) Tc[q] = 0.f;
#pragma unroll
            for (int t = 0; t < kL; ++t) {
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int s4 = 0; s4 < (t + 3) / 4; ++s4) {
                    const float2 a2 =
                        *reinterpret_cast<const float2 *>(tXU + tile_off_f32(64, t, s4 * 4) + p * 8);
                    acc0 = fmaf(a2.x, Tc[2 * s4], acc0);
                    acc1 = fmaf(a2.y, Tc[2 * s4 + 1], acc1);
                }
                float acc = acc0 + acc1;
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                const float val = (t == c) ? 1.f : ((t > c) ? acc : 0.f);
                if (((t & 3) >> 1) == p) Tc[2 * (t >> 2) + (t & 1)] = val;
                if (p == 0) st_tile(tBK, 128, t, c, round_tf32(val));
            }
        }
        fence_proxy_async();
        __syncthreads();
        // ---------------- M2: XY = [A_ak;A_rk] V + [At;Rt] Z0
        if (tid == 0) {
            tc_fence_after();
            mma_k64(tmem + kColXY, smem_u32(tAKRK), 128, smem_u32(tVT), 64, 64, false);
            mma_k64(tmem + kColXY, smem_u32(tAR), 128, smem_u32(tS), 64, 64, true);
            umma_commit(bar_mma);
        }
        {
            const bool ok = mbar_wait(bar_mma, mma_phase);
            mma_phase ^= 1;
            if (__syncthreads_or(!ok)) { failed = true; break; }
        }
        tc_fence_after();
        // ---------------- hop 2: X (lanes 0..63) -> X^T [i][t]
        if (tid < 64) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + kColXY + q * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) st_tile(tXU, 64, q * 32 + e, tid, round_tf32(__uint_as_float(v[e])));
            }
        }
        tc_fence_before();
        fence_proxy_async();
        __syncthreads();
        // ---------------- M3: U = T X
        if (tid == 0) {
            tc_fence_after();
            mma_k64(tmem + kColU, smem_u32(tBK), 128, smem_u32(tXU), 64, 64, false);
            umma_commit(bar_mma);
        }
        {
            const bool ok = mbar_wait(bar_mma, mma_phase);
            mma_phase ^= 1;
            if (__syncthreads_or(!ok)) { failed = true; break; }
        }
        tc_fence_after();
        // ---------------- hop 3: U (lanes 0..63) -> U^T [i][t]   (M3 has finished reading X^T)
        if (tid < 64) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + kColU + q * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) st_tile(tXU, 64, q * 32 + e, tid, round_tf32(__uint_as_float(v[e])));
            }
        }
        tc_fence_before();
        fence_proxy_async();
        __syncthreads();
        // ---------------- M4: XY[64..127] += A_rb U ; Z += Bh^T U
        if (tid == 0) {
            tc_fence_after();
            mma_k64(tmem + kColXY, smem_u32(tBK), 128, smem_u32(tXU), 64, 64, true);
            mma_k64(tmem + kColZ, smem_u32(tZT), 128, smem_u32(tXU), 64, 64, true);
            umma_commit(bar_mma);
        }
        {
            const bool ok = mbar_wait(bar_mma, mma_phase);
            mma_phase ^= 1;
            if (__syncthreads_or(!ok)) { failed = true; break; }
        }
        tc_fence_after();
        // ---------------- hop 4: state update (lanes 0..63) and y (lanes 64..127)
        if (tid < 64) {
            const float g = exp_cl[tid];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + kColZ + q * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) Z[q * 32 + e] = g * (Z[q * 32 + e] + __uint_as_float(v[e]));
            }
        } else {
            const int t = tid - 64;
            __nv_bfloat16 *dst = y + (((size_t)bi * Tlen + chunk * kL + t) * H + h) * kN;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + kColXY + q * 32, v);
                tmem_ld_wait();
                if (t < valid) {
#pragma unroll
                    for (int e8 = 0; e8 < 4; ++e8) {
                        uint4 o;
                        unsigned *ow = &o.x;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[e8 * 8 + 2 * e]),
                                                                            __uint_as_float(v[e8 * 8 + 2 * e + 1]));
                            ow[e] = *reinterpret_cast<const unsigned *>(&h2);
                        }
                        *reinterpret_cast<uint4 *>(dst + q * 32 + e8 * 8) = o;
                    }
                }
            }
        }
        tc_fence_before();
        __syncthreads();
    }

    // ---------------- epilogue
    // A tile batch still in flight must land before the CTA gives up its shared memory.
    if (failed && tma_issued > tma_consumed) mbar_wait(bar_tma, (uint32_t)(tma_consumed & 1));
    const bool bad_decay = *unsafe != 0;
    if (failed && !bad_decay && tid == 0) atomicExch(status, (int)kDevTimeout);
    if (tid == 0) flags[bh] = bad_decay ? 1 : 0;
    if (!failed && s_out != nullptr && tid < kN) {
#pragma unroll
        for (int i = 0; i < kN; ++i) s_out[((size_t)bh * kN + i) * kN + tid] = Z[i];
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---- host side --------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

}  // namespace

size_t wkv7_chunked_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N) {
    (void)T;
    if (N != kN) return 0;
    return (size_t)(B * H) * sizeof(int);  // one fallback flag per (b,h) chain
}

bool wkv7_chunked_supported(const Wkv7Args &p) {
    // TMA needs 16-byte aligned base pointers; the row pitch H*N*2 bytes is a multiple of 128.
    auto aligned = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    return p.N == kN && p.bf16 && aligned(p.r) && aligned(p.w) && aligned(p.k) && aligned(p.v) && aligned(p.a) &&
           aligned(p.b) && aligned(p.y) && p.B * p.T < (int64_t(1) << 31);
}

int launch_wkv7_chunked(const Wkv7Args &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    (void)workspace_bytes;
    EncodeTiledFn encode = encode_fn();
    if (encode == nullptr) return (int)cudaErrorNotSupported;
    TmaMaps maps;
    const void *ptrs[6] = {p.r, p.w, p.k, p.v, p.a, p.b};
    const cuuint64_t dims[2] = {(cuuint64_t)(p.H * p.N), (cuuint64_t)(p.B * p.T)};
    const cuuint64_t strides[1] = {(cuuint64_t)(p.H * p.N * 2)};
    const cuuint32_t box[2] = {(cuuint32_t)kN, (cuuint32_t)kL};
    const cuuint32_t estr[2] = {1, 1};
    for (int i = 0; i < 6; ++i) {
        CUresult r = encode(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptrs[i]), dims,
                            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    int *status = nullptr;
    if (int e = device_status_ptr(p.device, &status)) return e;
    cudaError_t e = cudaFuncSetAttribute(wkv7_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    int *flags = static_cast<int *>(workspace);
    wkv7_chunked_kernel<<<(unsigned)(p.B * p.H), kThreads, kSmemBytes, stream>>>(
        maps, p.s0, reinterpret_cast<__nv_bfloat16 *>(p.y), p.s_out, flags, (int)p.T, (int)p.H, status);
    count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    // Chains whose decay left the safe range are recomputed token by token; the
    // kernel exits at once for every chain that is not flagged.
    return launch_wkv7_sequential_flagged(p, flags, stream);
}

}  // namespace rwkv7
