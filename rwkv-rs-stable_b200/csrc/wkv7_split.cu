// Two-kernel WKV7 prefill for sm_100a (N == 64, bf16 or fp32 tensors, 64-token chunks, fp16 tensor-core
// operands): everything that does not depend on the running state is computed for all chunks in
// parallel by `wkv7_chunk_operator_kernel`, which folds a chunk into one linear operator, and
// `wkv7_state_scan_kernel` then walks each (b,h) chain with one dependent tensor-core product per
// chunk.
//
// Reference semantics: crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:179-242 (token
// recurrence; the reference kernel, kernel.rs:82-195, scans token by token).
//
// Per chain and chunk, with the in-chunk inclusive prefix c_t of the log-decay l_t = -exp(w_t),
// c_L its value at the chunk's end and the reference point m = c_L / 2 (per channel):
//     At = a_t e^{c_{t-1} - m}   Rt = r_t e^{c_t - m}   Bh = b_t e^{m - c_t}   Kh = k_t e^{m - c_t}
//     G  = [At;Rt] [Bh;Kh]^T  ->  A_ab, A_ak (strictly lower), A_rb, A_rk (lower)
//     T  = (I - A_ab)^-1                                   (fp32, CUDA cores, blocked)
//     [A~ | A~k] = T [At e^{m} | A_ak]                     (u_t = S_{t-1} a_t = A~ S^T + A~k V)
//     P  = A~^T Bh     Kt = Kh + A~k^T Bh     W = R + A_rb A~     Ark = A_rk + A_rb A~k
// so that, for the state S[i][j] entering the chunk and V[s][i]:
//     S'[i][j'] = e^{c_L} S[i][j'] + e^{c_L - m} ( sum_j S[i][j] P[j][j'] + sum_s V[s][i] Kt[s][j'] )
//     y[t][i]   = sum_j W[t][j] S[i][j] + sum_s Ark[t][s] V[s][i].
// The operator of a chunk is the 128 x 128 fp16 matrix O[k][n], k = (j | s), n = (j' | t):
//     O = [[P, W^T], [Kt, Ark^T]],
// stored in global memory exactly as its shared-memory image (two 128-row panels of 128 bytes,
// 128-byte swizzle), together with the two fp32 vectors e^{c_L} and e^{c_L - m}.
//
// Every tensor-core operand is fp16 (the same 11-bit significand as tf32).  fp16 has a narrow
// exponent range, which is why the decay factors are taken relative to the middle of the chunk;
// a chunk whose total log-decay exceeds kMaxLogDecay in any channel, or whose operator holds a
// non-finite value, flags its chain, and flagged chains are recomputed by the next kernel in line
// (the launcher passes them to the tf32 chunked kernel or the sequential scan).
//
// Shared-memory operand tiles are [rows][64] 16-bit panels with 128-byte rows, 16-byte chunks
// XOR-ed with (row & 7).  The same tile serves as a K-major operand (rows = M/N index) and as an
// MN-major operand (rows = K index): no transposed copies exist anywhere.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "kernels.h"
#include "sm100_umma.cuh"
#include "trace.h"

namespace rwkv7 {

int launch_wkv7_sequential_flagged(const Wkv7Args &p, const int *flags, cudaStream_t stream);

namespace {

using namespace sm100;

constexpr int kN = 64;
constexpr int kL = 64;
// |c_L| per chunk and channel up to which fp16 operands keep their precision (the small factor
// e^{-|c_L|/2} times a typical vector entry stays a normal fp16 number).  Whether the large factor
// e^{+|c_L|/2} overflows depends on the data (keys and receptances of magnitude 5 overflow from about
// |c_L| = 17); overflow is not predicted but detected: it turns the chunk's operator non-finite, the
// scan sees that in its outputs and flags the chain.
constexpr float kMaxLogDecay = 18.f;
constexpr float kOpScale = 4.f;          // decay-scaled operands are stored times 4: centres fp16's range
constexpr float kInvOpScale = 1.f / kOpScale;
constexpr uint32_t kPanel = 8192;        // one [64][64] 16-bit tile
constexpr uint32_t kOperatorBytes = 4 * kPanel;   // O: 128 x 128 fp16
constexpr uint32_t kVecFloats = 128;              // e^{c_L}[64], e^{c_L - m}[64]

// Byte offset of element (row, col) in a [rows][64] 16-bit panel.
__device__ __forceinline__ uint32_t off16(int row, int col) {
    return (uint32_t)row * 128u + ((((uint32_t)col >> 3) ^ ((uint32_t)row & 7u)) << 4) + ((uint32_t)col & 7u) * 2u;
}
// Descriptors.  K-major: rows = M/N index, one K-step (16 elements) is 32 bytes along the row.
// MN-major: rows = K index, one K-step is 16 rows (2048 bytes); `lbo` is the distance between
// consecutive 64-element blocks of the M/N index.
__device__ __forceinline__ uint64_t dK(uint32_t addr, int ks) { return make_smem_desc(addr + (uint32_t)ks * 32u, 16u, 1024u); }
__device__ __forceinline__ uint64_t dMN(uint32_t addr, uint32_t lbo, int ks) {
    return make_smem_desc(addr + (uint32_t)ks * 2048u, lbo, 1024u);
}
__host__ __device__ constexpr uint32_t idesc16(int M, int N, bool a_mn, bool b_mn) {
    return make_idesc(kFmtF16, M, N, a_mn, b_mn);
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&u));
}
__device__ __forceinline__ float2 unpack_bf2(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}

// ------------------------------------------------------------------------------------------
// Kernel 1: the operator of every chunk.  One CTA of 256 threads works through chunks
// blockIdx.x, blockIdx.x + gridDim.x, ...; two CTAs share an SM.
// ------------------------------------------------------------------------------------------
constexpr int kThreads1 = 256;
// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t kRaw = 0;                       // five bf16 tiles r, w, k, a, b (40 KB); later scratch
constexpr uint32_t kRawBytes = 5 * kPanel;
constexpr int kPitchF = 36;                        // floats per row of the fp32 scratch matrices (a row's own 32-block)
constexpr uint32_t kAm = kRaw;                     // fp32 diagonal 32 x 32 blocks of A_ab [64][36]
constexpr uint32_t kTm = kAm + 64 * kPitchF * 4;   // fp32 their inverses           [64][36]
constexpr uint32_t kWm = kTm + 64 * kPitchF * 4;   // fp32 join scratch [32][20]
constexpr uint32_t kT16 = kRaw + 24 * 1024;        // fp16 T [t][u]
constexpr uint32_t kW2 = kT16 + kPanel;            // fp16 A10 T00 [s][c], 32 rows
constexpr uint32_t kRtrue = kRaw + kRawBytes;      // fp16 r_t e^{c_t} [t][j]
constexpr uint32_t kAR = kRtrue + kPanel;          // fp16 [At; Rt] (Rt's half later holds A_ak)
constexpr uint32_t kAf = kAR;                      // fp16 [A~ e^m | A~k]^T [c][t], 128 rows: replaces [At | A_ak] once it has been read
constexpr uint32_t kArb = kAR + 2 * kPanel;        // fp16 A_rb [t][s]
constexpr uint32_t kArk = kArb + kPanel;           // fp16 A_rk [t][s]
constexpr uint32_t kStage = kAR;                   // the finished operator (32 KB) over AR, A_rb, A_rk
constexpr uint32_t kBK = kArk + kPanel;            // fp16 [Bh; Kh]
constexpr uint32_t kI64 = kBK + 2 * kPanel;        // fp16 identity [64][64]
constexpr uint32_t kMisc1 = kI64 + kPanel;         // barriers, group sums, e^m
constexpr uint32_t kSmem1 = kMisc1 + 3072 + 1024;  // + alignment slack
static_assert(kWm + 32 * 20 * 4 <= kT16, "inverse scratch runs into the fp16 tile of T");
static_assert(kW2 + kPanel / 2 <= kRaw + kRawBytes, "scratch exceeds the raw-tile region");
static_assert(kStage + kOperatorBytes == kBK, "operator staging must cover AR, A_rb, A_rk exactly");
static_assert(2 * (kSmem1 + 1024) <= 232448, "two CTAs per SM");
constexpr uint32_t kSmem1F32 = kSmem1 + kRawBytes;   // fp32 tensors: raw tiles of 16 KB, one CTA per SM
static_assert(kSmem1F32 + 1024 <= 232448, "the fp32 variant must fit an SM");

struct OperatorMaps {
    CUtensorMap m[5];   // r, w, k, a, b as [B*T, H*N] (bf16 or fp32), box 64 x 64, no swizzle
};
enum { XR = 0, XW = 1, XK = 2, XA = 3, XB = 4 };

template <typename TIn>
__global__ void __launch_bounds__(kThreads1, 2)
wkv7_chunk_operator_kernel(const __grid_constant__ OperatorMaps maps, unsigned char *__restrict__ operators,
                           float *__restrict__ vectors, int *__restrict__ flags, int Tlen, int H, int chunk0,
                           int seg_chunks, int nchains, int *work_counter, int *status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // fp32 tensors: the five raw tiles are twice as large, everything behind them moves up by X
    constexpr uint32_t kRawTile = kL * kN * sizeof(TIn), kRawBytesT = 5 * kRawTile, X = kRawBytesT - kRawBytes;
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(status, (int)kDevInternal);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3, hf = warp >> 2;
    const int row = quarter * 32 + lane;          // TMEM lane of this thread
    unsigned char *raw = smem + kRaw;
    float *Am = reinterpret_cast<float *>(smem + kAm);
    float *Tm = reinterpret_cast<float *>(smem + kTm);
    float *Wm = reinterpret_cast<float *>(smem + kWm);
    uint64_t *bar_tma = reinterpret_cast<uint64_t *>(smem + (kMisc1 + X));
    uint64_t *bar_mma = bar_tma + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (kMisc1 + X) + 32);
    int *abort_flag = reinterpret_cast<int *>(smem + (kMisc1 + X) + 48);
    int *next_slot = abort_flag + 1;   // the chunk this CTA works on next (thread 0 draws it, all read it)
    float *grp = reinterpret_cast<float *>(smem + (kMisc1 + X) + 256);     // [8][64]
    float *emv = reinterpret_cast<float *>(smem + (kMisc1 + X) + 256 + 2048);   // e^{m_j} / kOpScale [64]

    if (tid == 0) {
        mbar_init(bar_tma, 1);
        mbar_init(bar_mma, 1);
        mbar_fence_init();
        *abort_flag = 0;
        // Chunks are drawn from a counter (zeroed by the host), so that CTAs which start late - the scan of
        // the previous segment may still hold their place on the SM - simply take fewer of them.
        *next_slot = work_counter ? atomicAdd(work_counter, 1) : (int)blockIdx.x;
#pragma unroll
        for (int i = 0; i < 5; ++i) tma_prefetch_desc(&maps.m[i]);
    }
    // identity tile (constant for the whole kernel)
    for (int idx = tid; idx < kL * 8; idx += kThreads1) {
        const int r = idx >> 3, ch = idx & 7;
        uint4 z = make_uint4(0, 0, 0, 0);
        if ((r >> 3) == ch) {
            const uint32_t one = 0x3c00u << ((r & 1) * 16);
            uint32_t *w = &z.x;
            w[(r & 7) >> 1] = one;
        }
        *reinterpret_cast<uint4 *>(smem + (kI64 + X) + r * 128 + ((ch ^ (r & 7)) << 4)) = z;
    }
    if (warp == 0) tmem_alloc(tmem_slot, 128);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t sb = smem_u32(smem);
    const long long units = (long long)nchains * seg_chunks;

    auto issue_tma = [&](long long unit) {
        const int chain = (int)(unit / seg_chunks), chunk = chunk0 + (int)(unit % seg_chunks);
        const int bi = chain / H, h = chain % H;
        if (!RWKV7_IN_RANGE(chain < nchains && chunk * kL < Tlen, status)) return;   // (the wait then expires)
        mbar_expect_tx(bar_tma, kRawBytesT);
        const int trow = bi * Tlen + chunk * kL;
#pragma unroll
        for (int i = 0; i < 5; ++i) tma_load_2d(raw + i * kRawTile, &maps.m[i], h * kN, trow, bar_tma);
    };
    long long unit = *next_slot;
    if (tid == 0 && unit < units) issue_tma(unit);
    uint32_t tma_phase = 0, mma_phase = 0;
    bool tma_pending = unit < units;   // a tile batch is in flight (thread 0's view is what matters)
    bool failed = false;

    for (; unit < units; unit = *next_slot) {
        const int chain = (int)(unit / seg_chunks), chunk = chunk0 + (int)(unit % seg_chunks);
        const int valid = min(kL, Tlen - chunk * kL);
        if (!mbar_wait(bar_tma, tma_phase)) atomicOr(abort_flag, 1);
        tma_phase ^= 1;
        tma_pending = false;
        if (valid < kL) {
            // partial last chunk: rows past the end become no-op tokens (w = -inf: log-decay -0)
            for (int idx = tid; idx < (kL - valid) * kN; idx += kThreads1) {
                const int t = valid + idx / kN, jj = idx % kN;
#pragma unroll
                for (int x = 0; x < 5; ++x) {
                    if constexpr (sizeof(TIn) == 2)
                        *reinterpret_cast<unsigned short *>(raw + x * kRawTile + (t * kN + jj) * 2) =
                            (x == XW) ? (unsigned short)0xFF80 : (unsigned short)0;
                    else
                        *reinterpret_cast<uint32_t *>(raw + x * kRawTile + (t * kN + jj) * 4) = (x == XW) ? 0xFF800000u : 0u;
                }
            }
            __syncthreads();
        }
        // ---------------- phase A: decay prefix sums, scaled fp16 operands
        const int j2 = lane, tg = warp;            // channel pair (2 j2, 2 j2 + 1), tokens 8 tg .. 8 tg + 7
        const unsigned char *rp = raw + (tg * 8 * kN + 2 * j2) * sizeof(TIn);
        auto ld2 = [&](int tensor, int u) {
            if constexpr (sizeof(TIn) == 2)
                return unpack_bf2(*reinterpret_cast<const uint32_t *>(rp + tensor * kRawTile + u * (kN * 2)));
            else
                return *reinterpret_cast<const float2 *>(rp + tensor * kRawTile + u * (kN * 4));
        };
        float c0[8], c1[8];
        {
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float2 w2 = ld2(XW, u);
                s0 -= __expf(w2.x);
                s1 -= __expf(w2.y);
                c0[u] = s0;
                c1[u] = s1;
            }
            *reinterpret_cast<float2 *>(grp + tg * 64 + 2 * j2) = make_float2(s0, s1);
        }
        // the previous operator must have left its staging area before AR / A_rb / A_rk are rewritten
        if (tid == 0) bulk_wait_group_read<0>();
        __syncthreads();
        if (*abort_flag) { failed = true; break; }
        {
            float base0 = 0.f, base1 = 0.f, tot0 = 0.f, tot1 = 0.f;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const float2 x = *reinterpret_cast<const float2 *>(grp + g * 64 + 2 * j2);
                tot0 += x.x;
                tot1 += x.y;
                if (g < tg) { base0 += x.x; base1 += x.y; }
            }
            const float m0 = 0.5f * tot0, m1 = 0.5f * tot1;
            const float em0 = __expf(m0), em1 = __expf(m1);
            if (tg == 7) {
                if (tot0 < -kMaxLogDecay || tot1 < -kMaxLogDecay || !(tot0 <= 0.f) || !(tot1 <= 0.f))
                    atomicOr(&flags[chain], 1);
                float *vec = vectors + (size_t)unit * kVecFloats;
                if (RWKV7_IN_RANGE(unit < units && 2 * j2 + 1 < kN, status)) {
                    *reinterpret_cast<float2 *>(vec + 2 * j2) = make_float2(__expf(tot0), __expf(tot1));
                    *reinterpret_cast<float2 *>(vec + 64 + 2 * j2) = make_float2(__expf(tot0 - m0), __expf(tot1 - m1));
                }
                *reinterpret_cast<float2 *>(emv + 2 * j2) = make_float2(em0 * kInvOpScale, em1 * kInvOpScale);
            }
            float ep0 = __expf(base0 - m0) * kOpScale, ep1 = __expf(base1 - m1) * kOpScale;   // e^{c_{t-1} - m} * scale
            const float rs0 = em0 * kInvOpScale, rs1 = em1 * kInvOpScale;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = tg * 8 + u;
                const float e0 = __expf(base0 + c0[u] - m0) * kOpScale, e1 = __expf(base1 + c1[u] - m1) * kOpScale;
                // e^{m - c_t} * scale
                const float i0 = __fdividef(kOpScale * kOpScale, e0), i1 = __fdividef(kOpScale * kOpScale, e1);
                const float2 a2 = ld2(XA, u), r2 = ld2(XR, u), b2 = ld2(XB, u), k2 = ld2(XK, u);
                const uint32_t o = off16(t, 2 * j2);
                if (!RWKV7_IN_RANGE(o + 4 <= kPanel, status)) continue;
                *reinterpret_cast<uint32_t *>(smem + (kAR + X) + o) = pack_h2(a2.x * ep0, a2.y * ep1);
                *reinterpret_cast<uint32_t *>(smem + (kAR + X) + kPanel + o) = pack_h2(r2.x * e0, r2.y * e1);
                *reinterpret_cast<uint32_t *>(smem + (kBK + X) + o) = pack_h2(b2.x * i0, b2.y * i1);
                *reinterpret_cast<uint32_t *>(smem + (kBK + X) + kPanel + o) = pack_h2(k2.x * i0, k2.y * i1);
                *reinterpret_cast<uint32_t *>(smem + (kRtrue + X) + o) = pack_h2(r2.x * e0 * rs0, r2.y * e1 * rs1);
                ep0 = e0;
                ep1 = e1;
            }
        }
        fence_proxy_async();
        // A chain that is flagged (by this chunk's decay just now, or by an earlier chunk) is recomputed by
        // the next kernel in line whatever happens here: skip the rest of its chunks.  (Another CTA may set
        // the flag at any moment: the barrier makes one decision of what the threads read.)
        if (__syncthreads_or(*reinterpret_cast<volatile int *>(&flags[chain]) != 0)) {
            if (tid == 0) {
                const long long next = work_counter ? (long long)atomicAdd(work_counter, 1) : unit + gridDim.x;
                *next_slot = next < units ? (int)next : 0x7fffffff;
                if (next < units && !*abort_flag) {
                    issue_tma(next);
                    tma_pending = true;
                }
            }
            __syncthreads();
            continue;
        }
        // ---------------- G = [At;Rt] [Bh;Kh]^T   (128 x 128, contraction over the 64 channels)
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                umma_f16(tmem, dK(sb + (kAR + X), ks), dK(sb + (kBK + X), ks), idesc16(128, 128, false, false), ks > 0);
            umma_commit(bar_mma);
        }
        if (!mbar_wait(bar_mma, mma_phase)) atomicOr(abort_flag, 1);
        mma_phase ^= 1;
        tc_fence_after();
        // ---------------- G -> A_ab, A_ak, A_rb, A_rk, masked to the lower triangle.  A_ab's two diagonal
        // 32 x 32 blocks go to the fp32 scratch of the inverse, its lower-left block straight into the
        // fp16 tile of T (where the second level of the inverse replaces it); the others are fp16 tiles.
        {
            const bool rt_rows = quarter >= 2;        // Rt rows keep the diagonal
            const int t = row & 63;
            const bool low_rows = t < 32;             // (warp-uniform: one quarter is 32 consecutive rows)
            const int lim = rt_rows ? t : t - 1;      // keep s <= lim
            constexpr float sc = kInvOpScale * kInvOpScale;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const bool zero_half = low_rows && half == 1;   // columns 32..63 of rows 0..31: above the diagonal
                if (!rt_rows && hf == 0) {
                    if (zero_half) continue;
                    uint32_t v[32];
                    tmem_ld32(tmem + lane_base + half * 32, v);
                    tmem_ld_wait();
                    if (low_rows == (half == 0)) {   // diagonal block of this row: fp32, strictly lower
                        float *dst = Am + t * kPitchF;
#pragma unroll
                        for (int e4 = 0; e4 < 8; ++e4) {
                            float4 o;
                            float *of = &o.x;
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                of[e] = (half * 32 + e4 * 4 + e <= lim) ? __uint_as_float(v[e4 * 4 + e]) * sc : 0.f;
                            *reinterpret_cast<float4 *>(dst + e4 * 4) = o;
                        }
                    } else {                          // rows 32..63, columns 0..31: A_10 of the second level
#pragma unroll
                        for (int e8 = 0; e8 < 4; ++e8) {
                            uint32_t w[4];
#pragma unroll
                            for (int e2 = 0; e2 < 4; ++e2)
                                w[e2] = pack_h2(__uint_as_float(v[e8 * 8 + e2 * 2]) * sc, __uint_as_float(v[e8 * 8 + e2 * 2 + 1]) * sc);
                            *reinterpret_cast<uint4 *>(smem + kT16 + off16(t, e8 * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                } else {
                    const uint32_t tile = !rt_rows ? ((kAR + X) + kPanel) : (hf == 0 ? (kArb + X) : (kArk + X));   // A_ak takes Rt's place
                    uint32_t v[32];
                    if (!zero_half) {
                        tmem_ld32(tmem + lane_base + hf * 64 + half * 32, v);
                        tmem_ld_wait();
                    }
#pragma unroll
                    for (int e8 = 0; e8 < 4; ++e8) {
                        uint32_t w[4] = {0u, 0u, 0u, 0u};
                        if (!zero_half) {
#pragma unroll
                            for (int e2 = 0; e2 < 4; ++e2) {
                                const int sidx = half * 32 + e8 * 8 + e2 * 2;
                                const float x0 = (sidx <= lim) ? __uint_as_float(v[e8 * 8 + e2 * 2]) * sc : 0.f;
                                const float x1 = (sidx + 1 <= lim) ? __uint_as_float(v[e8 * 8 + e2 * 2 + 1]) * sc : 0.f;
                                w[e2] = pack_h2(x0, x1);
                            }
                        }
                        *reinterpret_cast<uint4 *>(smem + tile + off16(t, half * 32 + e8 * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
        tc_fence_before();
        // ---------------- T = (I - A_ab)^-1.  The two 32 x 32 diagonal blocks in fp32 on the CUDA cores:
        // 16 x 16 blocks by forward substitution (the 64 threads that wrote the scratch go on as soon as they
        // are done, the others are still writing their tiles), then [[T00, 0], [T11 A10 T00, T11]].
        if (tid < 64) {
            asm volatile("bar.sync 1, 64;" ::: "memory");
            const int b = tid >> 4, cc = tid & 15;
            const float *Ab = Am + (16 * b) * kPitchF + 16 * (b & 1);
            float x[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int s4 = 0; s4 < (t + 3) / 4; ++s4) {
                    const float4 a4 = *reinterpret_cast<const float4 *>(Ab + t * kPitchF + 4 * s4);
                    if (4 * s4 + 0 < t) acc0 = fmaf(a4.x, x[4 * s4 + 0], acc0);
                    if (4 * s4 + 1 < t) acc1 = fmaf(a4.y, x[4 * s4 + 1], acc1);
                    if (4 * s4 + 2 < t) acc0 = fmaf(a4.z, x[4 * s4 + 2], acc0);
                    if (4 * s4 + 3 < t) acc1 = fmaf(a4.w, x[4 * s4 + 3], acc1);
                }
                x[t] = (t == cc) ? 1.f : ((t > cc) ? acc0 + acc1 : 0.f);
                Tm[(16 * b + t) * kPitchF + 16 * (b & 1) + cc] = x[t];
            }
        }
        __syncthreads();
        if (*abort_flag) { failed = true; break; }
        {   // the two pairs of 16-blocks; 512 outputs per product, two per thread
            const int pr = tid >> 7, t = (tid >> 3) & 15, cb = (tid & 7) * 2;
            const float *arow = Am + (32 * pr + 16 + t) * kPitchF;       // A10[t][.]  (row-local columns 0..15)
            const float *tcol = Tm + (32 * pr) * kPitchF + cb;           // T00[.][cb..]
            float w0 = 0.f, w1 = 0.f;
#pragma unroll
            for (int s = 0; s < 16; ++s) {
                const float a = arow[s];
                const float2 tt = *reinterpret_cast<const float2 *>(tcol + s * kPitchF);
                w0 = fmaf(a, tt.x, w0);   // (T00 is complete: zeros above its diagonal were written)
                w1 = fmaf(a, tt.y, w1);
            }
            *reinterpret_cast<float2 *>(Wm + (16 * pr + t) * 20 + cb) = make_float2(w0, w1);
            __syncthreads();
            const float *trow = Tm + (32 * pr + 16 + t) * kPitchF + 16;   // T11[t][.]
            const float *wcol = Wm + (16 * pr) * 20 + cb;
            float z0 = 0.f, z1 = 0.f;
#pragma unroll
            for (int s = 0; s < 16; ++s) {
                const float a = trow[s];
                const float2 ww = *reinterpret_cast<const float2 *>(wcol + s * 20);
                z0 = fmaf(a, ww.x, z0);
                z1 = fmaf(a, ww.y, z1);
            }
            *reinterpret_cast<float2 *>(Tm + (32 * pr + 16 + t) * kPitchF + cb) = make_float2(z0, z1);
        }
        __syncthreads();
        {   // diagonal 32-blocks -> fp16 tile T[t][u] (zero above the diagonal), and zeros in the block above them
            const int t = tid >> 2, c0 = (tid & 3) * 8, tl = t & 31;
            const float *src = Tm + t * kPitchF + c0;
            const float4 x0 = *reinterpret_cast<const float4 *>(src), x1 = *reinterpret_cast<const float4 *>(src + 4);
            const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            uint32_t w[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2)
                w[e2] = pack_h2(c0 + 2 * e2 <= tl ? xs[2 * e2] : 0.f, c0 + 2 * e2 + 1 <= tl ? xs[2 * e2 + 1] : 0.f);
            *reinterpret_cast<uint4 *>(smem + kT16 + off16(t, 32 * (t >> 5) + c0)) = make_uint4(w[0], w[1], w[2], w[3]);
            if (tid < 128)   // rows 0..31, columns 32..63
                *reinterpret_cast<uint4 *>(smem + kT16 + off16(tid >> 2, 32 + (tid & 3) * 8)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        __syncthreads();
        // second level on the tensor core: T10 = T11 (A10 T00), fp16 operands, two dependent products
        // (N = 64: the upper 32 columns of both results are never read)
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)   // rows 32.. of the tile (A10) against T00[u][c] (rows u of the same tile, MN-major)
                umma_f16(tmem, dK(sb + kT16 + 32 * 128, ks), dMN(sb + kT16, kPanel, ks), idesc16(128, 64, false, true), ks > 0);
            umma_commit(bar_mma);
        }
        if (!mbar_wait(bar_mma, mma_phase)) atomicOr(abort_flag, 1);
        mma_phase ^= 1;
        tc_fence_after();
        if (quarter == 0) {   // lanes 0..31 hold the 32 rows; 16 columns per warp
            uint32_t v[16];
            tmem_ld16(tmem + hf * 16, v);
            tmem_ld_wait();
            uint32_t w[8];
#pragma unroll
            for (int e2 = 0; e2 < 8; ++e2) w[e2] = pack_h2(__uint_as_float(v[2 * e2]), __uint_as_float(v[2 * e2 + 1]));
            *reinterpret_cast<uint4 *>(smem + kW2 + off16(lane, hf * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4 *>(smem + kW2 + off16(lane, hf * 16 + 8)) = make_uint4(w[4], w[5], w[6], w[7]);
        }
        tc_fence_before();
        fence_proxy_async();
        __syncthreads();
        if (*abort_flag) { failed = true; break; }
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)   // T11 (rows 32.., columns 32..63) against W[s][c] (MN-major)
                umma_f16(tmem, dK(sb + kT16 + 32 * 128, 2 + ks), dMN(sb + kW2, kPanel, ks), idesc16(128, 64, false, true), ks > 0);
            umma_commit(bar_mma);
        }
        if (!mbar_wait(bar_mma, mma_phase)) atomicOr(abort_flag, 1);
        mma_phase ^= 1;
        tc_fence_after();
        if (quarter == 0) {
            uint32_t v[16];
            tmem_ld16(tmem + hf * 16, v);
            tmem_ld_wait();
            uint32_t w[8];
#pragma unroll
            for (int e2 = 0; e2 < 8; ++e2) w[e2] = pack_h2(__uint_as_float(v[2 * e2]), __uint_as_float(v[2 * e2 + 1]));
            *reinterpret_cast<uint4 *>(smem + kT16 + off16(32 + lane, hf * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4 *>(smem + kT16 + off16(32 + lane, hf * 16 + 8)) = make_uint4(w[4], w[5], w[6], w[7]);
        }
        tc_fence_before();
        fence_proxy_async();
        __syncthreads();
        // ---------------- [A~ | A~k]^T = [At | A_ak]^T T^T   (rows c = (j | s), columns t)
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                umma_f16(tmem, dMN(sb + (kAR + X), kPanel, ks), dK(sb + kT16, ks), idesc16(128, 64, true, false), ks > 0);
            umma_commit(bar_mma);
        }
        if (!mbar_wait(bar_mma, mma_phase)) atomicOr(abort_flag, 1);
        mma_phase ^= 1;
        tc_fence_after();
        // T has been read: the raw-tile region (scratch of the inverse, T, W) is dead, request the next chunk's tiles
        if (tid == 0) {
            const long long next = work_counter ? (long long)atomicAdd(work_counter, 1) : unit + gridDim.x;
            *next_slot = next < units ? (int)next : 0x7fffffff;
            if (next < units && !*abort_flag) {
                issue_tma(next);
                tma_pending = true;
            } else {
                // this CTA is on its last chunk: the kernel launched behind this one may be set up now
                asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            }
        }
        {
            uint32_t v[32];
            tmem_ld32(tmem + lane_base + hf * 32, v);
            tmem_ld_wait();
            const float scale = row < 64 ? emv[row] : 1.f;   // A~ rows: back to the true scale
#pragma unroll
            for (int e8 = 0; e8 < 4; ++e8) {
                uint32_t w[4];
#pragma unroll
                for (int e2 = 0; e2 < 4; ++e2)
                    w[e2] = pack_h2(__uint_as_float(v[e8 * 8 + 2 * e2]) * scale, __uint_as_float(v[e8 * 8 + 2 * e2 + 1]) * scale);
                *reinterpret_cast<uint4 *>(smem + (kAf + X) + off16(row, hf * 32 + e8 * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        tc_fence_before();
        fence_proxy_async();
        __syncthreads();
        if (*abort_flag) { failed = true; break; }
        // ---------------- O = [A~|A~k]^T [Bh | A_rb^T]  +  [R|A_rk]^T [0 | I]
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // columns j': contraction over t with Bh[t][j'] (MN-major B)
                umma_f16(tmem, dK(sb + (kAf + X), ks), dMN(sb + (kBK + X), kPanel, ks), idesc16(128, 64, false, true), ks > 0);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // columns t': contraction over t with A_rb[t'][t]
                umma_f16(tmem + 64, dK(sb + (kAf + X), ks), dK(sb + (kArb + X), ks), idesc16(128, 64, false, false), ks > 0);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // + R[t'][j] and A_rk[t'][s], through the identity
                umma_f16(tmem + 64, dMN(sb + (kRtrue + X), (kArk + X) - (kRtrue + X), ks), dK(sb + (kI64 + X), ks), idesc16(128, 64, true, false), true);
            umma_commit(bar_mma);
        }
        if (!mbar_wait(bar_mma, mma_phase)) atomicOr(abort_flag, 1);
        mma_phase ^= 1;
        tc_fence_after();
        {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + hf * 64 + half * 32, v);
                tmem_ld_wait();
                float add[32];
                const bool kt_rows = hf == 0 && row >= 64;      // Kt = Kh + A~k^T Bh
                const float sc = hf == 0 ? kInvOpScale : 1.f;   // Bh and Kh carry the operand scale
                if (kt_rows) {
#pragma unroll
                    for (int e8 = 0; e8 < 4; ++e8) {
                        const uint4 q = *reinterpret_cast<const uint4 *>(smem + (kBK + X) + kPanel + off16(row - 64, half * 32 + e8 * 8));
                        const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int e2 = 0; e2 < 4; ++e2) {
                            const float2 f = unpack_h2(qs[e2]);
                            add[e8 * 8 + 2 * e2] = f.x;
                            add[e8 * 8 + 2 * e2 + 1] = f.y;
                        }
                    }
                }
#pragma unroll
                for (int e8 = 0; e8 < 4; ++e8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e2 = 0; e2 < 4; ++e2) {
                        float x0 = __uint_as_float(v[e8 * 8 + 2 * e2]), x1 = __uint_as_float(v[e8 * 8 + 2 * e2 + 1]);
                        if (kt_rows) { x0 += add[e8 * 8 + 2 * e2]; x1 += add[e8 * 8 + 2 * e2 + 1]; }
                        w[e2] = pack_h2(x0 * sc, x1 * sc);
                    }
                    // panel hf, row k = this thread's lane, 16-byte chunk of columns n
                    const uint32_t so = hf * (2 * kPanel) + off16(row, half * 32 + e8 * 8);
                    if (RWKV7_IN_RANGE(so + 16 <= kOperatorBytes, status))
                        *reinterpret_cast<uint4 *>(smem + (kStage + X) + so) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
        tc_fence_before();
        fence_proxy_async();
        __syncthreads();
        if (tid == 0 && RWKV7_IN_RANGE(unit >= 0 && unit < units, status)) {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(operators + (size_t)unit * kOperatorBytes),
                         "r"(sb + (kStage + X)), "r"(kOperatorBytes)
                         : "memory");
            bulk_commit_group();
        }
    }
    // ---------------- epilogue
    __syncthreads();
    if (*abort_flag) failed = true;
    if (tid == 0) {
        bulk_wait_group<0>();
        if (failed) {
            if (tma_pending) mbar_wait(bar_tma, tma_phase);   // tiles in flight must land before the CTA leaves
            atomicExch(status, (int)kDevTimeout);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// ------------------------------------------------------------------------------------------
// Kernel 2: the scan.  One CTA per chain.  Warps 0-7 own the 128 TMEM lanes twice over (two
// column halves): lanes 0-63 are the state rows j' (fp32 state Z[j'][i] = S[i][j'] in registers),
// lanes 64-127 the output tokens t.  Warp 8 streams operators, V tiles and the decay vectors into a
// ring of stages, warp 9 issues the MMAs, warp 10 (four-stage variant) turns each V tile into fp16 as it
// lands.  Per chunk
// D[(j' | t)][i] = sum_k O[k][(j' | t)] [Z ; V][k][i]: the V half is issued as soon as a stage is
// ready, only the Z half waits for the previous chunk.
// ------------------------------------------------------------------------------------------
constexpr int kComputeWarps = 8;
// The four-stage variant (one CTA per SM) has warps of its own for the V conversion and one for issuing the V half
// of the products; in the two-stage variant
// (two CTAs per SM, or beside an operator CTA) the compute warps do it between their other work, which measured
// faster there (32 chains x 1024 chunks overlapped with the operator kernel: 1.41 against 1.53 ms).
template <int NS> struct ScanWarps {
    static constexpr bool kConvWarp = NS > 2;
    static constexpr int kConv = 4;   // converter warps (one alone needs about 770 cycles per tile: as long as the whole serial step)
    // warps 8 loader, 9 MMA issuer; then 10 converter, 11 issuer of the V half, 12.. the other converters
    static constexpr int kThreads = (kComputeWarps + 2 + (kConvWarp ? 1 + kConv : 0)) * 32;
};
constexpr uint32_t kVecBytes = kVecFloats * 4;              // the chunk's two decay vectors

// A stage: the operator, the fp16 V tile the tensor core reads and, for fp32 tensors, the fp32 tile as
// it lands (bf16 tiles are converted in place).
template <int NS, typename TIO>
struct ScanSmem {
    static constexpr bool kF32 = sizeof(TIO) == 4;
    static constexpr uint32_t kVLand = kOperatorBytes + (kF32 ? kPanel : 0u);      // where the V tile lands in a stage
    static constexpr uint32_t kVBytes = kL * kN * sizeof(TIO);
    static constexpr uint32_t kStage = kOperatorBytes + kPanel + (kF32 ? kVBytes : 0u);
    static constexpr uint32_t kStages = 0;
    static constexpr uint32_t kZ = NS * kStage;            // fp16 state tile Z[j][i]
    static constexpr uint32_t kY = kZ + kPanel;            // two output tiles [t][i] on their way out (128-byte swizzle; fp32: two panels of 32 channels each)
    static constexpr uint32_t kYTile = kL * kN * sizeof(TIO);
    static constexpr uint32_t kVecs = kY + 2 * kYTile;     // per stage: e^{c_L}[64], e^{c_L - m}[64]
    static constexpr uint32_t kBars = kVecs + NS * kVecBytes;
    static constexpr uint32_t kBytes = kBars + 512 + 1024;   // + alignment slack
};
static_assert(ScanSmem<4, __nv_bfloat16>::kBytes <= 232448 && ScanSmem<3, float>::kBytes <= 232448, "scan stages exceed an SM");

struct ScanMaps {
    CUtensorMap v;   // [B*T, H*N]: bf16, box 64 x 64, 128-byte swizzle; fp32, box 64 x 64, no swizzle
    CUtensorMap y;   // the output, same view: bf16, box 64 x 64; fp32, box 32 channels x 64 tokens; 128-byte swizzle
};

template <int NS, typename TIO>
__global__ void __launch_bounds__(ScanWarps<NS>::kThreads, NS <= 2 ? 2 : 1)
wkv7_state_scan_kernel(const __grid_constant__ ScanMaps maps, const unsigned char *__restrict__ operators,
                       const float *__restrict__ vectors, const float *state_in, float *state_out,
                       TIO *__restrict__ y, int *flags, int Tlen, int H, int chunk0,
                       int seg_chunks, int nseg, int check_flags, int *status) {
    using SM = ScanSmem<NS, TIO>;
    constexpr bool kF32 = SM::kF32;
    constexpr uint32_t kStageBytes = SM::kStage;
    static_assert(!kF32 || ScanWarps<NS>::kConvWarp, "fp32 tiles need the converter warp");
    extern __shared__ __align__(1024) unsigned char smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(status, (int)kDevInternal);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // (launched behind the operator kernel with programmatic stream serialization: this kernel may start while
    // that one is still finishing; everything below reads what it wrote)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(smem + SM::kBars);   // [NS] stage landed (bytes)
    constexpr bool kConvWarp = ScanWarps<NS>::kConvWarp;
    uint64_t *bar_vready = bar_full + NS;      // [NS] V tile converted to fp16 (one arrival per converting warp)
    uint64_t *bar_empty = bar_vready + NS;     // [NS] the stage's MMAs are done
    uint64_t *bar_accfull = bar_empty + NS;    // [2] accumulator complete
    uint64_t *bar_accfree = bar_accfull + 2;   // [2] accumulator read back (8 arrivals)
    uint64_t *bar_zready = bar_accfree + 2;    // state tile written (4 arrivals)
    uint64_t *bar_vdone = bar_zready + 1;      // [2] (four-stage variant) the V half of the accumulator is complete
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_vdone + 2);
    int *abort_flag = reinterpret_cast<int *>(tmem_slot + 1);
    int *chain_bad = abort_flag + 1;

    const int chain = blockIdx.x;
    const int bi = chain / H, h = chain % H;
    const int n = nseg;   // chunks this launch covers: chunk0 .. chunk0 + n - 1

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + s, 1);
            mbar_init(bar_vready + s, kConvWarp ? ScanWarps<NS>::kConv : 8);      // one arrival per converting warp
            mbar_init(bar_empty + s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_accfull + a, 1);
            mbar_init(bar_accfree + a, 8);                     // one arrival per compute warp
        }
        mbar_init(bar_zready, 4);                              // one arrival per state warp
        mbar_init(bar_vdone + 0, 1);
        mbar_init(bar_vdone + 1, 1);
        mbar_fence_init();
        *abort_flag = 0;
        *chain_bad = 0;
        tma_prefetch_desc(&maps.v);
        tma_prefetch_desc(&maps.y);
    }
    if (warp == 0) tmem_alloc(tmem_slot, 128);
    tc_fence_before();
    // A chain that is already flagged (by the operator kernel, or by the scan of an earlier segment) is
    // recomputed by the next kernel in line: nothing to do here.
    const bool skip_chain = __syncthreads_or(*reinterpret_cast<volatile int *>(&flags[chain]) != 0) != 0;
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (skip_chain) {
        tc_fence_before();
        __syncthreads();
        if (warp == 0) tmem_dealloc(tmem, 128);
        return;
    }
    // A warp's threads meet, then its first lane arrives for all of them: an mbarrier takes one arrival at a time,
    // and 128 or 256 of them in a row were a visible part of the chain's serial step.
    auto warp_arrive = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };
    // A wait of a whole warp: every lane polls (one polling lane and a broadcast measured far slower: 264 against
    // 231 us at 96 chains x 64 chunks), then a vote makes the outcome the same in all lanes, so that every lane takes
    // the same way out of a loop whose lanes meet at warp barriers.
    auto warp_wait = [&](uint64_t *bar, uint32_t parity, bool spin) -> bool {
        const bool ok = spin ? mbar_wait_spin(bar, parity) : mbar_wait(bar, parity);
        return __all_sync(0xffffffffu, ok) != 0;
    };
    const uint32_t sb = smem_u32(smem);
    const unsigned char *ops = operators + ((size_t)chain * seg_chunks) * kOperatorBytes;
    const float *vecs = vectors + ((size_t)chain * seg_chunks) * kVecFloats;

    if (warp == kComputeWarps) {
        // ---------------- loader: operator (bulk copy) + V tile (TMA) per stage
        if (lane == 0) {
            int issued = 0, landed_needed = 0;
            for (int c = 0; c < n; ++c) {
                const int s = c % NS;
                if (c >= NS && !mbar_wait(bar_empty + s, (uint32_t)((c / NS - 1) & 1))) { atomicOr(abort_flag, 1); break; }
                if (*reinterpret_cast<volatile int *>(abort_flag)) break;
                if (!RWKV7_IN_RANGE(c < seg_chunks && (chunk0 + c) * kL < Tlen, status)) break;
                mbar_expect_tx(bar_full + s, kOperatorBytes + SM::kVBytes + kVecBytes);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(sb + SM::kStages + s * kStageBytes), "l"(ops + (size_t)c * kOperatorBytes),
                               "r"(kOperatorBytes), "r"(smem_u32(bar_full + s))
                             : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(sb + SM::kVecs + s * kVecBytes), "l"(vecs + (size_t)c * kVecFloats),
                               "r"(kVecBytes), "r"(smem_u32(bar_full + s))
                             : "memory");
                tma_load_2d(smem + SM::kStages + s * kStageBytes + SM::kVLand, &maps.v, h * kN,
                            bi * Tlen + (chunk0 + c) * kL, bar_full + s);
                ++issued;
            }
            // On an abort the copies already requested must land before the CTA gives up its shared memory.
            if (*reinterpret_cast<volatile int *>(abort_flag)) {
                (void)landed_needed;
                for (int c = max(0, issued - NS); c < issued; ++c) mbar_wait(bar_full + c % NS, (uint32_t)((c / NS) & 1));
            }
        }
    } else if (warp == kComputeWarps + 1) {
        // ---------------- MMA issuer.  Two-stage variant: both halves of the chunk's product.  Four-stage variant:
        // the Z half only (k = j: rows 0..63 of the operator against Z[j][i]); the V half is issued ahead of time by
        // another thread into the same accumulator, and since products issued by different threads are ordered
        // only through a barrier, this thread waits until that half is complete before it adds to it.
        if (lane == 0) {
            constexpr uint32_t id = idesc16(128, 64, true, true);
            for (int c = 0; c < n; ++c) {
                const int s = c % NS, a = c & 1;
                const uint32_t op = sb + SM::kStages + s * kStageBytes, vt = op + kOperatorBytes;
                if constexpr (kConvWarp) {
                    if (!mbar_wait(bar_vdone + a, (uint32_t)((c >> 1) & 1))) { atomicOr(abort_flag, 1); break; }
                } else {
                    if (!mbar_wait(bar_vready + s, (uint32_t)((c / NS) & 1))) { atomicOr(abort_flag, 1); break; }
                    if (!mbar_wait(bar_accfree + a, (uint32_t)(((c >> 1) & 1) ^ 1))) { atomicOr(abort_flag, 1); break; }
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)   // k = 64 + s: rows 64.. of both operator panels against V[s][i]
                        umma_f16(tmem + a * 64, dMN(op, 2 * kPanel, 4 + ks), dMN(vt, kPanel, ks), id, ks > 0);
                }
                if (!mbar_wait_spin(bar_zready, (uint32_t)(c & 1))) { atomicOr(abort_flag, 1); break; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // k = j: rows 0..63 against Z[j][i]
                    umma_f16(tmem + a * 64, dMN(op, 2 * kPanel, ks), dMN(sb + SM::kZ, kPanel, ks), id, true);
                umma_commit(bar_accfull + a);
                umma_commit(bar_empty + s);
            }
        }
    } else if (kConvWarp && warp == kComputeWarps + 3) {
        // ---------------- issuer of the V half (four-stage variant): O[64 + s][(j' | t)] against V[s][i], as soon as
        // the tile is converted and the accumulator has been read back, one chunk ahead of the chain.
        if (lane == 0) {
            constexpr uint32_t id = idesc16(128, 64, true, true);
            for (int c = 0; c < n; ++c) {
                const int s = c % NS, a = c & 1;
                const uint32_t op = sb + SM::kStages + s * kStageBytes, vt = op + kOperatorBytes;
                if (!mbar_wait(bar_vready + s, (uint32_t)((c / NS) & 1))) { atomicOr(abort_flag, 1); break; }
                if (!mbar_wait(bar_accfree + a, (uint32_t)(((c >> 1) & 1) ^ 1))) { atomicOr(abort_flag, 1); break; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_f16(tmem + a * 64, dMN(op, 2 * kPanel, 4 + ks), dMN(vt, kPanel, ks), id, ks > 0);
                umma_commit(bar_vdone + a);
            }
        }
    } else if (kConvWarp && (warp == kComputeWarps + 2 || warp >= kComputeWarps + 4)) {
        // ---------------- V converters.  The V tile arrives as bf16 and the tensor core wants both operands
        // of a product in one format: these warps turn it into fp16 in place (element by element, the layout
        // is untouched; each a quarter of the tile) as soon as the stage has landed, well ahead of the product
        // that reads it.  (Done by the compute warps between their other work, the conversion sat on the chain's
        // serial path.)
        constexpr int kConv = ScanWarps<NS>::kConv;
        const int ci = warp == kComputeWarps + 2 ? 0 : warp - (kComputeWarps + 3);   // 0 .. kConv - 1
        for (int c = 0; c < n; ++c) {
            const int s = c % NS;
            if (!warp_wait(bar_full + s, (uint32_t)((c / NS) & 1), false)) { atomicOr(abort_flag, 1); break; }
            unsigned char *vt = smem + SM::kStages + s * kStageBytes + kOperatorBytes;
            if constexpr (!kF32) {
                uint4 *p = reinterpret_cast<uint4 *>(vt);
                constexpr int kShare = (int)(kPanel / 16 / 32) / kConv;
                uint4 x[kShare];
#pragma unroll
                for (int q = 0; q < kShare; ++q) x[q] = p[(ci * kShare + q) * 32 + lane];
#pragma unroll
                for (int q = 0; q < kShare; ++q) {
                    uint32_t *xs = &x[q].x;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = unpack_bf2(xs[e]);
                        xs[e] = pack_h2(f.x, f.y);
                    }
                    p[(ci * kShare + q) * 32 + lane] = x[q];
                }
            } else {
                // fp32 tile [t][i] (rows of 256 bytes) -> fp16 panel: eight channels of one token per step
                const unsigned char *land = smem + SM::kStages + s * kStageBytes + SM::kVLand;
                constexpr int kShare = kL * kN / 8 / 32 / kConv;
#pragma unroll
                for (int q = 0; q < kShare; ++q) {
                    const int idx = (ci * kShare + q) * 32 + lane, t = idx >> 3, cg = idx & 7;
                    const float4 x0 = *reinterpret_cast<const float4 *>(land + t * (kN * 4) + cg * 32);
                    const float4 x1 = *reinterpret_cast<const float4 *>(land + t * (kN * 4) + cg * 32 + 16);
                    *reinterpret_cast<uint4 *>(vt + off16(t, cg * 8)) =
                        make_uint4(pack_h2(x0.x, x0.y), pack_h2(x0.z, x0.w), pack_h2(x1.x, x1.y), pack_h2(x1.z, x1.w));
                }
            }
            fence_proxy_async();
            warp_arrive(bar_vready + s);
        }
    } else {
        const int quarter = warp & 3, hf = warp >> 2;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int i0 = hf * 32;                       // this thread's 32 value channels
        // Two-stage variant: the 256 compute threads turn the V tile into fp16 in place, 32 bytes each, one
        // chunk ahead of the product that reads it.
        auto convert_v = [&](int c) -> bool {
            if constexpr (kConvWarp) return true;
            const int s = c % NS;
            if (!warp_wait(bar_full + s, (uint32_t)((c / NS) & 1), false)) return false;
            uint4 *p = reinterpret_cast<uint4 *>(smem + SM::kStages + s * kStageBytes + kOperatorBytes + tid * 32);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint4 x = p[q];
                uint32_t *xs = &x.x;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf2(xs[e]);
                    xs[e] = pack_h2(f.x, f.y);
                }
                p[q] = x;
            }
            fence_proxy_async();
            warp_arrive(bar_vready + s);
            return true;
        };
        if (quarter < 2) {
            // ---------------- state rows j'
            const int jp = quarter * 32 + lane;
            float Z[32];
#pragma unroll
            for (int e = 0; e < 32; ++e)
                Z[e] = state_in ? state_in[((size_t)chain * kN + i0 + e) * kN + jp] : 0.f;
            auto put_tile = [&]() {
#pragma unroll
                for (int e8 = 0; e8 < 4; ++e8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e2 = 0; e2 < 4; ++e2) w[e2] = pack_h2(Z[e8 * 8 + 2 * e2], Z[e8 * 8 + 2 * e2 + 1]);
                    if (RWKV7_IN_RANGE(off16(jp, i0 + e8 * 8) + 16 <= kPanel, status))
                        *reinterpret_cast<uint4 *>(smem + SM::kZ + off16(jp, i0 + e8 * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                fence_proxy_async();
                warp_arrive(bar_zready);
            };
            put_tile();
            // this row's two decay factors per chunk come with the stage; they are read one chunk ahead (the
            // stage of chunk c + 1 cannot be refilled before this thread has handed over that chunk's state)
            const float *ring = reinterpret_cast<const float *>(smem + SM::kVecs);
            auto load_gg = [&](int c, float2 &out) -> bool {
                if (c >= n) { out = make_float2(1.f, 0.f); return true; }
                const int s = c % NS;
                // (in the two-stage variant this thread has just waited for the stage in convert_v)
                if (kConvWarp && !warp_wait(bar_full + s, (uint32_t)((c / NS) & 1), false)) return false;
                out = make_float2(ring[s * kVecFloats + jp], ring[s * kVecFloats + 64 + jp]);
                return true;
            };
            float2 gg, gg_next = make_float2(1.f, 0.f);
            if (n > 0 && !convert_v(0)) atomicOr(abort_flag, 1);
            if (!load_gg(0, gg)) atomicOr(abort_flag, 1);
            for (int c = 0; c < n; ++c) {
                const int a = c & 1;
                // (the tensor core is busy with this chunk's state product: time for the next chunk's vectors and tile)
                if (c + 1 < n && !convert_v(c + 1)) { atomicOr(abort_flag, 1); break; }
                if (!load_gg(c + 1, gg_next)) { atomicOr(abort_flag, 1); break; }
                // (polled without suspending: this wait is on the serial path of the chain)
                if (!warp_wait(bar_accfull + a, (uint32_t)((c >> 1) & 1), true)) { atomicOr(abort_flag, 1); break; }
                tc_fence_after();
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + a * 64 + i0, v);
                tmem_ld_wait();
                tc_fence_before();
                warp_arrive(bar_accfree + a);
#pragma unroll
                for (int e = 0; e < 32; ++e) Z[e] = fmaf(gg.y, __uint_as_float(v[e]), gg.x * Z[e]);
                if (c + 1 < n) put_tile();
                gg = gg_next;
            }
            // A non-finite operator (fp16 overflow upstream) shows in the state for good: flag the chain.
            bool bad = false;
#pragma unroll
            for (int e = 0; e < 32; ++e) bad |= !(fabsf(Z[e]) <= 3.0e38f);
            if (bad) atomicOr(chain_bad, 1);
            asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight compute warps: every flag of this chain is in
            const bool skip = *chain_bad != 0 || (check_flags && flags[chain] != 0);   // flagged chains are recomputed from state_in
            if (state_out != nullptr && !skip && !*reinterpret_cast<volatile int *>(abort_flag)) {
#pragma unroll
                for (int e = 0; e < 32; ++e)
                    if (RWKV7_IN_RANGE(i0 + e < kN && jp < kN, status)) state_out[((size_t)chain * kN + i0 + e) * kN + jp] = Z[e];
            }
        } else {
            // ---------------- output tokens t.  A chunk's y tile is staged in shared memory (one of two
            // buffers, 128-byte swizzle) and leaves by one bulk tensor store; a partial last chunk is stored
            // by the threads themselves.
            const int tq = (quarter - 2) * 32 + lane;     // token within the chunk
            const bool elected = warp == 2 && lane == 0;
            float ysum = 0.f;    // a non-finite output (or one too large for bf16) flags the chain for recomputation
            // After an expired wait this thread stops waiting but still walks the loop, so that the four
            // warps keep meeting at the named barrier below (the call then reports a time-out).
            bool dead = n > 0 && !convert_v(0);
            for (int c = 0; c < n; ++c) {
                const int a = c & 1;
                if (!dead && c + 1 < n && !convert_v(c + 1)) dead = true;
                if (!dead && !warp_wait(bar_accfull + a, (uint32_t)((c >> 1) & 1), false)) dead = true;
                tc_fence_after();
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + a * 64 + i0, v);
                tmem_ld_wait();
                tc_fence_before();
                warp_arrive(bar_accfree + a);
                const int t0 = (chunk0 + c) * kL;
                if constexpr (!kF32) {
                    uint32_t w[16];
#pragma unroll
                    for (int e2 = 0; e2 < 16; ++e2) {
                        const float x0 = __uint_as_float(v[2 * e2]), x1 = __uint_as_float(v[2 * e2 + 1]);
                        ysum += fabsf(x0) + fabsf(x1);   // (a non-finite output makes the sum non-finite for good)
                        const __nv_bfloat162 b2 = __floats2bfloat162_rn(x0, x1);
                        w[e2] = *reinterpret_cast<const uint32_t *>(&b2);
                    }
                    if (t0 + kL <= Tlen) {
                        unsigned char *stage = smem + SM::kY + a * SM::kYTile;
                        // the store that last read this buffer (two chunks ago) must be done with it
                        if (elected) bulk_wait_group_read<1>();
                        asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
                        for (int e8 = 0; e8 < 4; ++e8)
                            if (RWKV7_IN_RANGE(off16(tq, i0 + e8 * 8) + 16 <= kPanel, status))
                                *reinterpret_cast<uint4 *>(stage + off16(tq, i0 + e8 * 8)) = make_uint4(w[4 * e8], w[4 * e8 + 1], w[4 * e8 + 2], w[4 * e8 + 3]);
                        fence_proxy_async();
                        asm volatile("bar.sync 2, 128;" ::: "memory");
                        if (elected) {
                            tma_store_2d(&maps.y, h * kN, bi * Tlen + t0, stage);
                            bulk_commit_group();
                        }
                    } else if (t0 + tq < Tlen) {
                        TIO *dst = y + (((size_t)bi * Tlen + t0 + tq) * H + h) * kN + i0;
#pragma unroll
                        for (int e8 = 0; e8 < 4; ++e8)
                            *reinterpret_cast<uint4 *>(dst + e8 * 8) = make_uint4(w[4 * e8], w[4 * e8 + 1], w[4 * e8 + 2], w[4 * e8 + 3]);
                    }
                } else {
                    // fp32 output: this thread's 32 channels are one 128-byte row of panel `hf` of the staged tile
#pragma unroll
                    for (int e = 0; e < 32; ++e) ysum += fabsf(__uint_as_float(v[e]));
                    if (t0 + kL <= Tlen) {
                        unsigned char *stage = smem + SM::kY + a * SM::kYTile + hf * (SM::kYTile / 2);
                        if (elected) bulk_wait_group_read<1>();   // (a chunk's two stores form one group)
                        asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
                        for (int e4 = 0; e4 < 8; ++e4) {
                            const uint32_t o = (uint32_t)tq * 128u + (((uint32_t)e4 ^ ((uint32_t)tq & 7u)) << 4);
                            if (RWKV7_IN_RANGE(o + 16 <= SM::kYTile / 2, status))
                                *reinterpret_cast<uint4 *>(stage + o) = make_uint4(v[4 * e4], v[4 * e4 + 1], v[4 * e4 + 2], v[4 * e4 + 3]);
                        }
                        fence_proxy_async();
                        asm volatile("bar.sync 2, 128;" ::: "memory");
                        if (elected) {
                            unsigned char *tile = smem + SM::kY + a * SM::kYTile;
                            tma_store_2d(&maps.y, h * kN, bi * Tlen + t0, tile);
                            tma_store_2d(&maps.y, h * kN + 32, bi * Tlen + t0, tile + SM::kYTile / 2);
                            bulk_commit_group();
                        }
                    } else if (t0 + tq < Tlen) {
                        TIO *dst = y + (((size_t)bi * Tlen + t0 + tq) * H + h) * kN + i0;
#pragma unroll
                        for (int e4 = 0; e4 < 8; ++e4)
                            *reinterpret_cast<uint4 *>(dst + e4 * 4) = make_uint4(v[4 * e4], v[4 * e4 + 1], v[4 * e4 + 2], v[4 * e4 + 3]);
                    }
                }
            }
            if (elected) bulk_wait_group<0>();   // the stores read this CTA's shared memory
            if (dead) atomicOr(abort_flag, 1);
            if (!(ysum <= 3.0e38f)) atomicOr(chain_bad, 1);
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
    }
    __syncthreads();
    if (tid == 0) {
        if (*abort_flag) atomicExch(status, (int)kDevTimeout);
        if (*chain_bad) atomicOr(&flags[chain], 1);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

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

constexpr size_t kAlign = 256;
size_t align_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }
// Operator storage the launcher aims for: beyond this a call is cut into segments of chunks.
constexpr size_t kOperatorBudget = (size_t)768 << 20;

}  // namespace

// ---- host side ------------------------------------------------------------------------------
//
// Workspace: [flags: one int per chain][kMaxSegments work counters][carried fp32 state per chain]
//            [vectors of buffer 0][vectors of buffer 1][operators of buffer 0][operators of buffer 1].
// A call is cut into segments of chunks.  With at most as many chains as SMs the scan of a segment
// leaves most of the GPU idle (one latency-bound CTA per chain), so it runs on a second stream beside
// the operator kernel of the next segment, which writes the other buffer.

namespace {

constexpr int kMaxSegments = 1024;

struct WorkspaceLayout {
    size_t flags, counters, carry, vectors[2], operators[2], total;
    size_t seg;      // chunks per segment
    int buffers;     // 1 or 2
};

size_t fixed_part(size_t chains) {
    return align_up(chains * sizeof(int)) + align_up(kMaxSegments * sizeof(int)) + align_up(chains * kN * kN * sizeof(float));
}

WorkspaceLayout layout_for(size_t chains, size_t seg, int buffers) {
    WorkspaceLayout l{};
    l.seg = seg;
    l.buffers = buffers;
    l.flags = 0;
    l.counters = align_up(chains * sizeof(int));
    l.carry = l.counters + align_up(kMaxSegments * sizeof(int));
    size_t off = l.carry + align_up(chains * kN * kN * sizeof(float));
    for (int b = 0; b < 2; ++b) {
        l.vectors[b] = off;
        if (b < buffers) off += chains * seg * kVecFloats * sizeof(float);   // (512 bytes per chunk: stays aligned)
    }
    for (int b = 0; b < 2; ++b) {
        l.operators[b] = off;
        if (b < buffers) off += chains * seg * kOperatorBytes;
    }
    l.total = off;
    return l;
}

// How a call is cut: the number of segments that balances the scan of the last segment (which nothing
// overlaps) against the few microseconds a segment boundary costs, within the operator budget.
//
// When the scan of a segment may run beside the operator kernel of the next one.  The scan is one latency-bound
// CTA per chain (0.7 us per chunk with an SM to itself), the operator kernel throughput work that fills every SM
// twice over (8.7 us per chunk and CTA): with x = chains x 8.7 / (2 SMs x 0.7) the two in sequence take (x + 1)
// scan times.  On SM partitions (the scans on `chains` SMs rounded up to eight, the operator kernel on the rest)
// they take max(x SMs / (SMs - R), 1): a gain while x SMs / (SMs - R) < x + 1, which on 148 SMs is up to about
// 40 chains.  Measured (B200, 148 SMs; in sequence / on partitions, us): 12 chains x 1024 chunks 945 / 799;
// 32 x 1024 1489 / 1336; 64 x 512 1195 / 1638.  Without partitions the scan CTAs sit beside operator CTAs (the
// operator kernel then launches 2 SMs - chains CTAs) and run at half their pace: 32 x 1024 1381-1411, but 12 x 1024
// 1204 and 64 x 512 1424, both worse than in sequence; that schedule is kept for 24 to 40 chains where the driver
// offers no partitions.  Short sequences do not pay either way (32 chains x 128 chunks 257 against 236 us: the
// first operator kernel and the last scan overlap nothing; on partitions 32 x 128 216 against 207 us, but 24 x 192
// 234 against 256 and 12 x 128 133 against 138).  Hence: at most 27 % as many chains as SMs and at least 192
// chunks, or at most 11 % and at least 128.
bool overlap_applies(size_t chains, size_t nchunks, int num_sms) {
    return wkv7_split_overlap() != 0 && num_sms > 0 && chains * 100 <= (size_t)num_sms * 27 &&
           (nchunks >= 192 || (nchunks >= 128 && chains * 100 <= (size_t)num_sms * 11));
}
// (the schedule beside operator CTAs, where partitions are not to be had)
bool shared_sm_overlap_pays(size_t chains, size_t nchunks, int num_sms) {
    return chains * 100 >= (size_t)num_sms * 16 && nchunks >= 256;
}

size_t preferred_segment(size_t chains, size_t nchunks, bool overlap) {
    size_t seg = nchunks;
    if (overlap) {
        size_t nseg = 1;
        while ((nseg + 1) * (nseg + 1) * 16 <= nchunks && nseg < 32) ++nseg;   // about sqrt(nchunks / 16): measured best (1024 chunks: 8 segments)
        seg = (nchunks + nseg - 1) / nseg;
    }
    const size_t per_chunk = chains * kOperatorBytes * (overlap ? 2 : 1);
    if (seg * per_chunk > kOperatorBudget) seg = kOperatorBudget / per_chunk;
    if ((nchunks + seg - 1) / (seg ? seg : 1) > (size_t)kMaxSegments) seg = (nchunks + kMaxSegments - 1) / kMaxSegments;
    return seg < 1 ? 1 : seg;
}

// Second stream and events of a device, created on first use.
struct DeviceStreams {
    cudaStream_t side = nullptr;
    cudaEvent_t fork = nullptr, built[2] = {nullptr, nullptr}, scanned[2] = {nullptr, nullptr};
    bool ok = false;
};

std::mutex g_streams_mu;
DeviceStreams g_streams[64];

// (the caller holds g_streams_mu and has made `device` current)
DeviceStreams *device_streams(int device) {
    if (device < 0 || device >= 64) return nullptr;
    DeviceStreams &d = g_streams[device];
    if (!d.ok) {
        int least = 0, greatest = 0;
        if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) return nullptr;
        if (cudaStreamCreateWithPriority(&d.side, cudaStreamNonBlocking, greatest) != cudaSuccess) return nullptr;
        cudaEvent_t *evs[5] = {&d.fork, &d.built[0], &d.built[1], &d.scanned[0], &d.scanned[1]};
        for (cudaEvent_t *e : evs)
            if (cudaEventCreateWithFlags(e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        d.ok = true;
    }
    return &d;
}

// ---- SM partitions (green contexts) for the overlapped schedule ----------------------------------
// The scan of a segment and the operator kernel of the next one want different things from an SM: a scan CTA is
// one latency-bound chain that must not be slowed down, an operator CTA is throughput work.  Sharing SMs (a scan
// CTA beside an operator CTA) costs the scan about half its pace.  Where the driver offers it, the device's SMs
// are therefore split once into two partitions, each with a stream of its own: the scans run two to an SM on
// the small one, the operator kernels two to an SM on the rest, and neither sees the other's CTAs.
struct GreenApi {
    CUresult (*deviceGet)(CUdevice *, int) = nullptr;
    CUresult (*getRes)(CUdevice, CUdevResource *, CUdevResourceType) = nullptr;
    CUresult (*split)(CUdevResource *, unsigned int *, const CUdevResource *, CUdevResource *, unsigned int, unsigned int) = nullptr;
    CUresult (*genDesc)(CUdevResourceDesc *, CUdevResource *, unsigned int) = nullptr;
    CUresult (*create)(CUgreenCtx *, CUdevResourceDesc, CUdevice, unsigned int) = nullptr;
    CUresult (*streamCreate)(CUstream *, CUgreenCtx, unsigned int, int) = nullptr;
    CUresult (*ctxFromGreen)(CUcontext *, CUgreenCtx) = nullptr;
    CUresult (*ctxPush)(CUcontext) = nullptr;
    CUresult (*ctxPop)(CUcontext *) = nullptr;
    bool ok = false;
};

const GreenApi &green_api() {
    static GreenApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        auto get = [](const char *name, void **out) {
            cudaDriverEntryPointQueryResult q;
            return cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess &&
                   *out != nullptr;
        };
        api.ok = get("cuDeviceGet", reinterpret_cast<void **>(&api.deviceGet)) &&
                 get("cuDeviceGetDevResource", reinterpret_cast<void **>(&api.getRes)) &&
                 get("cuDevSmResourceSplitByCount", reinterpret_cast<void **>(&api.split)) &&
                 get("cuDevResourceGenerateDesc", reinterpret_cast<void **>(&api.genDesc)) &&
                 get("cuGreenCtxCreate", reinterpret_cast<void **>(&api.create)) &&
                 get("cuGreenCtxStreamCreate", reinterpret_cast<void **>(&api.streamCreate)) &&
                 get("cuCtxFromGreenCtx", reinterpret_cast<void **>(&api.ctxFromGreen)) &&
                 get("cuCtxPushCurrent", reinterpret_cast<void **>(&api.ctxPush)) &&
                 get("cuCtxPopCurrent", reinterpret_cast<void **>(&api.ctxPop));
        (void)cudaGetLastError();
    });
    return api;
}

struct DevicePartition {
    int scan_sms = 0, op_sms = 0;          // SMs of the two partitions as the driver cut them
    cudaStream_t scan_stream = nullptr, op_stream = nullptr;
    // (an event is recorded only on a stream of the context it was created in; waits may cross contexts)
    cudaEvent_t built[2] = {nullptr, nullptr}, scanned[2] = {nullptr, nullptr};
    bool tried = false, ok = false;
};

// per device, per size of the scan partition in units of eight SMs (the granularity of a split)
DevicePartition g_partitions[64][10];

// (the caller holds g_streams_mu and has made `device` current)  Null when the driver does not offer it.
DevicePartition *device_partition(int device, int want_scan_sms, int num_sms) {
    const GreenApi &api = green_api();
    const int slot = (want_scan_sms + 7) / 8;
    // A tool injected into the process (a profiler, a memory checker: they announce themselves through these
    // variables) may not support kernels in green contexts: Nsight Compute 2025.2 fails to prepare them for
    // profiling and ends the application.  Under such a tool the partitions are not used.
    static const bool injected = std::getenv("CUDA_INJECTION64_PATH") != nullptr ||
                                 std::getenv("NV_NSIGHT_INJECTION_PORT_BASE") != nullptr ||
                                 std::getenv("NV_COMPUTE_PROFILER_PERFWORKS_DIR") != nullptr;
    if (!api.ok || injected || device < 0 || device >= 64 || slot < 1 || slot >= 10) return nullptr;
    DevicePartition &d = g_partitions[device][slot];
    if (d.tried) return d.ok ? &d : nullptr;
    d.tried = true;
    CUdevice dev;
    CUdevResource all, scan_res, op_res;
    unsigned int nb = 1;
    if (api.deviceGet(&dev, device) != CUDA_SUCCESS) return nullptr;
    if (api.getRes(dev, &all, CU_DEV_RESOURCE_TYPE_SM) != CUDA_SUCCESS) return nullptr;
    if (api.split(&scan_res, &nb, &all, &op_res, 0, (unsigned int)(slot * 8)) != CUDA_SUCCESS || nb != 1) return nullptr;
    d.scan_sms = (int)scan_res.sm.smCount;
    d.op_sms = (int)op_res.sm.smCount;
    if (d.scan_sms < want_scan_sms || d.op_sms < num_sms / 2) return nullptr;
    int least = 0, greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) return nullptr;
    struct Half { CUdevResource *res; cudaStream_t *stream; cudaEvent_t *events; int priority; };
    const Half halves[2] = {{&scan_res, &d.scan_stream, d.scanned, greatest}, {&op_res, &d.op_stream, d.built, least}};
    for (const Half &h : halves) {
        CUdevResourceDesc desc;
        CUgreenCtx green;
        CUcontext ctx, popped;
        CUstream st;
        if (api.genDesc(&desc, h.res, 1) != CUDA_SUCCESS) return nullptr;
        if (api.create(&green, desc, dev, CU_GREEN_CTX_DEFAULT_STREAM) != CUDA_SUCCESS) return nullptr;
        if (api.streamCreate(&st, green, CU_STREAM_NON_BLOCKING, h.priority) != CUDA_SUCCESS) return nullptr;
        *h.stream = reinterpret_cast<cudaStream_t>(st);
        if (api.ctxFromGreen(&ctx, green) != CUDA_SUCCESS || api.ctxPush(ctx) != CUDA_SUCCESS) return nullptr;
        bool made = true;
        for (int i = 0; i < 2; ++i) made = made && cudaEventCreateWithFlags(&h.events[i], cudaEventDisableTiming) == cudaSuccess;
        api.ctxPop(&popped);
        if (!made) return nullptr;
    }
    d.ok = true;
    return &d;
}

std::atomic<int> g_split_overlap{1};

}  // namespace

int wkv7_split_overlap() { return g_split_overlap.load(); }
// 0: everything on the caller's stream; 1: overlapped, on SM partitions where the driver offers them;
// 2: overlapped on the second stream without partitions.
void wkv7_set_split_overlap(int on) { g_split_overlap.store(on < 0 || on > 2 ? 1 : on); }

size_t wkv7_split_min_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N) {
    (void)T;
    if (N != kN) return 0;
    return layout_for((size_t)(B * H), 1, 1).total;
}

size_t wkv7_split_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N, int num_sms) {
    if (N != kN) return 0;
    const size_t chains = (size_t)(B * H);
    const size_t nchunks = (size_t)((T + kL - 1) / kL);
    const bool overlap = overlap_applies(chains, nchunks, num_sms);
    return layout_for(chains, preferred_segment(chains, nchunks, overlap), overlap ? 2 : 1).total;
}

bool wkv7_split_supported(const Wkv7Args &p) {
    auto aligned = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    return p.N == kN && aligned(p.r) && aligned(p.w) && aligned(p.k) && aligned(p.v) && aligned(p.a) &&
           aligned(p.b) && aligned(p.y) && p.B * p.T < (int64_t(1) << 31) && p.B * p.H < (int64_t(1) << 24);
}

// Enqueues the two kernels, once per segment of chunks, and leaves one flag per chain in the first
// B*H ints of the workspace: 1 for chains that the caller's next kernel must recompute (their final
// state is not written: it may alias the initial state that the recomputation starts from).
int launch_wkv7_split(const Wkv7Args &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    EncodeTiledFn encode = encode_fn();
    if (encode == nullptr) return (int)cudaErrorNotSupported;
    const size_t chains = (size_t)(p.B * p.H);
    const int nchunks = (int)((p.T + kL - 1) / kL);
    // The plan: overlapped (two buffers) when it applies and the workspace holds two segments of a useful
    // length, else one buffer with the longest segment that fits.
    // (fp32 tensors: one operator CTA per SM and the three-stage scan, which does not fit beside it)
    bool overlap = p.bf16 && overlap_applies(chains, (size_t)nchunks, p.num_sms);
    // The second stream and its events, or the two SM partitions with theirs, are shared by all calls on a device:
    // the enqueueing of an overlapped call is serialised per process from here on.
    std::unique_lock<std::mutex> lock(g_streams_mu, std::defer_lock);
    DevicePartition *part = nullptr;
    if (overlap) {
        lock.lock();
        // (a stream that is being captured into a graph stays within its own context: no partitions then)
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) capturing = cudaStreamCaptureStatusActive;
        if (wkv7_split_overlap() == 1 && capturing == cudaStreamCaptureStatusNone)
            part = device_partition(p.device, (int)chains, p.num_sms);
        if (part == nullptr && !shared_sm_overlap_pays(chains, (size_t)nchunks, p.num_sms)) overlap = false;
    }
    size_t seg = preferred_segment(chains, (size_t)nchunks, overlap);
    const size_t fixed = fixed_part(chains);
    if (workspace_bytes < fixed) return (int)cudaErrorInvalidValue;
    const size_t per_chunk = chains * ((size_t)kVecFloats * sizeof(float) + kOperatorBytes);
    if (overlap && layout_for(chains, seg, 2).total > workspace_bytes) {
        const size_t fit = (workspace_bytes - fixed) / (2 * per_chunk);
        if (fit >= 8) seg = fit;
        else overlap = false;
    }
    if (!overlap) {
        seg = preferred_segment(chains, (size_t)nchunks, false);
        const size_t fit = (workspace_bytes - fixed) / per_chunk;
        if (fit < 1) return (int)cudaErrorInvalidValue;
        if (seg > fit) seg = fit;
    }
    if (seg > (size_t)nchunks) seg = (size_t)nchunks;
    const int nsegments = (int)(((size_t)nchunks + seg - 1) / seg);
    if (nsegments > kMaxSegments) return (int)cudaErrorInvalidValue;
    if (nsegments < 2) overlap = false;
    const WorkspaceLayout lay = layout_for(chains, seg, overlap ? 2 : 1);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    int *flags = reinterpret_cast<int *>(ws + lay.flags);
    int *counters = reinterpret_cast<int *>(ws + lay.counters);
    float *carry = reinterpret_cast<float *>(ws + lay.carry);

    OperatorMaps omaps;
    ScanMaps smaps;
    const void *ptrs[5] = {p.r, p.w, p.k, p.a, p.b};
    const cuuint64_t dims[2] = {(cuuint64_t)(p.H * p.N), (cuuint64_t)(p.B * p.T)};
    const size_t esize = p.bf16 ? 2 : 4;
    const CUtensorMapDataType etype = p.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const cuuint64_t strides[1] = {(cuuint64_t)(p.H * p.N * esize)};
    const cuuint32_t box[2] = {(cuuint32_t)kN, (cuuint32_t)kL};
    const cuuint32_t estr[2] = {1, 1};
    for (int i = 0; i < 5; ++i) {
        CUresult r = encode(&omaps.m[i], etype, 2, const_cast<void *>(ptrs[i]), dims, strides,
                            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    {   // V: bf16 tiles land swizzled and are converted in place; fp32 tiles land row-major beside their fp16 copy
        CUresult r = encode(&smaps.v, etype, 2, const_cast<void *>(p.v), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, p.bf16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    {   // y: rows of 128 bytes in shared memory (64 bf16 channels, or 32 fp32 channels: two stores per chunk)
        const cuuint32_t ybox[2] = {(cuuint32_t)(p.bf16 ? kN : kN / 2), (cuuint32_t)kL};
        CUresult r = encode(&smaps.y, etype, 2, p.y, dims, strides, ybox, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    int *status = nullptr;
    if (int e = device_status_ptr(p.device, &status)) return e;

    auto k1 = p.bf16 ? wkv7_chunk_operator_kernel<__nv_bfloat16> : wkv7_chunk_operator_kernel<float>;
    const size_t smem1 = p.bf16 ? kSmem1 : kSmem1F32;
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (e != cudaSuccess) return (int)e;
    if (!overlap) part = nullptr;
    cudaStream_t op_stream = part ? part->op_stream : stream;
    // Beside an operator CTA only the two-stage scan fits; it is also the one for more chains than SMs.  On its own
    // partition a scan CTA has an SM to itself.
    const bool small_scan = (overlap && part == nullptr) || (int64_t)chains > (int64_t)p.num_sms;
    auto launch_scan = [&](cudaStream_t st, int buf, const float *s_in, float *s_out, int c0, int n, int check) -> cudaError_t {
        const unsigned char *ops = ws + lay.operators[buf];
        const float *vecs = reinterpret_cast<const float *>(ws + lay.vectors[buf]);
        auto go = [&](auto kern, auto ytype, size_t smem_bytes, unsigned threads) -> cudaError_t {
            cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
            if (err != cudaSuccess) return err;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)chains);
            cfg.blockDim = dim3(threads);
            cfg.dynamicSmemBytes = smem_bytes;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = st == stream ? 1 : 0;   // directly behind its operator kernel on the caller's stream
            using YPtr = std::remove_pointer_t<decltype(ytype)> *;
            err = cudaLaunchKernelEx(&cfg, kern, smaps, ops, vecs, s_in, s_out, reinterpret_cast<YPtr>(p.y), flags,
                                     (int)p.T, (int)p.H, c0, n, n, check, status);
            if (err == cudaSuccess) count_launch();
            return err;
        };
        using bf = __nv_bfloat16;
        if (!p.bf16) return go(wkv7_state_scan_kernel<3, float>, (float *)nullptr, ScanSmem<3, float>::kBytes, ScanWarps<3>::kThreads);
        return small_scan ? go(wkv7_state_scan_kernel<2, bf>, (bf *)nullptr, ScanSmem<2, bf>::kBytes, ScanWarps<2>::kThreads)
                          : go(wkv7_state_scan_kernel<4, bf>, (bf *)nullptr, ScanSmem<4, bf>::kBytes, ScanWarps<4>::kThreads);
    };
    auto launch_operators = [&](int buf, int segment, int c0, int n) -> cudaError_t {
        const long long units = (long long)chains * n;
        // (see overlap_applies; on its own partition the kernel fills every SM it has twice over)
        const long long places = part ? 2LL * part->op_sms
                                      : (p.bf16 ? 2LL : 1LL) * p.num_sms - (overlap ? (long long)chains : 0);
        const unsigned grid = (unsigned)(units < places ? units : places);
        // (the operator of (chain, chunk) sits at index chain * n + chunk - c0 of the buffer in both kernels)
        k1<<<grid, kThreads1, smem1, op_stream>>>(omaps, ws + lay.operators[buf], reinterpret_cast<float *>(ws + lay.vectors[buf]),
                                                flags, (int)p.T, (int)p.H, c0, n, (int)chains, counters + segment, status);
        count_launch();
        return cudaGetLastError();
    };
    // flags and work counters start at zero
    e = cudaMemsetAsync(ws, 0, lay.carry, stream);
    if (e != cudaSuccess) return (int)e;

    if (!overlap) {
        int segment = 0;
        for (int c0 = 0; c0 < nchunks; c0 += (int)seg, ++segment) {
            const int n = (int)((size_t)(nchunks - c0) < seg ? (size_t)(nchunks - c0) : seg);
            e = launch_operators(0, segment, c0, n);
            if (e != cudaSuccess) return (int)e;
            const bool first = c0 == 0, last = c0 + n >= nchunks;
            e = launch_scan(stream, 0, first ? p.s0 : carry, last ? p.s_out : carry, c0, n, last ? 1 : 0);
            if (e != cudaSuccess) return (int)e;
        }
        return 0;
    }
    // Overlapped: operator kernels on the caller's stream (or the stream of the operator partition), scans on the
    // device's second, high-priority stream (or the stream of the scan partition); events order a scan after its
    // operators, and an operator kernel after the scan that last read the buffer it is about to overwrite.
    DeviceStreams *ds = device_streams(p.device);
    if (ds == nullptr) return (int)cudaErrorUnknown;
    cudaStream_t scan_stream = part ? part->scan_stream : ds->side;
    cudaEvent_t *built = part ? part->built : ds->built, *scanned = part ? part->scanned : ds->scanned;
    e = cudaEventRecord(ds->fork, stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(scan_stream, ds->fork, 0);
    if (e == cudaSuccess && part) e = cudaStreamWaitEvent(op_stream, ds->fork, 0);
    if (e != cudaSuccess) return (int)e;
    int segment = 0;
    for (int c0 = 0; c0 < nchunks; c0 += (int)seg, ++segment) {
        const int n = (int)((size_t)(nchunks - c0) < seg ? (size_t)(nchunks - c0) : seg);
        const int buf = segment & 1;
        if (segment >= 2) {
            e = cudaStreamWaitEvent(op_stream, scanned[buf], 0);
            if (e != cudaSuccess) return (int)e;
        }
        e = launch_operators(buf, segment, c0, n);
        if (e == cudaSuccess) e = cudaEventRecord(built[buf], op_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(scan_stream, built[buf], 0);
        if (e != cudaSuccess) return (int)e;
        const bool first = c0 == 0, last = c0 + n >= nchunks;
        e = launch_scan(scan_stream, buf, first ? p.s0 : carry, last ? p.s_out : carry, c0, n, last ? 1 : 0);
        if (e == cudaSuccess) e = cudaEventRecord(scanned[buf], scan_stream);
        if (e != cudaSuccess) return (int)e;
    }
    // join: the caller's stream continues after the last scan (scans run in order on their stream, and every
    // operator kernel is ordered before the scan of its segment)
    e = cudaStreamWaitEvent(stream, scanned[(segment - 1) & 1], 0);
    return (int)e;
}

}  // namespace rwkv7
