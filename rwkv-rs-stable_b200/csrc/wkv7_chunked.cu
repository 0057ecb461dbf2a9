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
//     X  = At Z0 + A_ak V           U = (I - A_ab)^-1 X      (u_t = S_{t-1} a_t)
//         solved by 16-token blocks: T_bb = (I - A_bb)^-1 on CUDA cores, then
//         X_b += A_{b,<b} U_{<b}, U_b = T_bb X_b on the tensor core
//     Y  = Rt Z0 + A_rb U + A_rk V
//     Z1 = diag(exp(c_L)) (Z0 + Bh^T U + Kh^T V)
// The state path is computed transposed (value index on the TMEM lanes), so X^T
// and U^T stay in TMEM and are the A operand of the MMAs that consume them.
// Every shared-memory MMA operand is fp32 rounded to tf32 (round-to-nearest);
// accumulation is fp32 in TMEM; the state itself never leaves fp32 registers
// except as a tf32-rounded MMA operand.  exp(-c_t) stays finite because the
// kernel requires |c_L| <= 80 per chunk (the model's decay range gives <= 38.9);
// a chain that violates this is flagged and recomputed by the sequential kernel.
//
// All MMAs are M = 128.  Where only 64 rows are meaningful the other 64 rows of
// the A operand alias neighbouring shared memory and the matching accumulator
// lanes are never read.
//
// One CTA of 16 warps per (b,h).  Warp w reads TMEM lanes 32*(w%4).. and, among
// the four warps that share a lane quarter, column group w/4.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
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
constexpr int kThreads = 512;
constexpr float kMaxLogDecay = 80.f;

// Shared-memory map (bytes from a 1024-aligned base).
constexpr uint32_t kRawBytes = 6 * kL * kN * 2;        // six bf16 tiles; scratch after phase A
constexpr uint32_t kOffRaw = 0;
constexpr uint32_t kOffAR = kOffRaw + kRawBytes;        // [At;Rt]        128 x 64 fp32
constexpr uint32_t kOffBK = kOffAR + 32768;             // [Bh;Kh]        128 x 64, later [T;A_rb]
constexpr uint32_t kOffZT = kOffBK + 32768;             // [Bh^T;Kh^T]    128 x 64
constexpr uint32_t kOffS = kOffZT + 32768;              // S [i][j]       64 x 64
constexpr uint32_t kOffVT = kOffS + 16384;              // V^T [i][s]     64 x 64
constexpr uint32_t kOffAKRK = kOffVT + 16384;           // [A_ak;A_rk]    128 x 64
constexpr uint32_t kOffXU = kOffAKRK + 32768;           // group sums, then X^T, then U^T   64 x 64
constexpr uint32_t kOffMisc = kOffXU + 16384;
constexpr uint32_t kMiscBytes = 1024;
constexpr uint32_t kSmemBytes = kOffMisc + kMiscBytes + 1024;  // + alignment slack
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory of an sm_100 CTA");

// fp32 scratch of the triangular solve: the diagonal 16 x 16 blocks of A_ab, inside the
// raw-tile region (free between phase A and the next TMA request).
#ifndef RWKV7_SOLVE_BLOCK
#define RWKV7_SOLVE_BLOCK 32
#endif
#ifndef RWKV7_TRUNC_DEBIAS
#define RWKV7_TRUNC_DEBIAS 3.4e-4f
#endif
constexpr int kBlk = RWKV7_SOLVE_BLOCK;   // token block of the triangular solve (16 or 32)
// An MMA whose A operand is read from TMEM truncates that operand to tf32, losing on
// average about 0.7 * 2^-11 of its magnitude.  The shared-memory operand of such an MMA
// is scaled up by the same factor before it is rounded, which removes the bias.
constexpr float kDebias = 1.f + RWKV7_TRUNC_DEBIAS;
static_assert(kBlk == 16 || kBlk == 32, "solve block of 16 or 32 tokens");
constexpr int kPitch = 20;    // floats per row of a 16-column scratch matrix (conflict-free 16-byte stores)
constexpr int kPitchA = 36;   // floats per row of the A_ab scratch: the row's diagonal 16 x 16 block, then (odd
                              // 16-token blocks) its block left of the diagonal
constexpr uint32_t kOffAm = kOffRaw;                          // fp32 blocks of A_ab           [64][36]
constexpr uint32_t kOffTm = kOffAm + 64 * kPitchA * 4;        // fp32 16 x 16 block inverses   [64][20]
constexpr uint32_t kOffWm = kOffTm + 64 * kPitch * 4;         // A_10 T_00 of the two pairs    [32][20]
constexpr uint32_t kScratchEnd = kOffWm + 32 * kPitch * 4;
static_assert(kScratchEnd <= kOffRaw + kRawBytes, "inverse scratch exceeds the raw-tile region");

// TMEM columns.
// X^T and Y^T are neighbours: products whose second operands are the two halves of one 128-row tile
// (S [At;Rt]^T, V^T [A_ak;A_rk]^T) then fill both with one N = 128 MMA per K-step instead of two N = 64.
constexpr uint32_t kColG = 0, kColXT = 128, kColYT = 192, kColUT = 256, kColDS = 320, kTmemCols = 512;
static_assert(kColYT == kColXT + 64, "X^T and Y^T must be adjacent accumulators");
constexpr uint32_t kColTX = 384, kColTT = 448;   // cluster of 4: the solve applied to the identity (never with SAVE)
// Identity operand tile [64][64] of that product, inside the raw-tile region past the inverse scratch.
constexpr uint32_t kOffIdent = kOffRaw + 17408;
static_assert(kScratchEnd <= kOffIdent && kOffIdent % 1024 == 0 && kOffIdent + 16384 + 8192 <= kOffRaw + kRawBytes,
              "identity tile (read as a 128-row operand) must stay inside the raw-tile region");

struct TmaMaps {
    CUtensorMap m[6];  // r, w, k, v, a, b as [B*T, H*N] bf16, box 64 x 64
    CUtensorMap snap;  // SAVE: snapshots as [B*H*(T/16)*64, 64] fp32, box 64 rows x 32 columns, 128-byte swizzle
    CUtensorMap y;     // output as [B*T, H*N] bf16, box 64 x 64 (one CTA per chain: y leaves by tensor stores)
};

enum { TR = 0, TW = 1, TK = 2, TV = 3, TA = 4, TB = 5 };

__device__ __forceinline__ float bf16_at(const unsigned char *raw, int tensor, int t, int j) {
    const unsigned short u = *reinterpret_cast<const unsigned short *>(raw + tensor * (kL * kN * 2) + (t * kN + j) * 2);
    return __uint_as_float((unsigned)u << 16);
}

__device__ __forceinline__ void st_tile(unsigned char *tile, int rows, int row, int col, float v) {
    *reinterpret_cast<float *>(tile + tile_off_f32(rows, row, col)) = v;
}
__device__ __forceinline__ void st_tile4(unsigned char *tile, int rows, int row, int col, float4 v) {
    *reinterpret_cast<float4 *>(tile + tile_off_f32(rows, row, col)) = v;
}

// Issues the 8 K-steps of one 128 x N x 64 tf32 product, both operands K-major.
// a0 / b0 are the descriptors of K-step 0; later steps only move the start address.
template <int A_ROWS, int B_ROWS, int N>
__device__ __forceinline__ void mma_k64(uint32_t d_tmem, uint64_t a0, uint64_t b0, bool accumulate) {
    constexpr uint32_t idesc = make_idesc(kFmtTF32, 128, N, false, false);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint64_t ao = (uint64_t)(((ks >> 2) * A_ROWS * 128 + (ks & 3) * 32) >> 4);
        const uint64_t bo = (uint64_t)(((ks >> 2) * B_ROWS * 128 + (ks & 3) * 32) >> 4);
        umma_tf32(d_tmem, a0 + ao, b0 + bo, idesc, accumulate || ks > 0);
    }
}

// Two consecutive K-steps (16 tokens) of the same product, starting a new accumulation.
template <int A_ROWS, int B_ROWS, int N>
__device__ __forceinline__ void mma_kpair(uint32_t d_tmem, uint64_t a0, uint64_t b0, int ks0) {
    constexpr uint32_t idesc = make_idesc(kFmtTF32, 128, N, false, false);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int ks = ks0 + u;
        const uint64_t ao = (uint64_t)(((ks >> 2) * A_ROWS * 128 + (ks & 3) * 32) >> 4);
        const uint64_t bo = (uint64_t)(((ks >> 2) * B_ROWS * 128 + (ks & 3) * 32) >> 4);
        umma_tf32(d_tmem, a0 + ao, b0 + bo, idesc, u > 0);
    }
}

// Same with the A operand read from TMEM (a previous accumulator: 128 lanes x 64
// fp32 columns, 8 columns per K-step; the tensor core truncates it to tf32).
template <int B_ROWS, int N>
__device__ __forceinline__ void mma_k64_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b0, bool accumulate) {
    constexpr uint32_t idesc = make_idesc(kFmtTF32, 128, N, false, false);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint64_t bo = (uint64_t)(((ks >> 2) * B_ROWS * 128 + (ks & 3) * 32) >> 4);
        umma_tf32_ts(d_tmem, a_tmem + ks * 8, b0 + bo, idesc, accumulate || ks > 0);
    }
}

// D[128 x N] (+)= A[tmem, 8 columns per K-step] * B^T, B = rows row0.. and columns col0..
// of a 128-row K-major tile whose K-step-0 descriptor is `tile0`.
template <int N>
__device__ __forceinline__ void mma_ts_block(uint32_t d_tmem, uint32_t a_tmem, uint64_t tile0, int row0, int col0,
                                             int ksteps, bool accumulate) {
    constexpr uint32_t idesc = make_idesc(kFmtTF32, 128, N, false, false);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        if (ks < ksteps) {
            const int col = col0 + 8 * ks;
            const uint64_t bo = (uint64_t)(((col >> 5) * 128 * 128 + row0 * 128 + (col & 31) * 4) >> 4);
            umma_tf32_ts(d_tmem, a_tmem + ks * 8, tile0 + bo, idesc, accumulate || ks > 0);
        }
    }
}

// SAVE: also write what the backward pass needs (wkv7/forward.rs:368-375): the state after every
// 16th token (snapshots [B,H,T/16,N,N], fp32) and state_replacement = U (sa_t = S_{t-1} a_t).  The
// state update dS is then accumulated per 16-token block in four TMEM regions; the state after
// token 16m-1 is diag(exp(c_{16m-1})) (Z0 + the first m blocks).
//
// K > 1: a thread-block cluster of K CTAs shares one chain.  CTA rho owns the chunks
// c = rho (mod K) with all their tiles; everything that does not depend on the incoming state
// (phase A, G, the masks, the block inverses, the products with V) runs ahead, and only the state
// travels: after its chunk a CTA writes the new state into the shared memory of the next CTA
// (the tf32 operand tile, plus the bf16-rounded residual so that the fp32 state is rebuilt to
// 2^-20) and arrives on that CTA's mbarrier.  For workloads with fewer chains than SMs this takes
// the state-independent two thirds of a chunk off the serial path.
template <bool SAVE, int K>
__global__ void __launch_bounds__(kThreads, 1)
wkv7_chunked_kernel(const __grid_constant__ TmaMaps maps, const float *s0,
                    __nv_bfloat16 *__restrict__ y, float *s_out, int *__restrict__ flags,
                    int Tlen, int H, int *status, float *__restrict__ snapshots,
                    __nv_bfloat16 *__restrict__ state_repl, int chain0, int only_flagged) {
    // Every pointer is derived from the array itself so that the accesses stay in
    // the shared address space; the 1024-byte alignment the swizzled tiles need is
    // what the runtime provides and is verified before anything else happens.
    extern __shared__ __align__(1024) unsigned char smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(status, (int)kDevInternal);
        return;
    }
    if constexpr (K == 1 && !SAVE) {
        // Second in line after the two-kernel prefill: only the chains that one left flagged are computed.
        if (only_flagged) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // (may have been launched before the flags' writer finished)
            if (flags[chain0 + blockIdx.x] == 0) return;
        }
    }
    unsigned char *raw = smem + kOffRaw, *tAR = smem + kOffAR, *tBK = smem + kOffBK, *tZT = smem + kOffZT,
                  *tS = smem + kOffS, *tVT = smem + kOffVT, *tAKRK = smem + kOffAKRK, *tXU = smem + kOffXU;
    float *Am = reinterpret_cast<float *>(smem + kOffAm);
    float *Tm = reinterpret_cast<float *>(smem + kOffTm);
    float *Wm = reinterpret_cast<float *>(smem + kOffWm);
    float *grp_tot = reinterpret_cast<float *>(tXU);  // [8][64], phase A only
    // One CTA per chain: a chunk's y tile [t][i] (bf16, 8 KB) is staged here and stored by one bulk tensor
    // copy; stored by the threads themselves (a thread holds 16 tokens of one channel, 2 bytes each) the
    // 128 store instructions of a chunk took 830 cycles of the hop.
    unsigned char *y_stage = tXU + 4096;
    uint64_t *bar_tma = reinterpret_cast<uint64_t *>(smem + kOffMisc);
    uint64_t *bar_mma = bar_tma + 1;
    uint64_t *bar_y = bar_tma + 2;     // cluster of 4: Y^T is complete (the state leaves before y is stored)
    uint64_t *bar_dep = bar_tma + 3;   // used by the MMA-issuing thread alone, between dependent MMAs
    uint64_t *bar_state = bar_tma + 4; // K > 1: the previous CTA of the cluster has delivered the state
    unsigned char *lo_buf = tXU + 2048;   // K > 1: [64][64] bf16 residual of the delivered state (8 KB)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kOffMisc + 48);   // past the five barriers
    float *exp_cl = reinterpret_cast<float *>(smem + kOffMisc + 64);   // [2][64] exp(c_L), by chunk parity
    int *unsafe = reinterpret_cast<int *>(exp_cl + 128);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3;   // TMEM lane quarter this warp may read
    const int cgrp = warp >> 2;     // column group among the four warps of a quarter
    static_assert(!(SAVE && K > 1), "the cluster variant does not write the training tensors");
    // Cluster of 4: a CTA has three chunk periods of slack, so it also applies the block solve to the
    // identity ahead of time.  T = (I - A_ab)^-1 then sits in shared memory as one operand tile and
    // the state-dependent part of the solve shrinks from eight dependent MMA steps to one.
    constexpr bool kFullInv = (K == 4);
    const int rank = K > 1 ? (int)cluster_ctarank() : 0;
    const int bh = chain0 + blockIdx.x / K;   // a launch covers the chains chain0 .. chain0 + gridDim.x / K - 1
    const int bi = bh / H, h = bh % H;
    const int nchunks = (Tlen + kL - 1) / kL;

    if (tid == 0) {
        mbar_init(bar_tma, 1);
        mbar_init(bar_mma, 1);
        mbar_init(bar_y, 1);
        mbar_init(bar_dep, 1);
        mbar_init(bar_state, 1);   // armed by this CTA with the byte count of a delivered state
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
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    if constexpr (K > 1) cluster_sync_all();   // every CTA's barriers exist before anyone writes to a peer

    auto issue_tma = [&](int chunk) {
        mbar_expect_tx(bar_tma, kRawBytes);
        const int row = bi * Tlen + chunk * kL;
#pragma unroll
        for (int i = 0; i < 6; ++i) tma_load_2d(raw + i * (kL * kN * 2), &maps.m[i], h * kN, row, bar_tma);
    };
    if (tid == 0 && rank < nchunks) issue_tma(rank);

    // fp32 state: the thread at TMEM lane i (< 64), column group g holds S[i][16g .. 16g+15].
    const int zj = quarter * 32 + lane;  // value row i, meaningful for quarter < 2
    float Z[16];
    if (quarter < 2 && rank == 0) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s0) x = *reinterpret_cast<const float4 *>(s0 + ((size_t)bh * kN + zj) * kN + cgrp * 16 + 4 * q4);
            Z[4 * q4] = x.x; Z[4 * q4 + 1] = x.y; Z[4 * q4 + 2] = x.z; Z[4 * q4 + 3] = x.w;
            st_tile4(tS, 64, zj, cgrp * 16 + 4 * q4,
                     make_float4(round_tf32(x.x), round_tf32(x.y), round_tf32(x.z), round_tf32(x.w)));
        }
    }

    // K-step-0 descriptors of every operand tile (constant for the whole kernel).
    const uint64_t dAR = desc_kmajor(smem_u32(tAR), 128, 0), dBK = desc_kmajor(smem_u32(tBK), 128, 0),
                   dZT = desc_kmajor(smem_u32(tZT), 128, 0),
                   dS = desc_kmajor(smem_u32(tS), 64, 0), dVT = desc_kmajor(smem_u32(tVT), 64, 0),
                   dAKRK = desc_kmajor(smem_u32(tAKRK), 128, 0);
    constexpr uint64_t kLower = (64 * 128) >> 4;   // rows 64..127 of a stacked 128-row tile
    uint32_t mma_phase = 0, dep_phase = 0, state_phase = 0, y_phase = 0;
    // TMEM columns of the dS accumulator of token block b (the last one reuses G's, dead by then)
    auto ds_col = [](int b) -> uint32_t { return !SAVE ? kColDS : (b == 3 ? kColG : kColDS + 64u * (uint32_t)b); };
    float *exp_sub = reinterpret_cast<float *>(tXU + 2048);   // [3][64] exp(c_15), exp(c_31), exp(c_47); SAVE only
    bool failed = false;
    int tma_issued = 1, tma_consumed = 0;  // tile batches requested / received

    int iter = 0;   // chunks this CTA has started
    for (int chunk = rank; chunk < nchunks; chunk += K, ++iter) {
        const int valid = min(kL, Tlen - chunk * kL);
        if constexpr (K > 1) {
            // tf32 tile (16 KB) + bf16 residual (8 KB) will arrive from the previous CTA
            if (tid == 0 && chunk > 0) mbar_expect_tx(bar_state, kN * kN * 6);
        }
        // ---------------- wait for this chunk's six input tiles
        // A wait that expires sets a sticky flag; every thread sees it after the next
        // CTA barrier and leaves the loop there, so no extra barrier is spent on it.
        if (!mbar_wait(bar_tma, (uint32_t)(iter & 1))) atomicOr(unsafe, 2);
        ++tma_consumed;
        // ---------------- phase A: decay prefix sums and scaled operands
        if (valid < kL) {
            // Last, partial chunk: turn the rows past the end into no-op tokens
            // (w = -inf gives a log-decay of -0, every other vector is zero).
            for (int idx = tid; idx < (kL - valid) * kN; idx += kThreads) {
                const int t = valid + idx / kN, jj = idx % kN;
#pragma unroll
                for (int x = 0; x < 6; ++x)
                    *reinterpret_cast<unsigned short *>(raw + x * (kL * kN * 2) + (t * kN + jj) * 2) =
                        (x == TW) ? (unsigned short)0xFF80 : (unsigned short)0;
            }
            __syncthreads();
        }
        {
            const int j = tid & 63, tg = tid >> 6;  // channel, group of 8 tokens
            const int t0 = tg * 8;
            const unsigned char *rp = raw + (t0 * kN + j) * 2;
            auto ld = [&](int tensor, int u) {
                return __uint_as_float(
                    (unsigned)*reinterpret_cast<const unsigned short *>(rp + tensor * (kL * kN * 2) + u * (kN * 2)) << 16);
            };
            float c[8];
            float sum = 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                sum -= __expf(ld(TW, u));
                c[u] = sum;  // inclusive prefix inside this group
            }
            grp_tot[tg * 64 + j] = sum;
            __syncthreads();
            float base = 0.f, total = 0.f;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const float x = grp_tot[g * 64 + j];
                total += x;
                if (g < tg) base += x;
            }
            if (tg == 7) {
                exp_cl[(iter & 1) * 64 + j] = __expf(total);
                if (total < -kMaxLogDecay) atomicOr(unsafe, 1);
            }
            // Row t0 + u of a 128-row tile: t0 is a multiple of 8, so the swizzle term is u.
            const uint32_t cb = (uint32_t)(j & 31) * 4u;
            unsigned char *pAR = tAR + (j >> 5) * (128 * 128) + t0 * 128;
            unsigned char *pBK = tBK + (j >> 5) * (128 * 128) + t0 * 128;
            float e_prev = __expf(base);  // exp(c_{t0-1})
            float bhv[8], khv[8], vv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float e = __expf(base + c[u]);   // exp(c_t)
                float einv;                             // exp(-c_t)
                asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(einv) : "f"(e));
                vv[u] = ld(TV, u);                      // bf16 values are tf32-exact
                const float bh = ld(TB, u) * einv;
                bhv[u] = round_tf32(bh * kDebias);   // transposed copy: operand of dS += U^T Bh
                khv[u] = round_tf32(ld(TK, u) * einv);
                const uint32_t o = (uint32_t)u * 128u + (cb ^ ((uint32_t)u << 4));
                *reinterpret_cast<float *>(pAR + o) = round_tf32(ld(TA, u) * e_prev);
                *reinterpret_cast<float *>(pAR + 64 * 128 + o) = round_tf32(ld(TR, u) * e);
                *reinterpret_cast<float *>(pBK + o) = round_tf32(bh);
                *reinterpret_cast<float *>(pBK + 64 * 128 + o) = khv[u];
                e_prev = e;
            }
            if constexpr (SAVE) {
                if ((tg & 1) && tg < 7) exp_sub[(tg >> 1) * 64 + j] = e_prev;   // exp(c_t) at t = 15, 31, 47
            }
            // transposed copies: Bh^T, Kh^T [j][t] and V^T [i][s], 8 consecutive tokens per thread
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {
                st_tile4(tZT, 128, j, t0 + 4 * q4, make_float4(bhv[4 * q4], bhv[4 * q4 + 1], bhv[4 * q4 + 2], bhv[4 * q4 + 3]));
                st_tile4(tZT, 128, 64 + j, t0 + 4 * q4, make_float4(khv[4 * q4], khv[4 * q4 + 1], khv[4 * q4 + 2], khv[4 * q4 + 3]));
                st_tile4(tVT, 64, j, t0 + 4 * q4, make_float4(vv[4 * q4], vv[4 * q4 + 1], vv[4 * q4 + 2], vv[4 * q4 + 3]));
            }
        }
        if constexpr (SAVE || K == 1) {
            // the last snapshots have left the [A_ak;A_rk] tile, the last y tile its staging area
            if (tid == 0) bulk_wait_group_read<0>();
        }
        fence_proxy_async();
        __syncthreads();  // operands visible to the tensor core; raw tiles and group sums are dead
        // A cluster keeps going on a decay flag (its chain is recomputed afterwards anyway): a CTA
        // that left here would keep its successors waiting for a state.
        if (K > 1 ? (*unsafe & 2) : *unsafe) { failed = true; break; }
        // ---------------- M1: G = [At;Rt] [Bh;Kh]^T
        if (tid == 0) {
            tc_fence_after();
            mma_k64<128, 128, 128>(tmem + kColG, dAR, dBK, false);
            umma_commit(bar_mma);
            // State path, part 1: value-major products (M = value index i, 64 valid lanes) that
            // need only this chunk's scaled operands.  They run while G is read back below.
            if constexpr (K == 1) {
                mma_k64<64, 128, 128>(tmem + kColXT, dS, dAR, false);              // [X^T | Y^T] = S [At;Rt]^T
            }
            if constexpr (!SAVE) mma_k64<64, 128, 64>(tmem + kColDS, dVT, dZT + kLower, false);     // dS   = V^T Kh
        }
        if (!mbar_wait(bar_mma, mma_phase)) atomicOr(unsafe, 2);
        mma_phase ^= 1;
        tc_fence_after();
        // ---------------- hop 1: G -> masked A_ab (fp32 scratch), A_ak, A_rb, A_rk (tf32 tiles)
        {
            const bool upper = quarter >= 2;          // Rt rows: inclusive lower triangle
            const int t = (quarter & 1) * 32 + lane;
            const int lim = upper ? t : t - 1;        // keep s <= lim
            const int s_base = (cgrp & 1) * 32;       // column offset inside the 64-wide quadrant
            uint32_t v[32];
            tmem_ld32(tmem + lane_base + kColG + cgrp * 32, v);
            tmem_ld_wait();
            if (cgrp < 2 && !upper) {
                // A_ab: tf32 into rows 0..63 of the [T;A_rb] tile (its blocks below the block
                // diagonal are operands of the solve as they are), and the diagonal 16x16
                // block of this row in exact fp32 into the scratch of the block inverses.
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    float4 o;
                    float *of = &o.x;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int s = s_base + e4 * 4 + e;
                        v[e4 * 4 + e] = (s <= lim) ? v[e4 * 4 + e] : 0u;
                        of[e] = round_tf32(__uint_as_float(v[e4 * 4 + e]) * kDebias);
                    }
                    st_tile4(tBK, 128, t, s_base + e4 * 4, o);
                }
                const int rb = t >> 4;
                if ((rb >> 1) == (cgrp & 1)) {
                    const bool hi = rb & 1;
#pragma unroll
                    for (int e4 = 0; e4 < 4; ++e4)
                        *reinterpret_cast<uint4 *>(Am + t * kPitchA + e4 * 4) =
                            make_uint4(hi ? v[16 + e4 * 4] : v[e4 * 4], hi ? v[17 + e4 * 4] : v[e4 * 4 + 1],
                                       hi ? v[18 + e4 * 4] : v[e4 * 4 + 2], hi ? v[19 + e4 * 4] : v[e4 * 4 + 3]);
                    if (kBlk == 32 && hi) {   // A_10: this row against the even block of its pair
#pragma unroll
                        for (int e4 = 0; e4 < 4; ++e4)
                            *reinterpret_cast<uint4 *>(Am + t * kPitchA + 16 + e4 * 4) =
                                make_uint4(v[e4 * 4], v[e4 * 4 + 1], v[e4 * 4 + 2], v[e4 * 4 + 3]);
                    }
                }
            } else {
                unsigned char *dst = (cgrp < 2) ? tBK : tAKRK;   // A_rb under T, or [A_ak;A_rk]
                const float scale = (cgrp < 2) ? kDebias : 1.f;   // A_rb meets U^T read from TMEM
                const int row = upper ? 64 + t : t;
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    float4 o;
                    float *of = &o.x;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int s = s_base + e4 * 4 + e;
                        of[e] = (s <= lim) ? round_tf32(__uint_as_float(v[e4 * 4 + e]) * scale) : 0.f;
                    }
                    st_tile4(dst, 128, row, s_base + e4 * 4, o);
                }
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (K > 1 ? (*unsafe & 2) : *unsafe) { failed = true; break; }
        // ---------------- state path, part 2: the products with the masked A_ak, A_rk just
        // staged; they run on the tensor core while the diagonal blocks are inverted below.
        if (tid == 0) {
            tc_fence_after();
            // (K > 1: the state has not arrived yet, these products start the accumulators)
            mma_k64<64, 128, 128>(tmem + kColXT, dVT, dAKRK, K == 1);            // [X^T | Y^T] (+)= V^T [A_ak;A_rk]^T
            if constexpr (SAVE) {
#pragma unroll
                for (int b = 0; b < kL / 16; ++b)   // dS_b = V^T Kh over the 16 tokens of block b (G is dead now)
                    mma_kpair<64, 128, 64>(tmem + ds_col(b), dVT, dZT + kLower, 2 * b);
            }
            if constexpr (K == 1) umma_commit(bar_dep);   // K > 1: one commit after the products with the state
        }
        // ---------------- U = (I - A_ab)^-1 X is solved block-wise: only the diagonal blocks
        // T_bb = (I - A_bb)^-1 are formed here, the coupling between blocks is part of the MMA
        // chain below.  16 x 16 blocks by forward substitution in fp32 (one column per thread);
        // with 32-token solve blocks two of them are then joined by all threads,
        // [[T_00, 0], [T_11 A_10 T_00, T_11]], which halves the dependent steps of the chain.
        if (tid >= 64 && tid < 128) {   // warps 2 and 3: warp 0 is busy issuing
            const int b = (tid - 64) >> 4, cc = tid & 15;
            const float *Ab = Am + (16 * b) * kPitchA;
            float x[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int s4 = 0; s4 < (t + 3) / 4; ++s4) {
                    const float4 a4 = *reinterpret_cast<const float4 *>(Ab + t * kPitchA + 4 * s4);
                    if (4 * s4 + 0 < t) acc0 = fmaf(a4.x, x[4 * s4 + 0], acc0);
                    if (4 * s4 + 1 < t) acc1 = fmaf(a4.y, x[4 * s4 + 1], acc1);
                    if (4 * s4 + 2 < t) acc0 = fmaf(a4.z, x[4 * s4 + 2], acc0);
                    if (4 * s4 + 3 < t) acc1 = fmaf(a4.w, x[4 * s4 + 3], acc1);
                }
                x[t] = (t == cc) ? 1.f : ((t > cc) ? acc0 + acc1 : 0.f);
                *reinterpret_cast<float *>(tBK + tile_off_f32(128, 16 * b + t, 16 * b + cc)) = round_tf32(x[t] * kDebias);
                if constexpr (kBlk == 32) Tm[(16 * b + t) * kPitch + cc] = x[t];
            }
        }
        if constexpr (kBlk == 32) {
            // T_10 = T_11 (A_10 T_00) for the two pairs of blocks, one element per thread and product
            const int pr = tid >> 8, t = (tid >> 4) & 15, c = tid & 15;
            __syncthreads();
            {
                const float *arow = Am + (32 * pr + 16 + t) * kPitchA + 16;   // A_10[t][.]
                const float *tcol = Tm + (32 * pr) * kPitch + c;              // T_00[.][c]
                float w = 0.f;
#pragma unroll
                for (int s4 = 0; s4 < 4; ++s4) {
                    const float4 a4 = *reinterpret_cast<const float4 *>(arow + 4 * s4);
                    w = fmaf(a4.x, tcol[(4 * s4 + 0) * kPitch], w);
                    w = fmaf(a4.y, tcol[(4 * s4 + 1) * kPitch], w);
                    w = fmaf(a4.z, tcol[(4 * s4 + 2) * kPitch], w);
                    w = fmaf(a4.w, tcol[(4 * s4 + 3) * kPitch], w);
                }
                Wm[(16 * pr + t) * kPitch + c] = w;
            }
            __syncthreads();
            {
                const float *trow = Tm + (32 * pr + 16 + t) * kPitch;   // T_11[t][.] (zero right of the diagonal)
                const float *wcol = Wm + (16 * pr) * kPitch + c;
                float z = 0.f;
#pragma unroll
                for (int s4 = 0; s4 < 4; ++s4) {
                    const float4 a4 = *reinterpret_cast<const float4 *>(trow + 4 * s4);
                    z = fmaf(a4.x, wcol[(4 * s4 + 0) * kPitch], z);
                    z = fmaf(a4.y, wcol[(4 * s4 + 1) * kPitch], z);
                    z = fmaf(a4.z, wcol[(4 * s4 + 2) * kPitch], z);
                    z = fmaf(a4.w, wcol[(4 * s4 + 3) * kPitch], z);
                }
                *reinterpret_cast<float *>(tBK + tile_off_f32(128, 32 * pr + 16 + t, 32 * pr + c)) = round_tf32(z * kDebias);
            }
        }
        if constexpr (kFullInv) {
            if (tid >= 128) {   // identity tile for X^T := I, next to the scratch of the block inverses
                unsigned char *ident = smem + kOffIdent;
                for (int idx = tid - 128; idx < kN * kN / 4; idx += kThreads - 128) {
                    const int row = idx >> 4, c0 = (idx & 15) * 4;
                    st_tile4(ident, 64, row, c0,
                             make_float4(row == c0 ? 1.f : 0.f, row == c0 + 1 ? 1.f : 0.f, row == c0 + 2 ? 1.f : 0.f,
                                         row == c0 + 3 ? 1.f : 0.f));
                }
            }
        }
        fence_proxy_async();
        __syncthreads();  // scratch matrices are dead: the raw-tile region may be refilled
        if constexpr (!kFullInv) {
            if (chunk + K < nchunks) {
                if (tid == 32) issue_tma(chunk + K);   // not the thread that issues the MMAs
                ++tma_issued;
            }
        } else {
            // ---------------- T^T = I (I - A_ab)^-T by the same block substitution, before the state is
            // needed; the raw-tile region is refilled once the identity tile has been read.
            if (tid == 0) {
                auto dep_commit = [&]() { umma_commit(bar_dep); };
                auto dep_wait = [&]() {
                    if (!mbar_wait_spin(bar_dep, dep_phase)) atomicOr(unsafe, 2);
                    dep_phase ^= 1;
                    tc_fence_after();
                };
                tc_fence_after();
                const uint64_t dI = desc_kmajor(smem_u32(smem + kOffIdent), 64, 0);
                mma_k64<64, 64, 64>(tmem + kColTX, dI, dI, false);
                dep_commit();
                dep_wait();
                if (chunk + K < nchunks) issue_tma(chunk + K);
#pragma unroll
                for (int b = 0; b < kL / kBlk; ++b) {
                    if (b > 0) {
                        mma_ts_block<kBlk>(tmem + kColTX + b * kBlk, tmem + kColTT, dBK, b * kBlk, 0, b * kBlk / 8, true);
                        dep_commit();
                        dep_wait();
                    }
                    mma_ts_block<kBlk>(tmem + kColTT + b * kBlk, tmem + kColTX + b * kBlk, dBK, b * kBlk, b * kBlk,
                                       kBlk / 8, false);
                    if (b + 1 < kL / kBlk) {
                        dep_commit();
                        dep_wait();
                    }
                }
                umma_commit(bar_mma);
            }
            if (chunk + K < nchunks) ++tma_issued;
            __syncwarp();
            if (!mbar_wait(bar_mma, mma_phase)) atomicOr(unsafe, 2);
            mma_phase ^= 1;
            tc_fence_after();
            // T^T (lane s, column t) -> rows t of the [T;A_rb] tile, replacing A_ab and the block inverses.
            // No debias factor here: the identity is exact as a TMEM operand, so the factor carried by
            // the block inverses and by A_ab has come through once, which is what U^T = X^T T^T needs.
            if (quarter < 2) {
                uint32_t tv[16];
                tmem_ld16(tmem + lane_base + kColTT + cgrp * 16, tv);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    st_tile(tBK, 128, cgrp * 16 + e, zj, round_tf32(__uint_as_float(tv[e])));
            }
            fence_proxy_async();
            tc_fence_before();
            __syncthreads();
        }
        if constexpr (K > 1) {
            // ---------------- the state arrives from the previous CTA of the cluster (the very
            // first chunk of the chain starts from the initial state, staged above by rank 0)
            if (chunk > 0) {
                if (!mbar_wait_cluster(bar_state, state_phase)) atomicOr(unsafe, 2);
                state_phase ^= 1;
                if (quarter < 2) {   // fp32 state = delivered tf32 tile + bf16 residual
                    // (residual rows are 128 bytes; their 16-byte pieces are XOR-ed with the row so that the
                    // 32 rows of a warp do not meet in one bank)
                    const unsigned char *lo_row = lo_buf + zj * (kN * 2);
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const uint4 lo = *reinterpret_cast<const uint4 *>(lo_row + (((cgrp * 2 + h2) ^ (zj & 7)) << 4));
                        const unsigned l4[4] = {lo.x, lo.y, lo.z, lo.w};
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const int q4 = 2 * h2 + q;
                            const float4 hi = *reinterpret_cast<const float4 *>(tS + tile_off_f32(64, zj, cgrp * 16 + 4 * q4));
                            Z[4 * q4 + 0] = hi.x + __uint_as_float(l4[2 * q] << 16);
                            Z[4 * q4 + 1] = hi.y + __uint_as_float(l4[2 * q] & 0xffff0000u);
                            Z[4 * q4 + 2] = hi.z + __uint_as_float(l4[2 * q + 1] << 16);
                            Z[4 * q4 + 3] = hi.w + __uint_as_float(l4[2 * q + 1] & 0xffff0000u);
                        }
                    }
                }
            }
        }
        // ---------------- state path, part 3: the triangular solve and what depends on U.
        // X^T and U^T stay in TMEM and feed later MMAs as their A operand.  An MMA that
        // reads a TMEM operand written by an earlier MMA is ordered after it only through a
        // commit and a wait (MMAs with different accumulators are not guaranteed to execute
        // in issue order); MMAs that do not depend on the pending result are issued between
        // the commit and the wait so that the tensor core stays busy.
        if (tid == 0) {
            auto dep_commit = [&]() { umma_commit(bar_dep); };
            auto dep_wait = [&]() {
                if (!mbar_wait_spin(bar_dep, dep_phase)) atomicOr(unsafe, 2);
                dep_phase ^= 1;
                tc_fence_after();
            };
            auto leaves = [&](int b) {   // what U_b^T contributes to Y^T and dS
                mma_ts_block<64>(tmem + kColYT, tmem + kColUT + b * kBlk, dBK, 64, b * kBlk, kBlk / 8, true);   // A_rb
                if constexpr (SAVE && kBlk == 32) {   // the snapshots need the update per 16 tokens
                    mma_ts_block<64>(tmem + ds_col(2 * b), tmem + kColUT + b * kBlk, dZT, 0, b * kBlk, 2, true);
                    mma_ts_block<64>(tmem + ds_col(2 * b + 1), tmem + kColUT + b * kBlk + 16, dZT, 0, b * kBlk + 16, 2, true);
                } else {
                    mma_ts_block<64>(tmem + ds_col(b), tmem + kColUT + b * kBlk, dZT, 0, b * kBlk, kBlk / 8, true);    // Bh
                }
            };
            if constexpr (K > 1) {
                // (the state tile was written by a bulk copy, i.e. through the async proxy the tensor
                // core reads it with: no proxy fence is needed here)
                mma_k64<64, 128, 64>(tmem + kColXT, dS, dAR, true);               // X^T += S At^T
                dep_commit();   // completes after the products with V issued earlier, too
                mma_k64<64, 128, 64>(tmem + kColYT, dS, dAR + kLower, true);      // Y^T += S Rt^T (not needed by the solve)
            }
            dep_wait();   // parts 1 and 2 have finished: X^T is complete
            if constexpr (kFullInv) {
                mma_k64_ts<128, 64>(tmem + kColUT, tmem + kColXT, dBK, false);            // U^T = X^T T^T
                dep_commit();
                dep_wait();
                // the state update first: the next CTA waits for it, nobody waits for y
                mma_k64_ts<128, 64>(tmem + kColDS, tmem + kColUT, dZT, true);             // dS  += U^T Bh
                umma_commit(bar_mma);
                mma_k64_ts<128, 64>(tmem + kColYT, tmem + kColUT, dBK + kLower, true);    // Y^T += U^T A_rb^T
                umma_commit(bar_y);
            }
            // U^T = X^T (I - A_ab)^-T by block forward substitution over the token blocks b:
            // X_b^T += U_{<b}^T A_{b,<b}^T, then U_b^T = X_b^T T_bb^T.
#pragma unroll
            for (int b = 0; b < (kFullInv ? 0 : kL / kBlk); ++b) {
                if (b > 0) {
                    mma_ts_block<kBlk>(tmem + kColXT + b * kBlk, tmem + kColUT, dBK, b * kBlk, 0, b * kBlk / 8, true);
                    dep_commit();
                    leaves(b - 1);   // independent of the pending result
                    dep_wait();
                }
                mma_ts_block<kBlk>(tmem + kColUT + b * kBlk, tmem + kColXT + b * kBlk, dBK, b * kBlk, b * kBlk,
                                   kBlk / 8, false);
                dep_commit();
                dep_wait();
            }
            if constexpr (!kFullInv) {
                leaves(kL / kBlk - 1);
                umma_commit(bar_mma);
            }
        }
        // The other lanes of the issuing warp must not poll the barrier below while lane 0 is
        // still issuing: a suspended poll would stall lane 0's own waits between dependent MMAs.
        __syncwarp();
        if (!mbar_wait(bar_mma, mma_phase)) atomicOr(unsafe, 2);
        mma_phase ^= 1;
        tc_fence_after();
        // ---------------- hop: state update and y, by the 8 warps that own lanes 0..63
        if (quarter < 2) {
            uint32_t v[16];
            // SAVE: a snapshot leaves by TMA.  The thread's 16 values go into a staging tile in the
            // swizzled operand layout (the two halves of the [A_ak;A_rk] tile, dead during the hop, take
            // turns), and one thread stores the tile with two bulk tensor copies, which undo the swizzle.
            // Stored by the threads themselves a snapshot costs a warp 32 cache lines per instruction
            // (a thread owns 64 bytes of one row) and the hop 7.3 k cycles per chunk instead of 1.4 k.
            auto stage_put = [&](int m, const float (&x)[16]) {
                unsigned char *stage = tAKRK + (m & 1) * 16384;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    st_tile4(stage, 64, zj, cgrp * 16 + 4 * q4, make_float4(x[4 * q4], x[4 * q4 + 1], x[4 * q4 + 2], x[4 * q4 + 3]));
                fence_proxy_async();
                // the copy that read this tile two snapshots ago was waited for before the previous barrier
                if (tid == 0) bulk_wait_group_read<0>();
                asm volatile("bar.sync 2, 256;" ::: "memory");
            };
            auto stage_store = [&](int m, size_t snap_index) {   // snapshot number within [B*H*T/16]
                if (tid == 0) {
                    const unsigned char *stage = tAKRK + (m & 1) * 16384;
                    const int row0 = (int)(snap_index * kN);
                    tma_store_2d(&maps.snap, 0, row0, stage);
                    tma_store_2d(&maps.snap, 32, row0, stage + 8192);
                    bulk_commit_group();
                }
            };
            if constexpr (SAVE) {
                // v accumulates the blocks; after block m the state after token 16m+15 is known
                const size_t nsnap = (size_t)Tlen / 16;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    uint32_t w[16];
                    tmem_ld16(tmem + lane_base + ds_col(m) + cgrp * 16, w);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        v[e] = m == 0 ? w[e] : __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(w[e]));
                    if (m < 3 && 16 * (m + 1) <= valid) {
                        const float4 *e4 = reinterpret_cast<const float4 *>(exp_sub + m * 64 + cgrp * 16);
                        float sv[16];
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            const float4 g = e4[q4];
                            sv[4 * q4 + 0] = g.x * (Z[4 * q4 + 0] + __uint_as_float(v[4 * q4 + 0]));
                            sv[4 * q4 + 1] = g.y * (Z[4 * q4 + 1] + __uint_as_float(v[4 * q4 + 1]));
                            sv[4 * q4 + 2] = g.z * (Z[4 * q4 + 2] + __uint_as_float(v[4 * q4 + 2]));
                            sv[4 * q4 + 3] = g.w * (Z[4 * q4 + 3] + __uint_as_float(v[4 * q4 + 3]));
                        }
                        stage_put(m, sv);
                        stage_store(m, (size_t)bh * nsnap + (size_t)chunk * 4 + m);
                    }
                }
                uint32_t uv[16];   // U^T: this thread's value channel for tokens 16*cgrp .. +15
                tmem_ld16(tmem + lane_base + kColUT + cgrp * 16, uv);
                tmem_ld_wait();
                __nv_bfloat16 *sr = state_repl + (((size_t)bi * Tlen + chunk * kL + cgrp * 16) * H + h) * kN + zj;
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    if (cgrp * 16 + e < valid) sr[(size_t)e * H * kN] = __float2bfloat16_rn(__uint_as_float(uv[e]));
            } else {
                tmem_ld16(tmem + lane_base + kColDS + cgrp * 16, v);
            }
            uint32_t yv[16];
            if constexpr (!kFullInv) tmem_ld16(tmem + lane_base + kColYT + cgrp * 16, yv);
            tmem_ld_wait();
            const float4 *g4 = reinterpret_cast<const float4 *>(exp_cl + (iter & 1) * 64 + cgrp * 16);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const float4 g = g4[q4];
                Z[4 * q4 + 0] = g.x * (Z[4 * q4 + 0] + __uint_as_float(v[4 * q4 + 0]));
                Z[4 * q4 + 1] = g.y * (Z[4 * q4 + 1] + __uint_as_float(v[4 * q4 + 1]));
                Z[4 * q4 + 2] = g.z * (Z[4 * q4 + 2] + __uint_as_float(v[4 * q4 + 2]));
                Z[4 * q4 + 3] = g.w * (Z[4 * q4 + 3] + __uint_as_float(v[4 * q4 + 3]));
                if constexpr (K == 1)
                    st_tile4(tS, 64, zj, cgrp * 16 + 4 * q4,   // operand of the next chunk
                             make_float4(round_tf32(Z[4 * q4]), round_tf32(Z[4 * q4 + 1]), round_tf32(Z[4 * q4 + 2]),
                                         round_tf32(Z[4 * q4 + 3])));
            }
            if constexpr (SAVE) {
                if (valid == kL) {   // the state after the chunk's last token is its fourth snapshot
                    stage_put(3, Z);
                    stage_store(3, (size_t)bh * ((size_t)Tlen / 16) + (size_t)chunk * 4 + 3);
                }
            }
            if constexpr (K > 1) {
                // The state leaves as the tf32 operand tile plus the residual Z - tf32(Z) in bf16, staged
                // in this CTA's own (now idle) state tile and residual buffer and shipped below by two
                // bulk copies.  Nobody writes into these buffers before the copies have been consumed:
                // the state for this CTA's next chunk is produced by a chain of CTAs that starts at the
                // consumer of these very copies.
                unsigned lo[8];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    float hi[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) hi[e] = round_tf32(Z[4 * q4 + e]);
                    st_tile4(tS, 64, zj, cgrp * 16 + 4 * q4, make_float4(hi[0], hi[1], hi[2], hi[3]));
                    const __nv_bfloat162 l01 = __floats2bfloat162_rn(Z[4 * q4] - hi[0], Z[4 * q4 + 1] - hi[1]);
                    const __nv_bfloat162 l23 = __floats2bfloat162_rn(Z[4 * q4 + 2] - hi[2], Z[4 * q4 + 3] - hi[3]);
                    lo[2 * q4] = *reinterpret_cast<const unsigned *>(&l01);
                    lo[2 * q4 + 1] = *reinterpret_cast<const unsigned *>(&l23);
                }
                unsigned char *lo_row = lo_buf + zj * (kN * 2);   // 16-byte pieces XOR-ed with the row, as read above
                *reinterpret_cast<uint4 *>(lo_row + (((cgrp * 2) ^ (zj & 7)) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4 *>(lo_row + (((cgrp * 2 + 1) ^ (zj & 7)) << 4)) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                fence_proxy_async();   // the bulk copies read these buffers through the async proxy
                asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight warps that hold the state
                if (tid == 0 && chunk + 1 < nchunks) {
                    const uint32_t peer = (uint32_t)((rank + 1) % K);
                    const uint32_t peer_bar = map_to_cta(smem_u32(bar_state), peer);
                    bulk_copy_to_cta(map_to_cta(smem_u32(tS), peer), tS, kN * kN * 4, peer_bar);
                    bulk_copy_to_cta(map_to_cta(smem_u32(lo_buf), peer), lo_buf, kN * kN * 2, peer_bar);
                }
            }
            if constexpr (kFullInv) {   // Y^T was issued after the state update and completes here
                if (!mbar_wait(bar_y, y_phase)) atomicOr(unsafe, 2);
                tc_fence_after();
                tmem_ld16(tmem + lane_base + kColYT + cgrp * 16, yv);
                tmem_ld_wait();
            }
            // y[t][i]: this thread holds value channel i = zj for tokens 16*cgrp .. +15
            if (K == 1 && valid == kL) {
                __nv_bfloat16 *st = reinterpret_cast<__nv_bfloat16 *>(y_stage) + (cgrp * 16) * kN + zj;
#pragma unroll
                for (int e = 0; e < 16; ++e) st[e * kN] = __float2bfloat16_rn(__uint_as_float(yv[e]));
                fence_proxy_async();
                asm volatile("bar.sync 3, 256;" ::: "memory");   // the eight warps of the hop
                if (tid == 0) {
                    tma_store_2d(&maps.y, h * kN, bi * Tlen + chunk * kL, y_stage);
                    bulk_commit_group();
                }
            } else {
                __nv_bfloat16 *dst = y + (((size_t)bi * Tlen + chunk * kL + cgrp * 16) * H + h) * kN + zj;
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    if (cgrp * 16 + e < valid) dst[(size_t)e * H * kN] = __float2bfloat16_rn(__uint_as_float(yv[e]));
            }
        }
        if constexpr (kFullInv) y_phase ^= 1;
        // No CTA barrier here: the next chunk's phase A touches neither TMEM nor any
        // buffer this hop reads (exp(c_L) is kept per chunk parity), and its own
        // barriers come before the next MMA that overwrites the accumulators read above.
        tc_fence_before();
    }
    __syncthreads();
    if (*unsafe) failed = true;   // also catches a flag raised during the last chunk

    // ---------------- epilogue
    if constexpr (SAVE || K == 1) {
        if (tid == 0) bulk_wait_group<0>();   // snapshot / y copies still in flight read this CTA's shared memory
    }
    // A tile batch still in flight must land before the CTA gives up its shared memory.
    if (failed && tma_issued > tma_consumed) mbar_wait(bar_tma, (uint32_t)(tma_consumed & 1));
    const bool bad_decay = (*unsafe & 1) != 0;
    if (failed && !bad_decay && tid == 0) atomicExch(status, (int)kDevTimeout);
    if constexpr (K == 1) {
        if (tid == 0) flags[bh] = bad_decay ? 1 : 0;
    } else {
        if (tid == 0 && bad_decay) atomicOr(&flags[bh], 1);   // zeroed by the host before the launch
    }
    auto store_state = [&]() {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<float4 *>(s_out + ((size_t)bh * kN + zj) * kN + cgrp * 16 + 4 * q4) =
                make_float4(Z[4 * q4], Z[4 * q4 + 1], Z[4 * q4 + 2], Z[4 * q4 + 3]);
    };
    const bool owns_last = s_out != nullptr && quarter < 2 && (nchunks - 1) % K == rank;
    if constexpr (K == 1) {
        if (!failed && owns_last) store_state();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
    if constexpr (K > 1) {
        // No CTA of a cluster may exit while a peer can still write into its shared memory.
        cluster_sync_all();
        // The final state is written only if no CTA of the cluster flagged the chain: next_state may
        // alias initial_state, and the sequential recomputation of a flagged chain starts from
        // initial_state.  Every flag was OR-ed before the cluster barrier above (release / acquire at
        // cluster scope), so the value read back here is final.
        if (!failed && owns_last && atomicOr(&flags[bh], 0) == 0) store_state();
    }
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

// ---- scratch that lives in the library image ----------------------------------------
//
// The fallback flags of the chunked kernel (one int per (b,h) chain) can also be
// taken from this fixed array instead of a caller-provided workspace, for callers
// that may not allocate device memory when they call in.  Every GPU that loads
// the library holds the array (256 KiB) until the process exits.  In host code the
// array's name is only a stand-in: the device address is resolved per device with
// cudaGetSymbolAddress while that device is current.
constexpr int64_t kStaticScratchChains = 65536;
static __device__ __align__(256) int g_static_chain_flags[kStaticScratchChains];

int64_t wkv7_static_scratch_max_chains() { return kStaticScratchChains; }

// Resolves (once per device) and returns the device address of the static flag
// array.  `device` must be the current device of the calling thread.
int wkv7_static_scratch(int device, void **ptr, size_t *bytes) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int *cached[kMaxDevices] = {};
    if (device < 0 || device >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[device] == nullptr) {
        int current = -1;
        cudaError_t e = cudaGetDevice(&current);
        if (e != cudaSuccess) return (int)e;
        if (current != device) return (int)cudaErrorInvalidDevice;
        int *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_static_chain_flags);
        if (e != cudaSuccess) return (int)e;
        cached[device] = p;
    }
    *ptr = cached[device];
    *bytes = sizeof(int) * (size_t)kStaticScratchChains;
    return 0;
}

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

// 0 = choose by the number of chains, else the cluster size to use (1, 2 or 4).
std::atomic<int> g_cluster_override{0};
int wkv7_cluster_override() { return g_cluster_override.load(); }
void wkv7_set_cluster_override(int k) { g_cluster_override.store(k); }

// Number of SMs of `device` (0 if the query fails); queried once per device.
static int sm_count(int device) {
    constexpr int kMaxDevices = 64;
    static std::atomic<int> cached[kMaxDevices];
    if (device < 0 || device >= kMaxDevices) return 0;
    int n = cached[device].load();
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) n = -1;
        cached[device].store(n > 0 ? n : -1);
    }
    return n > 0 ? n : 0;
}

// How many clusters of `k` CTAs of the (one CTA per SM) chunked kernel can be resident on `device`;
// queried once per device and cluster size.
static int max_resident_clusters(int device, int k) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int cached[kMaxDevices][5] = {};
    if (device < 0 || device >= kMaxDevices || (k != 2 && k != 4)) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[device][k] == 0) {
        auto kern = k == 4 ? (const void *)wkv7_chunked_kernel<false, 4> : (const void *)wkv7_chunked_kernel<false, 2>;
        int n = 0;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(k * 64));
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = kSmemBytes;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)k;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
        }
        (void)cudaGetLastError();
        cached[device][k] = n > 0 ? n : -1;
    }
    return cached[device][k] > 0 ? cached[device][k] : 0;
}

int launch_wkv7_sequential_flagged_saved(const Wkv7Args &p, const int *flags, float *snapshots,
                                         void *state_replacement, int chunk_len, cudaStream_t stream);

static int launch_chunked_impl(const Wkv7Args &p, void *workspace, float *snapshots, void *state_replacement,
                               cudaStream_t stream, bool only_flagged = false) {
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
    {
        CUresult r = encode(&maps.y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.y, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    const bool save = snapshots != nullptr;
    std::memset(&maps.snap, 0, sizeof(maps.snap));
    if (save) {
        const int64_t snap_rows = p.B * p.H * (p.T / 16) * kN;
        // (TMA coordinates are 32-bit; larger problems take the sequential scan)
        if (snap_rows >= (int64_t(1) << 31) || (reinterpret_cast<uintptr_t>(snapshots) & 15u) != 0)
            return launch_wkv7_forward_saved(p, snapshots, state_replacement, 16, stream);
        const cuuint64_t sdims[2] = {(cuuint64_t)kN, (cuuint64_t)snap_rows};
        const cuuint64_t sstrides[1] = {(cuuint64_t)(kN * sizeof(float))};
        const cuuint32_t sbox[2] = {32, (cuuint32_t)kN};
        CUresult r = encode(&maps.snap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, snapshots, sdims, sstrides, sbox, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    int *status = nullptr;
    if (int e = device_status_ptr(p.device, &status)) return e;
    int *flags = static_cast<int *>(workspace);
    const int64_t chains = p.B * p.H;
    // Few chains: a cluster of CTAs per chain (needs at least one chunk per CTA to pay).
    // A cluster must fit one GPC, so fewer clusters are resident than SMs / K (on a 148-SM B200:
    // 74 of two, 33 of four): all chains of a cluster launch must be resident at once or it runs in waves.
    const int64_t nchunks = (p.T + kL - 1) / kL;
    auto cluster_for = [&](int64_t n) -> int {
        if (nchunks >= 8 && n <= max_resident_clusters(p.device, 4)) return 4;
        if (nchunks >= 4 && n <= max_resident_clusters(p.device, 2)) return 2;
        return 1;
    };
    // Launch plan: `head` chains with one CTA each, then `chains - head` chains with `cluster` CTAs each.
    // More chains than SMs run in waves of one CTA per SM; when the last wave would leave at least half
    // of the SMs idle, its chains form a second launch with a cluster per chain, which ends sooner.
    int cluster = 1;
    int64_t head = 0;
    if (!save && !only_flagged) {
        const int forced = wkv7_cluster_override();
        if (forced > 0) cluster = forced;
        else {
            cluster = cluster_for(chains);
            const int sms = sm_count(p.device);
            if (cluster == 1 && sms > 0 && chains > sms && chains % sms != 0) {
                const int tail = cluster_for(chains % sms);
                if (tail > 1) {
                    cluster = tail;
                    head = chains - chains % sms;
                }
            }
        }
    }
    cudaError_t e;
    auto launch = [&](auto kern, int k, int64_t first, int64_t count) -> cudaError_t {
        cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (err != cudaSuccess) return err;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(count * k));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)k;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = k > 1 ? 1 : 0;
        if (only_flagged) {   // behind the scan on the same stream: its launch may overlap the scan's tail
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.numAttrs = 1;
        }
        err = cudaLaunchKernelEx(&cfg, kern, maps, p.s0, reinterpret_cast<__nv_bfloat16 *>(p.y), p.s_out, flags,
                                 (int)p.T, (int)p.H, status, snapshots,
                                 reinterpret_cast<__nv_bfloat16 *>(state_replacement), (int)first,
                                 only_flagged ? 1 : 0);
        if (err == cudaSuccess) count_launch();
        return err;
    };
    if (cluster > 1) {   // CTAs of a cluster only ever set a flag
        e = cudaMemsetAsync(flags + head, 0, sizeof(int) * (size_t)(chains - head), stream);
        if (e != cudaSuccess) return (int)e;
    }
    if (save) e = launch(wkv7_chunked_kernel<true, 1>, 1, 0, chains);
    else {
        e = head > 0 ? launch(wkv7_chunked_kernel<false, 1>, 1, 0, head) : cudaSuccess;
        if (e != cudaSuccess) return (int)e;
        if (cluster == 4) e = launch(wkv7_chunked_kernel<false, 4>, 4, head, chains - head);
        else if (cluster == 2) e = launch(wkv7_chunked_kernel<false, 2>, 2, head, chains - head);
        else e = launch(wkv7_chunked_kernel<false, 1>, 1, head, chains - head);
    }
    if (e != cudaSuccess) return (int)e;
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    // Chains whose decay left the safe range are recomputed token by token; the
    // kernel exits at once for every chain that is not flagged.
    if (save) return launch_wkv7_sequential_flagged_saved(p, flags, snapshots, state_replacement, 16, stream);
    return launch_wkv7_sequential_flagged(p, flags, stream);
}

int launch_wkv7_chunked(const Wkv7Args &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    (void)workspace_bytes;
    return launch_chunked_impl(p, workspace, nullptr, nullptr, stream);
}

// The chains whose flag (first B*H ints of the workspace) is set, by the one-CTA kernel; chains it cannot
// resolve either stay flagged and go through the sequential scan.
int launch_wkv7_chunked_flagged(const Wkv7Args &p, void *workspace, cudaStream_t stream) {
    return launch_chunked_impl(p, workspace, nullptr, nullptr, stream, true);
}

// Training forward on the tensor cores: chunk_len 16, T a multiple of 16.
int launch_wkv7_chunked_saved(const Wkv7Args &p, void *workspace, float *snapshots, void *state_replacement,
                              cudaStream_t stream) {
    return launch_chunked_impl(p, workspace, snapshots, state_replacement, stream);
}

}  // namespace rwkv7
