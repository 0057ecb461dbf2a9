// WKV7 backward pass, time-parallel form (N = 64, bf16 tensors, chunk_len 16, T >= 64).
//
// Gradient definitions: the reference's wkv7_backward_kernel
// (crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/kernel.rs:395-690); with S_t the state after
// token t (S_{-1} the initial state), u_t = S_{t-1} a_t the saved state_replacement and
// d_t = exp(-exp(w_t)):
//     G_t  = Gh_t + dy_t r_t^T        (Gh_t: gradient of S_t from every later token; Gh_{T-1} = next_state_grad)
//     dr_t = S_t^T dy_t     dv_t = G_t k_t     dk_t = G_t^T v_t     db_t = G_t^T u_t
//     dsa_t = G_t b_t       da_t = S_{t-1}^T dsa_t      dd_t = colsum(G_t . S_{t-1})     dw_t = -exp(w_t) d_t dd_t
//     Gh_{t-1} = G_t diag(d_t) + dsa_t a_t^T            initial_state_grad = Gh_{-1}
//
// The reference walks the sequence backwards one token at a time (T dependent steps per chain).
// Here the only sequential part, the recurrence of Gh, is recognised as a *forward* WKV7
// recurrence over the reversed sequence,
//     Gh_{t-1} = Gh_t diag(d_t) + (Gh_t b_t) a_t^T + dy_t (r_t . d_t + (r_t.b_t) a_t)^T,
// i.e. the forward op with  w' = w_t, a' = b_t, b' = a_t, v' = dy_t, k' = r_t.d_t + (r_t.b_t) a_t,
// initial state next_state_grad; its state_replacement output is Gh_t b_t, its output with the
// receptance r' = k_{t-1} is Gh_{t-1} k_{t-1}, its snapshots are Gh at every 16th token and its
// final state is initial_state_grad.  So:
//   1. wkv7_bwd_prepare_kernel writes the six transformed, time-reversed tensors;
//   2. the tcgen05 prefill kernel (training variant) runs on them;
//   3. wkv7_bwd_local_kernel finishes every 16-token chunk independently of all others: it
//      replays S forwards from the forward snapshot at the chunk's start (elementwise, u_t being
//      saved) for dr and da, and Gh backwards from the snapshot of step 2 at the chunk's end
//      (elementwise, dsa_t being known) for dk and db.  dd needs S_{t-1} and G_t together; instead
//      of keeping either it follows from phi_t = colsum(Gh_t . S_t), known at the chunk's end:
//          d_t dd_t = phi_t - b_t db_t - k_t dk_t + r_t dr_t,     phi_{t-1} = d_t dd_t + a_t da_t
//      (both are identities of the two replays, exact up to fp32 rounding).
// Steps 1 and 3 are bandwidth / FMA-throughput kernels over B*H*T/16 independent units; step 2
// is the sequential part, on the tensor cores.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.h"

namespace rwkv7 {
namespace {

constexpr int kN = 64;
constexpr int kC = 16;   // chunk length (tokens between snapshots)

__device__ __forceinline__ float4 bf16x4_to_float4(uint2 p) {
    return make_float4(__uint_as_float(p.x << 16), __uint_as_float(p.x & 0xffff0000u), __uint_as_float(p.y << 16),
                       __uint_as_float(p.y & 0xffff0000u));
}
__device__ __forceinline__ uint2 float4_to_bf16x4(float4 f) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
    return make_uint2(*reinterpret_cast<const unsigned *>(&lo), *reinterpret_cast<const unsigned *>(&hi));
}
__device__ __forceinline__ float sum16(float x) {   // over the 16 lanes of a half warp
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// ---- step 1: transformed, time-reversed inputs of the gradient recurrence ------------------------
// 16 lanes per (b,t,h), four channels each.  Reversed index tau = T-1-t.
__global__ void __launch_bounds__(256)
wkv7_bwd_prepare_kernel(const uint2 *__restrict__ r, const uint2 *__restrict__ w, const uint2 *__restrict__ k,
                        const uint2 *__restrict__ a, const uint2 *__restrict__ b, const uint2 *__restrict__ dy,
                        uint2 *__restrict__ r_rev, uint2 *__restrict__ w_rev, uint2 *__restrict__ k_rev,
                        uint2 *__restrict__ v_rev, uint2 *__restrict__ a_rev, uint2 *__restrict__ b_rev,
                        long long B, long long T, long long H) {
    const long long unit = (long long)blockIdx.x * 16 + (threadIdx.x >> 4);   // (b*T + t)*H + h
    const int c4 = threadIdx.x & 15;
    if (unit >= B * T * H) return;   // never true for part of a warp: T is a multiple of 16
    const long long h = unit % H, bt = unit / H, t = bt % T, bi = bt / T;
    const size_t src = (size_t)unit * 16 + c4;
    const size_t dst = ((size_t)(bi * T + (T - 1 - t)) * H + h) * 16 + c4;
    const float4 rv = bf16x4_to_float4(r[src]), bv = bf16x4_to_float4(b[src]), av = bf16x4_to_float4(a[src]),
                 wv = bf16x4_to_float4(w[src]);
    const float rb = sum16(rv.x * bv.x + rv.y * bv.y + rv.z * bv.z + rv.w * bv.w);
    float4 kp;
    kp.x = rv.x * __expf(-__expf(wv.x)) + rb * av.x;
    kp.y = rv.y * __expf(-__expf(wv.y)) + rb * av.y;
    kp.z = rv.z * __expf(-__expf(wv.z)) + rb * av.z;
    kp.w = rv.w * __expf(-__expf(wv.w)) + rb * av.w;
    k_rev[dst] = float4_to_bf16x4(kp);
    w_rev[dst] = w[src];
    v_rev[dst] = dy[src];
    a_rev[dst] = b[src];
    b_rev[dst] = a[src];
    r_rev[dst] = t > 0 ? k[src - (size_t)H * 16] : make_uint2(0u, 0u);   // k_{t-1}
}

// ---- step 3: one 16-token chunk of one chain per CTA -------------------------------------------
struct LocalArgs {
    const __nv_bfloat16 *r, *w, *k, *v, *a, *b, *u, *dy;   // [B,T,H,64]
    const __nv_bfloat16 *sa_rev, *y_rev;                    // outputs of the reversed run, [B,T,H,64]
    const float *snapshots;        // forward: S after tokens 15, 31, ...   [B,H,T/16,64,64]
    const float *grad_snapshots;   // reversed run: state after 16, 32, ... reversed tokens
    const float *initial_state;    // or null (zero)
    const float *next_state_grad;  // or null (zero)
    __nv_bfloat16 *dr, *dw, *dk, *dv, *da, *db;
    int T, H;
};

enum { RU = 0, RV, RDY, RDSA, kRowVecs };          // vectors indexed by the value row i
enum { CD = 0, CR, CK, CA, CB, CEW, kColVecs };    // vectors indexed by the key column j
enum { ODR = 0, ODA, ODK, ODB, ODW, kOutVecs };

constexpr size_t kLocalSmemFloats = (size_t)(kRowVecs + kColVecs + kOutVecs) * kC * kN + 2 * kN;
constexpr int kLocalThreads = 256;

// Sums `acc` (two kinds x four columns) over the eight row groups of a warp (lane bits 2..4) so that
// every lane ends up with one total: kind = lane bit 4, column = 2 * bit 3 + bit 2.
__device__ __forceinline__ float reduce_scatter_rows(const float (&acc)[2][4], int lane) {
    float h4[4];
    const bool k1 = lane & 16;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float send = k1 ? acc[0][c] : acc[1][c];
        h4[c] = (k1 ? acc[1][c] : acc[0][c]) + __shfl_xor_sync(0xffffffffu, send, 16);
    }
    float h2[2];
    const bool c2 = lane & 8;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const float send = c2 ? h4[c] : h4[2 + c];
        h2[c] = (c2 ? h4[2 + c] : h4[c]) + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const bool c1 = lane & 4;
    const float send = c1 ? h2[0] : h2[1];
    return (c1 ? h2[1] : h2[0]) + __shfl_xor_sync(0xffffffffu, send, 4);
}

// 256 threads: warps 0..3 replay S forwards, warps 4..7 replay Gh backwards.  Within a pass a warp
// owns 16 key columns and a thread a block of 8 value rows x 4 key columns of the matrix
// (lane = column group + 4 * row group): a row-indexed vector element is then shared by four
// columns and a column-indexed one by eight rows, which keeps the shared-memory traffic (the bound
// of a one-column-per-thread layout) at a quarter.
__global__ void __launch_bounds__(kLocalThreads, 3) wkv7_bwd_local_kernel(LocalArgs p) {
    extern __shared__ __align__(16) float sm[];
    float *rowv = sm;                                     // [4][16][64]
    float *colv = rowv + kRowVecs * kC * kN;              // [6][16][64]
    float *outv = colv + kColVecs * kC * kN;              // [5][16][64]
    float *phi_end = outv + kOutVecs * kC * kN;           // [64]
    float *dv_last = phi_end + kN;                        // [64]  next_state_grad k_{T-1}

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = p.T / kC;
    const int q = blockIdx.x % nq, bh = blockIdx.x / nq;
    const int bi = bh / p.H, h = bh % p.H;
    const bool last_chunk = q == nq - 1;

    // ---- this thread's block of its pass's matrix
    const bool g_pass = warp >= 4;
    const int j0 = (warp & 3) * 16 + (lane & 3) * 4;   // first key column
    const int i0 = (lane >> 2) * 8;                    // first value row
    const float *s_src = (q == 0) ? p.initial_state : p.snapshots;
    const size_t s_off = (q == 0) ? (size_t)bh * kN * kN : ((size_t)bh * nq + (q - 1)) * kN * kN;
    const float *g_src = last_chunk ? p.next_state_grad : p.grad_snapshots;
    const size_t g_off = last_chunk ? (size_t)bh * kN * kN : ((size_t)bh * nq + (nq - q - 2)) * kN * kN;
    const float *msrc = g_pass ? g_src : s_src;
    const size_t moff = g_pass ? g_off : s_off;
    // Rows are held in pairs, M[rp][c] = (row 2 rp, row 2 rp + 1) of column c: the replays below use the
    // packed fp32 instructions of sm_100 (two FMAs per issue slot), and a pair of consecutive
    // elements of a row-indexed vector is what a 16-byte shared-memory load delivers.
    float2 M[4][4];
#pragma unroll
    for (int rp = 0; rp < 4; ++rp) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
        if (msrc != nullptr) {
            x = *reinterpret_cast<const float4 *>(msrc + moff + (size_t)(i0 + 2 * rp) * kN + j0);
            y = *reinterpret_cast<const float4 *>(msrc + moff + (size_t)(i0 + 2 * rp + 1) * kN + j0);
        }
        M[rp][0] = make_float2(x.x, y.x); M[rp][1] = make_float2(x.y, y.y);
        M[rp][2] = make_float2(x.z, y.z); M[rp][3] = make_float2(x.w, y.w);
    }

    // ---- prologue: the chunk's vectors, 16 lanes per token, four channels per lane
    const int tt = tid >> 4, c4 = tid & 15;
    const int t_glob = q * kC + tt;
    const size_t tok = ((size_t)bi * p.T + t_glob) * p.H + h;                      // token-head index
    const size_t tok_rev = ((size_t)bi * p.T + (p.T - 1 - t_glob)) * p.H + h;      // same token in the reversed tensors
    auto ld4 = [&](const __nv_bfloat16 *base, size_t th) {
        return bf16x4_to_float4(*reinterpret_cast<const uint2 *>(base + th * kN + 4 * c4));
    };
    float4 dvv;   // dv of (token tt, channels 4 c4 ..): Gh_t k_t + dy_t (r_t.k_t)
    {
        const float4 rv = ld4(p.r, tok), wv = ld4(p.w, tok), kv = ld4(p.k, tok), vv = ld4(p.v, tok), av = ld4(p.a, tok),
                     bv = ld4(p.b, tok), uv = ld4(p.u, tok), dyv = ld4(p.dy, tok), sav = ld4(p.sa_rev, tok_rev);
        // Gh_t k_t is the reversed run's output at reversed index T-2-t (the token after this one)
        float4 ghk = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t_glob < p.T - 1) ghk = ld4(p.y_rev, tok_rev - (size_t)p.H);
        const float rb = sum16(rv.x * bv.x + rv.y * bv.y + rv.z * bv.z + rv.w * bv.w);
        const float rk = sum16(rv.x * kv.x + rv.y * kv.y + rv.z * kv.z + rv.w * kv.w);
        const float4 ew = make_float4(__expf(wv.x), __expf(wv.y), __expf(wv.z), __expf(wv.w));
        const float4 dv4 = make_float4(__expf(-ew.x), __expf(-ew.y), __expf(-ew.z), __expf(-ew.w));
        auto colp = [&](int x) { return reinterpret_cast<float4 *>(colv + (x * kC + tt) * kN + 4 * c4); };
        *colp(CD) = dv4; *colp(CR) = rv; *colp(CK) = kv; *colp(CA) = av; *colp(CB) = bv; *colp(CEW) = ew;
        auto rowp = [&](int x) { return reinterpret_cast<float4 *>(rowv + (x * kC + tt) * kN + 4 * c4); };
        *rowp(RU) = uv; *rowp(RV) = vv; *rowp(RDY) = dyv;
        *rowp(RDSA) = make_float4(sav.x + dyv.x * rb, sav.y + dyv.y * rb, sav.z + dyv.z * rb, sav.w + dyv.w * rb);
        dvv = make_float4(ghk.x + dyv.x * rk, ghk.y + dyv.y * rk, ghk.z + dyv.z * rk, ghk.w + dyv.w * rk);
    }
    if (tid < kN) dv_last[tid] = 0.f;
    __syncthreads();

    // rows i0 + 4 half .. + 3 of a row-indexed vector, as two row pairs
    auto row4 = [&](int x, int t, int half, float2 (&o)[2]) {
        const float4 f = *reinterpret_cast<const float4 *>(rowv + (x * kC + t) * kN + i0 + 4 * half);
        o[0] = make_float2(f.x, f.y); o[1] = make_float2(f.z, f.w);
    };
    // columns j0 .. j0 + 3 of a column-indexed vector, each duplicated for the two rows of a pair
    auto col4 = [&](int x, int t, float2 (&o)[4]) {
        const float4 f = *reinterpret_cast<const float4 *>(colv + (x * kC + t) * kN + j0);
        o[0] = make_float2(f.x, f.x); o[1] = make_float2(f.y, f.y); o[2] = make_float2(f.z, f.z); o[3] = make_float2(f.w, f.w);
    };
    // where this lane's total of a reduce_scatter_rows lands
    const int out_kind = (lane >> 4) & 1;
    const int out_j = j0 + 2 * ((lane >> 3) & 1) + ((lane >> 2) & 1);

    if (!g_pass) {
        // ---- S-pass, forwards: da_t = S_{t-1}^T dsa_t, then the step, then dr_t = S_t^T dy_t
#pragma unroll 1
        for (int t = 0; t < kC; ++t) {
            float2 d[4], bb[4], kk[4];
            col4(CD, t, d); col4(CB, t, bb); col4(CK, t, kk);
            float2 acc_a[4] = {}, acc_r[4] = {};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float2 ds[2], uu[2], vv[2], yy[2];
                row4(RDSA, t, half, ds); row4(RU, t, half, uu); row4(RV, t, half, vv); row4(RDY, t, half, yy);
#pragma unroll
                for (int pr = 0; pr < 2; ++pr)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float2 s2 = M[2 * half + pr][c];
                        acc_a[c] = __ffma2_rn(s2, ds[pr], acc_a[c]);
                        s2 = __ffma2_rn(s2, d[c], __ffma2_rn(uu[pr], bb[c], __fmul2_rn(vv[pr], kk[c])));
                        acc_r[c] = __ffma2_rn(s2, yy[pr], acc_r[c]);
                        M[2 * half + pr][c] = s2;
                    }
            }
            float acc[2][4];   // [0]: da, [1]: dr
#pragma unroll
            for (int c = 0; c < 4; ++c) { acc[0][c] = acc_a[c].x + acc_a[c].y; acc[1][c] = acc_r[c].x + acc_r[c].y; }
            const float total = reduce_scatter_rows(acc, lane);
            outv[((out_kind ? ODR : ODA) * kC + t) * kN + out_j] = total;
        }
        // phi at the chunk's end: colsum(Gh_end . S_end)
        float phi[4] = {0.f, 0.f, 0.f, 0.f};
        if (g_src != nullptr) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float4 g = *reinterpret_cast<const float4 *>(g_src + g_off + (size_t)(i0 + r) * kN + j0);
                const float gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) phi[c] = fmaf(gg[c], (r & 1) ? M[r >> 1][c].y : M[r >> 1][c].x, phi[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) phi[c] += __shfl_xor_sync(0xffffffffu, phi[c], o);
        }
        if ((lane >> 2) == 0) *reinterpret_cast<float4 *>(phi_end + j0) = make_float4(phi[0], phi[1], phi[2], phi[3]);
    } else {
        // ---- G-pass, backwards: G_t = Gh_t + dy_t r_t^T, dk_t, db_t, then Gh_{t-1}
        if (last_chunk && p.next_state_grad != nullptr) {
            // the last token's dv also needs next_state_grad k_{T-1} (no later token produces it)
            float2 kk[4];
            col4(CK, kC - 1, kk);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                float x = 0.f;
#pragma unroll
                for (int c = 0; c < 4; ++c) x = fmaf((r & 1) ? M[r >> 1][c].y : M[r >> 1][c].x, kk[c].x, x);
                x += __shfl_xor_sync(0xffffffffu, x, 1);
                x += __shfl_xor_sync(0xffffffffu, x, 2);
                if ((lane & 3) == 0) atomicAdd(&dv_last[i0 + r], x);
            }
        }
#pragma unroll 1
        for (int t = kC - 1; t >= 0; --t) {
            float2 d[4], rr[4], aa[4];
            col4(CD, t, d); col4(CR, t, rr); col4(CA, t, aa);
            float2 acc_k[4] = {}, acc_b[4] = {};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float2 ds[2], uu[2], vv[2], yy[2];
                row4(RDSA, t, half, ds); row4(RU, t, half, uu); row4(RV, t, half, vv); row4(RDY, t, half, yy);
#pragma unroll
                for (int pr = 0; pr < 2; ++pr)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float2 g2 = __ffma2_rn(yy[pr], rr[c], M[2 * half + pr][c]);
                        acc_k[c] = __ffma2_rn(g2, vv[pr], acc_k[c]);
                        acc_b[c] = __ffma2_rn(g2, uu[pr], acc_b[c]);
                        M[2 * half + pr][c] = __ffma2_rn(g2, d[c], __fmul2_rn(ds[pr], aa[c]));
                    }
            }
            float acc[2][4];   // [0]: dk, [1]: db
#pragma unroll
            for (int c = 0; c < 4; ++c) { acc[0][c] = acc_k[c].x + acc_k[c].y; acc[1][c] = acc_b[c].x + acc_b[c].y; }
            const float total = reduce_scatter_rows(acc, lane);
            outv[((out_kind ? ODB : ODK) * kC + t) * kN + out_j] = total;
        }
    }
    __syncthreads();

    // ---- decay gradient.  With x_t = b_t db_t + k_t dk_t - r_t dr_t and z_t = x_t - a_t da_t the two
    // identities give phi_{t-1} = phi_t - z_t, so d_t dd_t = phi_end - sum_{s>t} z_s - x_t: a suffix sum
    // over the chunk, taken by every (token, four channels) thread for itself.
    auto st4 = [&](__nv_bfloat16 *base, float4 x) {
        *reinterpret_cast<uint2 *>(base + tok * kN + 4 * c4) = float4_to_bf16x4(x);
    };
    auto outp = [&](int x, int t) { return reinterpret_cast<float4 *>(outv + (x * kC + t) * kN + 4 * c4); };
    auto colq = [&](int x) { return *reinterpret_cast<const float4 *>(colv + (x * kC + tt) * kN + 4 * c4); };
    float4 xs;
    {
        const float4 gr = *outp(ODR, tt), ga = *outp(ODA, tt), gk = *outp(ODK, tt), gb = *outp(ODB, tt);
        const float4 rv = colq(CR), kv = colq(CK), av = colq(CA), bv = colq(CB);
        xs = make_float4(bv.x * gb.x + kv.x * gk.x - rv.x * gr.x, bv.y * gb.y + kv.y * gk.y - rv.y * gr.y,
                         bv.z * gb.z + kv.z * gk.z - rv.z * gr.z, bv.w * gb.w + kv.w * gk.w - rv.w * gr.w);
        *outp(ODW, tt) = make_float4(xs.x - av.x * ga.x, xs.y - av.y * ga.y, xs.z - av.z * ga.z, xs.w - av.w * ga.w);
        st4(p.dr, gr);
        st4(p.dk, gk);
        st4(p.da, ga);
        st4(p.db, gb);
    }
    __syncthreads();
    {
        float4 ph = *reinterpret_cast<const float4 *>(phi_end + 4 * c4);
#pragma unroll
        for (int s2 = kC - 1; s2 > 0; --s2) {
            if (s2 > tt) {
                const float4 z = *outp(ODW, s2);
                ph.x -= z.x; ph.y -= z.y; ph.z -= z.z; ph.w -= z.w;
            }
        }
        const float4 ew = colq(CEW);
        st4(p.dw, make_float4(-ew.x * (ph.x - xs.x), -ew.y * (ph.y - xs.y), -ew.z * (ph.z - xs.z), -ew.w * (ph.w - xs.w)));
    }
    if (last_chunk && tt == kC - 1) {
        const float4 x = *reinterpret_cast<const float4 *>(dv_last + 4 * c4);
        dvv = make_float4(dvv.x + x.x, dvv.y + x.y, dvv.z + x.z, dvv.w + x.w);
    }
    st4(p.dv, dvv);
}

}  // namespace

bool wkv7_backward_parallel_supported(const Wkv7BackwardArgs &p) {
    // The reversed run is the TMA prefill kernel (32-bit row coordinates): B*T >= 2^31 takes the
    // token-by-token kernel.  (Pointer alignment is a host-side contract of every entry point.)
    return p.bf16 && p.N == kN && p.chunk_len == kC && p.T >= 64 && p.T % kC == 0 &&
           p.B * p.T < (int64_t(1) << 31);
}

// Workspace: six reversed tensors, the reversed run's two outputs (bf16 [B,T,H,64] each), its
// snapshots (fp32 [B,H,T/16,64,64]) and the prefill kernel's own workspace.
size_t wkv7_backward_parallel_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N) {
    if (N != kN || T % kC != 0) return 0;
    const size_t seq = ((size_t)(B * T * H * N) * 2 + 255) / 256 * 256;
    const size_t snaps = (size_t)(B * H * (T / kC)) * kN * kN * sizeof(float);
    return 8 * seq + snaps + (wkv7_chunked_workspace_bytes(B, T, H, N) + 255) / 256 * 256;
}

int launch_wkv7_backward_parallel(const Wkv7BackwardArgs &p, void *workspace, int device, int num_sms,
                                  cudaStream_t stream) {
    if (p.B * p.H == 0 || p.T == 0) return 0;
    const size_t seq = ((size_t)(p.B * p.T * p.H * p.N) * 2 + 255) / 256 * 256;
    const size_t snaps = (size_t)(p.B * p.H * (p.T / kC)) * kN * kN * sizeof(float);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    void *rev[6];
    for (int i = 0; i < 6; ++i) rev[i] = ws + (size_t)i * seq;
    __nv_bfloat16 *y_rev = reinterpret_cast<__nv_bfloat16 *>(ws + 6 * seq);
    __nv_bfloat16 *sa_rev = reinterpret_cast<__nv_bfloat16 *>(ws + 7 * seq);
    float *gsnap = reinterpret_cast<float *>(ws + 8 * seq);
    void *chunked_ws = ws + 8 * seq + snaps;

    // 1. transformed, reversed inputs
    const long long units = (long long)(p.B * p.T * p.H);
    wkv7_bwd_prepare_kernel<<<(unsigned)((units + 15) / 16), 256, 0, stream>>>(
        static_cast<const uint2 *>(p.r), static_cast<const uint2 *>(p.w), static_cast<const uint2 *>(p.k),
        static_cast<const uint2 *>(p.a), static_cast<const uint2 *>(p.b), static_cast<const uint2 *>(p.output_grad),
        static_cast<uint2 *>(rev[0]), static_cast<uint2 *>(rev[1]), static_cast<uint2 *>(rev[2]),
        static_cast<uint2 *>(rev[3]), static_cast<uint2 *>(rev[4]), static_cast<uint2 *>(rev[5]), (long long)p.B,
        (long long)p.T, (long long)p.H);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;

    // 2. the gradient recurrence, as a forward pass over the reversed sequence
    Wkv7Args f{};
    f.r = rev[0]; f.w = rev[1]; f.k = rev[2]; f.v = rev[3]; f.a = rev[4]; f.b = rev[5];
    f.s0 = p.next_state_grad;
    f.y = y_rev;
    f.s_out = p.initial_state_grad;
    f.B = p.B; f.T = p.T; f.H = p.H; f.N = p.N;
    f.bf16 = true;
    f.device = device;
    f.num_sms = num_sms;
    if (int err = launch_wkv7_chunked_saved(f, chunked_ws, gsnap, sa_rev, stream)) return err;

    // 3. every chunk on its own
    LocalArgs l{};
    l.r = static_cast<const __nv_bfloat16 *>(p.r); l.w = static_cast<const __nv_bfloat16 *>(p.w);
    l.k = static_cast<const __nv_bfloat16 *>(p.k); l.v = static_cast<const __nv_bfloat16 *>(p.v);
    l.a = static_cast<const __nv_bfloat16 *>(p.a); l.b = static_cast<const __nv_bfloat16 *>(p.b);
    l.u = static_cast<const __nv_bfloat16 *>(p.state_replacement);
    l.dy = static_cast<const __nv_bfloat16 *>(p.output_grad);
    l.sa_rev = sa_rev; l.y_rev = y_rev;
    l.snapshots = p.snapshots; l.grad_snapshots = gsnap;
    l.initial_state = p.initial_state; l.next_state_grad = p.next_state_grad;
    l.dr = static_cast<__nv_bfloat16 *>(p.receptance_grad); l.dw = static_cast<__nv_bfloat16 *>(p.weight_decay_grad);
    l.dk = static_cast<__nv_bfloat16 *>(p.replacement_key_grad); l.dv = static_cast<__nv_bfloat16 *>(p.value_grad);
    l.da = static_cast<__nv_bfloat16 *>(p.removal_key_normalized_grad); l.db = static_cast<__nv_bfloat16 *>(p.replacement_grad);
    l.T = (int)p.T; l.H = (int)p.H;
    const size_t smem = kLocalSmemFloats * sizeof(float);
    e = cudaFuncSetAttribute(wkv7_bwd_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    wkv7_bwd_local_kernel<<<(unsigned)(p.B * p.H * (p.T / kC)), kLocalThreads, smem, stream>>>(l);
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace rwkv7
