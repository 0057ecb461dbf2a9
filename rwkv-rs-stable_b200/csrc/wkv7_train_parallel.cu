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
constexpr int kRowPitch = 72;   // floats per row vector: the upper 32 rows start 4 floats later (bank spread)
__device__ __forceinline__ int row_slot(int i) { return i + ((i >> 5) << 2); }

constexpr size_t kLocalSmemFloats = (size_t)kRowVecs * kC * kRowPitch + (size_t)(kColVecs + kOutVecs) * kC * kN + 2 * kN;
constexpr int kLocalThreads = 256;

__global__ void __launch_bounds__(kLocalThreads, 3) wkv7_bwd_local_kernel(LocalArgs p) {
    extern __shared__ __align__(16) float sm[];
    float *rowv = sm;                                     // [4][16][72]
    float *colv = rowv + kRowVecs * kC * kRowPitch;       // [6][16][64]
    float *outv = colv + kColVecs * kC * kN;              // [5][16][64]
    float *phi_end = outv + kOutVecs * kC * kN;           // [64]
    float *dv_last = phi_end + kN;                        // [64]  next_state_grad k_{T-1}

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = p.T / kC;
    const int q = blockIdx.x % nq, bh = blockIdx.x / nq;
    const int bi = bh / p.H, h = bh % p.H;
    const bool last_chunk = q == nq - 1;

    // ---- this thread's matrix column: S-pass warps 0..3, G-pass warps 4..7
    const bool g_pass = warp >= 4;
    const int j = (warp & 3) * 16 + (lane & 15);   // key column
    const int rh = lane >> 4;                      // row half
    const float *msrc;
    if (!g_pass) msrc = q == 0 ? p.initial_state + (p.initial_state ? (size_t)bh * kN * kN : 0)
                               : p.snapshots + ((size_t)bh * nq + (q - 1)) * kN * kN;
    else msrc = last_chunk ? p.next_state_grad + (p.next_state_grad ? (size_t)bh * kN * kN : 0)
                           : p.grad_snapshots + ((size_t)bh * nq + (nq - q - 2)) * kN * kN;
    const bool mzero = !g_pass ? (q == 0 && p.initial_state == nullptr) : (last_chunk && p.next_state_grad == nullptr);
    float M[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) M[i] = mzero ? 0.f : msrc[(size_t)(32 * rh + i) * kN + j];

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
        auto rowp = [&](int x) { return reinterpret_cast<float4 *>(rowv + (x * kC + tt) * kRowPitch + row_slot(4 * c4)); };
        *rowp(RU) = uv; *rowp(RV) = vv; *rowp(RDY) = dyv;
        *rowp(RDSA) = make_float4(sav.x + dyv.x * rb, sav.y + dyv.y * rb, sav.z + dyv.z * rb, sav.w + dyv.w * rb);
        dvv = make_float4(ghk.x + dyv.x * rk, ghk.y + dyv.y * rk, ghk.z + dyv.z * rk, ghk.w + dyv.w * rk);
    }
    if (tid < kN) dv_last[tid] = 0.f;
    __syncthreads();

    const float *rbase = rowv + row_slot(32 * rh);
    if (!g_pass) {
        // ---- S-pass, forwards: da_t = S_{t-1}^T dsa_t, then the step, then dr_t = S_t^T dy_t
#pragma unroll 1
        for (int t = 0; t < kC; ++t) {
            const float dj = colv[(CD * kC + t) * kN + j], bj = colv[(CB * kC + t) * kN + j], kj = colv[(CK * kC + t) * kN + j];
            float acc_a = 0.f, acc_r = 0.f;
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const float4 ds = *reinterpret_cast<const float4 *>(rbase + (RDSA * kC + t) * kRowPitch + 4 * m);
                const float4 u4 = *reinterpret_cast<const float4 *>(rbase + (RU * kC + t) * kRowPitch + 4 * m);
                const float4 v4 = *reinterpret_cast<const float4 *>(rbase + (RV * kC + t) * kRowPitch + 4 * m);
                const float4 y4 = *reinterpret_cast<const float4 *>(rbase + (RDY * kC + t) * kRowPitch + 4 * m);
                const float dsv[4] = {ds.x, ds.y, ds.z, ds.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w},
                            vv[4] = {v4.x, v4.y, v4.z, v4.w}, yy[4] = {y4.x, y4.y, y4.z, y4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float s = M[4 * m + e];
                    acc_a = fmaf(s, dsv[e], acc_a);
                    s = fmaf(s, dj, fmaf(uu[e], bj, vv[e] * kj));
                    acc_r = fmaf(s, yy[e], acc_r);
                    M[4 * m + e] = s;
                }
            }
            acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 16);
            acc_r += __shfl_xor_sync(0xffffffffu, acc_r, 16);
            if (rh == 0) outv[(ODA * kC + t) * kN + j] = acc_a;
            else outv[(ODR * kC + t) * kN + j] = acc_r;
        }
        // phi at the chunk's end: colsum(Gh_end . S_end)
        const float *gsrc = last_chunk ? p.next_state_grad + (p.next_state_grad ? (size_t)bh * kN * kN : 0)
                                       : p.grad_snapshots + ((size_t)bh * nq + (nq - q - 2)) * kN * kN;
        float phi = 0.f;
        if (!(last_chunk && p.next_state_grad == nullptr)) {
#pragma unroll
            for (int i = 0; i < 32; ++i) phi = fmaf(gsrc[(size_t)(32 * rh + i) * kN + j], M[i], phi);
        }
        phi += __shfl_xor_sync(0xffffffffu, phi, 16);
        if (rh == 0) phi_end[j] = phi;
    } else {
        // ---- G-pass, backwards: G_t = Gh_t + dy_t r_t^T, dk_t, db_t, then Gh_{t-1}
        if (last_chunk && p.next_state_grad != nullptr) {
            // the last token's dv also needs next_state_grad k_{T-1} (no later token produces it)
            const float kj = colv[(CK * kC + kC - 1) * kN + j];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float x = sum16(M[i] * kj);
                if ((lane & 15) == 0) atomicAdd(&dv_last[32 * rh + i], x);
            }
        }
#pragma unroll 1
        for (int t = kC - 1; t >= 0; --t) {
            const float dj = colv[(CD * kC + t) * kN + j], rj = colv[(CR * kC + t) * kN + j], aj = colv[(CA * kC + t) * kN + j];
            float acc_k = 0.f, acc_b = 0.f;
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const float4 ds = *reinterpret_cast<const float4 *>(rbase + (RDSA * kC + t) * kRowPitch + 4 * m);
                const float4 u4 = *reinterpret_cast<const float4 *>(rbase + (RU * kC + t) * kRowPitch + 4 * m);
                const float4 v4 = *reinterpret_cast<const float4 *>(rbase + (RV * kC + t) * kRowPitch + 4 * m);
                const float4 y4 = *reinterpret_cast<const float4 *>(rbase + (RDY * kC + t) * kRowPitch + 4 * m);
                const float dsv[4] = {ds.x, ds.y, ds.z, ds.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w},
                            vv[4] = {v4.x, v4.y, v4.z, v4.w}, yy[4] = {y4.x, y4.y, y4.z, y4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float g = fmaf(yy[e], rj, M[4 * m + e]);
                    acc_k = fmaf(g, vv[e], acc_k);
                    acc_b = fmaf(g, uu[e], acc_b);
                    M[4 * m + e] = fmaf(g, dj, dsv[e] * aj);
                }
            }
            acc_k += __shfl_xor_sync(0xffffffffu, acc_k, 16);
            acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 16);
            if (rh == 0) outv[(ODK * kC + t) * kN + j] = acc_k;
            else outv[(ODB * kC + t) * kN + j] = acc_b;
        }
    }
    __syncthreads();

    // ---- decay gradient: d_t dd_t from phi, one channel per thread
    if (tid < kN) {
        float phi = phi_end[tid];
#pragma unroll 1
        for (int t = kC - 1; t >= 0; --t) {
            const int o = t * kN + tid;
            const float ddd = phi - colv[CB * kC * kN + o] * outv[ODB * kC * kN + o] - colv[CK * kC * kN + o] * outv[ODK * kC * kN + o] +
                              colv[CR * kC * kN + o] * outv[ODR * kC * kN + o];
            outv[ODW * kC * kN + o] = -colv[CEW * kC * kN + o] * ddd;
            phi = fmaf(colv[CA * kC * kN + o], outv[ODA * kC * kN + o], ddd);
        }
    }
    __syncthreads();

    // ---- gradients of (token tt, channels 4 c4 ..) leave as bf16
    auto st4 = [&](__nv_bfloat16 *base, float4 x) {
        *reinterpret_cast<uint2 *>(base + tok * kN + 4 * c4) = float4_to_bf16x4(x);
    };
    auto outp = [&](int x) { return *reinterpret_cast<const float4 *>(outv + (x * kC + tt) * kN + 4 * c4); };
    st4(p.dr, outp(ODR));
    st4(p.dw, outp(ODW));
    st4(p.dk, outp(ODK));
    st4(p.da, outp(ODA));
    st4(p.db, outp(ODB));
    if (last_chunk && tt == kC - 1) {
        const float4 x = *reinterpret_cast<const float4 *>(dv_last + 4 * c4);
        dvv = make_float4(dvv.x + x.x, dvv.y + x.y, dvv.z + x.z, dvv.w + x.w);
    }
    st4(p.dv, dvv);
}

}  // namespace

bool wkv7_backward_parallel_supported(const Wkv7BackwardArgs &p) {
    return p.bf16 && p.N == kN && p.chunk_len == kC && p.T >= 64 && p.T % kC == 0;
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
