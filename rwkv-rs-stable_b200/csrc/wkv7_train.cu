// WKV7 backward pass for sm_100a (any head size N <= 64).
//
// Semantics: the reference's wkv7_backward_kernel
// (crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/kernel.rs:395-690), i.e. reverse-mode
// differentiation of   sa = S a;  S' = S diag(d) + sa b^T + v k^T;  y = S' r,  d = exp(-exp(w)):
//     dS += dy r^T                 dr = S'^T dy
//     dd  = colsum(dS . S)         dw = dd * (-exp(w) d)      dk = dS^T v    db = dS^T sa
//     dv  = dS k                   dsa = dS b                 da = S^T dsa
//     dS  = dS diag(d) + dsa a^T
// with dS starting from next_state_grad and ending as initial_state_grad.
//
// The state S before each token.  The reference rebuilds it going backwards,
// S = (S' - v k^T - sa b^T) diag(1/d) (kernel.rs:516-521), restarting from a saved snapshot
// every chunk_len tokens.  That divides by the decay once per token, and a rounding error made
// at one token is multiplied by every 1/d after it: with the reference's own test inputs
// (w in [0,1), d down to 0.066) the rebuilt state is wrong by orders of magnitude after a few
// tokens.  Here no division happens: since sa_t is saved, the forward step is elementwise,
// S' = S diag(d) + sa b^T + v k^T, so each chunk is replayed forwards from the snapshot at its
// start (or from the initial state), keeping the state before every 4th token, and each group
// of 4 tokens is replayed once more just before it is differentiated.  Same results as the
// reference's formula wherever that formula is stable; exact gradients where it is not.
//
// Where the reference keeps its N x N work matrices in global memory and gives every row to
// one thread, here all of them (S^T at 8 points of the chunk, dS, dS^T) live in shared memory,
// four threads share a row (every reduction above is then a row sum finished by two shuffles:
// both orientations of dS are kept so that column sums never occur; a thread only ever touches
// its own elements of the state copies, so replaying needs no barrier), and the nine per-token
// vectors of a whole chunk are staged in shared memory at once.  One CTA per (b,h) chain; fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels.h"

namespace rwkv7 {
namespace {

template <typename T>
__device__ __forceinline__ float ld(const void *p, size_t i) {
    return static_cast<float>(reinterpret_cast<const T *>(p)[i]);
}
template <typename T>
__device__ __forceinline__ void st(void *p, size_t i, float x) {
    if constexpr (sizeof(T) == 4) reinterpret_cast<float *>(p)[i] = x;
    else reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(x);
}

template <int LANES>
__device__ __forceinline__ float row_sum(float x) {
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}

enum { VR = 0, VD, VK, VV, VA, VB, VSA, VDY, VEW, kVecs };   // VD = decay, VEW = exp(w)
enum { OR_ = 0, OW, OK_, OB, OV, kOuts };
#ifndef RWKV7_BWD_ROWS
#define RWKV7_BWD_ROWS 2
#endif
#ifndef RWKV7_BWD_COLS
#define RWKV7_BWD_COLS 4
#endif
constexpr int kGroup = 4;         // tokens between kept states
constexpr int kMaxChunk = 16;     // chunk_len supported by the staging buffers
constexpr int kStates = kMaxChunk / kGroup + (kGroup - 1) + 1;   // checkpoints, in-group states, S after the chunk

template <typename T>
__global__ void wkv7_backward_kernel(Wkv7BackwardArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int N = (int)p.N, P = N + 4;   // row pitch: the four threads of 8 rows hit 32 different banks
    const size_t M = (size_t)N * P;
    float *states = reinterpret_cast<float *>(smem_raw);   // kStates copies of S^T [j][i]
    float *dS = states + kStates * M;                      // dS   [i][j]
    float *dSt = dS + M;                                   // dS^T [j][i]
    float *vec = dSt + M;                                  // [chunk_len][kVecs][N]
    float *dsa = vec + (size_t)kMaxChunk * kVecs * N;      // [N]
    float *outs = dsa + N;                                 // [kOuts][N]
    float *ckpt = states;                                  // [chunk_len / kGroup]: state before token kGroup * g
    float *grp = states + (kMaxChunk / kGroup) * M;        // [kGroup - 1]: states before the other tokens of a group
    float *s_end = grp + (kGroup - 1) * M;                 // state after the last token of the chunk

    const int bh = blockIdx.x, bi = bh / (int)p.H, h = bh % (int)p.H;
    const int tid = threadIdx.x, row = tid >> 2, q = tid & 3;
    const bool live = row < N;
    // Threads past the last row (4N is rounded up to whole warps) run the same code with empty
    // loops, so that every shuffle is executed by the whole warp.
    const int rr = live ? row : 0, n_cols = live ? N : 0;
    const int Tlen = (int)p.T, chunk_len = (int)p.chunk_len, nchunks = Tlen / chunk_len;
    const size_t tok_stride = (size_t)p.H * N;
    const size_t seq_base = ((size_t)bi * Tlen * p.H + h) * N;
    const size_t state_base = (size_t)bh * N * N;

    for (int idx = tid; idx < N * N; idx += blockDim.x) {
        const int i = idx / N, j = idx % N;
        const float g = p.next_state_grad ? p.next_state_grad[state_base + idx] : 0.f;
        dS[i * P + j] = g;
        dSt[j * P + i] = g;
    }

    // One forward step on this thread's elements of row j = rr of a transposed state:
    // dst[j][c] = src[j][c] d[j] + b[j] sa[c] + k[j] v[c].
    auto replay = [&](const float *src, float *dst, const float *v_t) {
        const float d_j = v_t[VD * N + rr], b_j = v_t[VB * N + rr], k_j = v_t[VK * N + rr];
        for (int c = q; c < n_cols; c += 4)
            dst[rr * P + c] = fmaf(src[rr * P + c], d_j, fmaf(b_j, v_t[VSA * N + c], k_j * v_t[VV * N + c]));
    };

    for (int chunk = nchunks - 1; chunk >= 0; --chunk) {
        const int t0 = chunk * chunk_len;
        // ---- stage the nine vectors of every token of the chunk, and the state at its start
        for (int idx = tid; idx < chunk_len * 8 * N; idx += blockDim.x) {
            const int j = idx % N, tensor = (idx / N) % 8, tt = idx / (8 * N);
            const void *src = tensor == VR ? p.r : tensor == VD ? p.w : tensor == VK ? p.k : tensor == VV ? p.v
                            : tensor == VA ? p.a : tensor == VB ? p.b : tensor == VSA ? p.state_replacement
                                                                                     : p.output_grad;
            float x = ld<T>(src, seq_base + (size_t)(t0 + tt) * tok_stride + j);
            float *v_t = vec + (size_t)tt * kVecs * N;
            if (tensor == VD) {
                const float ew = expf(x);
                v_t[VEW * N + j] = ew;
                x = expf(-ew);
            }
            v_t[tensor * N + j] = x;
        }
        {
            const float *start = chunk > 0 ? p.snapshots + ((size_t)bh * nchunks + chunk - 1) * N * N
                                           : (p.initial_state ? p.initial_state + state_base : nullptr);
            for (int idx = tid; idx < N * N; idx += blockDim.x)
                ckpt[(idx % N) * P + idx / N] = start ? start[idx] : 0.f;
        }
        __syncthreads();
        // ---- replay the chunk forwards, keeping the state before every kGroup-th token
        {
            const float *cur = ckpt;   // state before token 0 of the chunk
            for (int tt = 0; tt < chunk_len; ++tt) {
                float *dst = (tt + 1 == chunk_len) ? s_end
                             : ((tt + 1) % kGroup == 0) ? ckpt + (size_t)((tt + 1) / kGroup) * M
                                                        : grp + (size_t)(tt % kGroup) * M;   // scratch, rebuilt below
                replay(cur, dst, vec + (size_t)tt * kVecs * N);
                cur = dst;
            }
        }
        // ---- differentiate the chunk backwards, one group of kGroup tokens at a time
        const float *s_new = s_end;   // state after the token being differentiated
        for (int g = chunk_len / kGroup - 1; g >= 0; --g) {
            {
                const float *cur = ckpt + (size_t)g * M;
                for (int u = 0; u + 1 < kGroup; ++u) {   // states before tokens kGroup*g + 1 ..
                    replay(cur, grp + (size_t)u * M, vec + (size_t)(g * kGroup + u) * kVecs * N);
                    cur = grp + (size_t)u * M;
                }
            }
            for (int u = kGroup - 1; u >= 0; --u) {
                const int tt = g * kGroup + u;
                const size_t o = seq_base + (size_t)(t0 + tt) * tok_stride;
                const float *v_t = vec + (size_t)tt * kVecs * N;
                const float *s_old = u == 0 ? ckpt + (size_t)g * M : grp + (size_t)(u - 1) * M;   // state before the token
                const float *Sn_j = s_new + rr * P, *So_j = s_old + rr * P;
                float *dS_i = dS + rr * P, *dSt_j = dSt + rr * P;
                float dsa_i = 0.f;
                {
                    const float r_j = v_t[VR * N + rr], dy_i = v_t[VDY * N + rr];
                    float dr = 0.f, dd = 0.f, dk = 0.f, db = 0.f, dv = 0.f;
                    for (int c = q; c < n_cols; c += 4) {
                        const float dy_c = v_t[VDY * N + c];
                        dr = fmaf(Sn_j[c], dy_c, dr);
                        const float gij = fmaf(dy_i, v_t[VR * N + c], dS_i[c]);
                        dS_i[c] = gij;
                        const float gt = fmaf(r_j, dy_c, dSt_j[c]);
                        dSt_j[c] = gt;
                        dd = fmaf(gt, So_j[c], dd);
                        dk = fmaf(gt, v_t[VV * N + c], dk);
                        db = fmaf(gt, v_t[VSA * N + c], db);
                        dv = fmaf(gij, v_t[VK * N + c], dv);
                        dsa_i = fmaf(gij, v_t[VB * N + c], dsa_i);
                    }
                    dr = quad_sum(dr); dd = quad_sum(dd); dk = quad_sum(dk); db = quad_sum(db); dv = quad_sum(dv);
                    dsa_i = quad_sum(dsa_i);
                    if (live && q == 0) {
                        outs[OR_ * N + row] = dr;
                        outs[OW * N + row] = dd * (-v_t[VEW * N + row] * v_t[VD * N + row]);
                        outs[OK_ * N + row] = dk;
                        outs[OB * N + row] = db;
                        outs[OV * N + row] = dv;
                        dsa[row] = dsa_i;
                    }
                }
                __syncthreads();
                if (tid < N) {   // coalesced stores of the five gradients finished above
                    st<T>(p.receptance_grad, o + tid, outs[OR_ * N + tid]);
                    st<T>(p.weight_decay_grad, o + tid, outs[OW * N + tid]);
                    st<T>(p.replacement_key_grad, o + tid, outs[OK_ * N + tid]);
                    st<T>(p.replacement_grad, o + tid, outs[OB * N + tid]);
                    st<T>(p.value_grad, o + tid, outs[OV * N + tid]);
                }
                float da = 0.f;
                {
                    const float d_j = v_t[VD * N + rr], a_j = v_t[VA * N + rr];
                    for (int c = q; c < n_cols; c += 4) {
                        const float dsa_c = dsa[c];
                        da = fmaf(So_j[c], dsa_c, da);
                        dS_i[c] = fmaf(dS_i[c], v_t[VD * N + c], dsa_i * v_t[VA * N + c]);
                        dSt_j[c] = fmaf(dSt_j[c], d_j, a_j * dsa_c);
                    }
                }
                da = quad_sum(da);
                if (live && q == 0) st<T>(p.removal_key_normalized_grad, o + row, da);
                __syncthreads();   // dsa and outs are rewritten by the next token
                s_new = s_old;
            }
        }
    }

    if (p.initial_state_grad)
        for (int idx = tid; idx < N * N; idx += blockDim.x)
            p.initial_state_grad[state_base + idx] = dS[(idx / N) * P + idx % N];
}

// N == 64: the same algorithm with every work matrix in registers.  A thread owns an R x E
// block (rows row0 .., columns c0 ..) of S^T, dS and dS^T; no thread ever reads another thread's
// matrix elements, so only the per-token vectors, dsa and the output staging go through shared
// memory, read as 128-bit vectors, and a row sum is finished by shuffles among the 64/E threads
// of the row.  The kept states of the chunk replay are spilled to shared memory in a
// thread-private layout.  Measured on B=8, T=4096, H=12: 1 x 16 per thread (256 threads) 9.6 ms,
// bound by shared-memory bandwidth (every thread re-reads 16 columns of eight vectors per token);
// 2 x 8 7.3 ms; 4 x 4 7.1 ms; 2 x 4 (512 threads) 6.9 ms, the default.
template <typename T, int R, int E>
__global__ void __launch_bounds__(64 * 64 / (R * E), 1) wkv7_backward64_kernel(Wkv7BackwardArgs p) {
    static_assert(E % 4 == 0 && 64 % R == 0 && 64 % E == 0, "R rows x E columns of every work matrix per thread");
    constexpr int N = 64, TPR = N / E, THREADS = N * N / (R * E), Q4 = R * E / 4;   // threads per row group
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *vec = reinterpret_cast<float *>(smem_raw);        // [chunk_len][kVecs][N]
    float *dsa2 = vec + (size_t)kMaxChunk * kVecs * N;       // [2][N], by token parity
    float *outs2 = dsa2 + 2 * N;                             // [2][kOuts][N], by token parity
    float4 *keep = reinterpret_cast<float4 *>(outs2 + 2 * kOuts * N);   // [kStates - 1][Q4][THREADS]: thread-private states

    const int bh = blockIdx.x, bi = bh / (int)p.H, h = bh % (int)p.H;
    const int tid = threadIdx.x, row0 = (tid / TPR) * R, q = tid % TPR, c0 = q * E;
    const int Tlen = (int)p.T, chunk_len = (int)p.chunk_len, nchunks = Tlen / chunk_len;
    const size_t tok_stride = (size_t)p.H * N;
    const size_t seq_base = ((size_t)bi * Tlen * p.H + h) * N;
    const size_t state_base = (size_t)bh * N * N;

    // dS[row0 + rho][c0 + e] and dS^T[row0 + rho][c0 + e] = dS[c0 + e][row0 + rho]
    float dS[R][E], dSt[R][E];
#pragma unroll
    for (int rho = 0; rho < R; ++rho)
#pragma unroll
        for (int e = 0; e < E; ++e) {
            dS[rho][e] = p.next_state_grad ? p.next_state_grad[state_base + (size_t)(row0 + rho) * N + c0 + e] : 0.f;
            dSt[rho][e] = p.next_state_grad ? p.next_state_grad[state_base + (size_t)(c0 + e) * N + row0 + rho] : 0.f;
        }
    auto keep_store = [&](int slot, const float (&x)[R][E]) {
        const float *f = &x[0][0];
#pragma unroll
        for (int e4 = 0; e4 < Q4; ++e4)
            keep[((size_t)slot * Q4 + e4) * THREADS + tid] = make_float4(f[4 * e4], f[4 * e4 + 1], f[4 * e4 + 2], f[4 * e4 + 3]);
    };
    auto keep_load = [&](int slot, float (&x)[R][E]) {
        float *f = &x[0][0];
#pragma unroll
        for (int e4 = 0; e4 < Q4; ++e4) {
            const float4 v = keep[((size_t)slot * Q4 + e4) * THREADS + tid];
            f[4 * e4] = v.x; f[4 * e4 + 1] = v.y; f[4 * e4 + 2] = v.z; f[4 * e4 + 3] = v.w;
        }
    };
    auto ldv = [&](const float *base, float (&x)[E]) {   // this thread's E columns of one staged vector
#pragma unroll
        for (int e4 = 0; e4 < E / 4; ++e4) {
            const float4 v = *reinterpret_cast<const float4 *>(base + c0 + 4 * e4);
            x[4 * e4] = v.x; x[4 * e4 + 1] = v.y; x[4 * e4 + 2] = v.z; x[4 * e4 + 3] = v.w;
        }
    };
    // One forward step on this thread's elements of S^T: x[j][c] = x[j][c] d[j] + b[j] sa[c] + k[j] v[c].
    auto replay = [&](float (&x)[R][E], const float *v_t) {
        float sa[E], vv[E];
        ldv(v_t + VSA * N, sa);
        ldv(v_t + VV * N, vv);
#pragma unroll
        for (int rho = 0; rho < R; ++rho) {
            const float d_j = v_t[VD * N + row0 + rho], b_j = v_t[VB * N + row0 + rho], k_j = v_t[VK * N + row0 + rho];
#pragma unroll
            for (int e = 0; e < E; ++e) x[rho][e] = fmaf(x[rho][e], d_j, fmaf(b_j, sa[e], k_j * vv[e]));
        }
    };

    const int ngroups = chunk_len / kGroup;
    for (int chunk = nchunks - 1; chunk >= 0; --chunk) {
        const int t0 = chunk * chunk_len;
        __syncthreads();   // the previous chunk's vectors are no longer read
        // Stage the chunk's vectors: 16-byte loads, all requested before the first is used.
        {
            constexpr int EPV = 16 / (int)sizeof(T);            // elements per 16-byte vector
            constexpr int VPT = N / EPV;                        // vectors per token row
            constexpr int MAXV = (kMaxChunk * 8 * VPT + THREADS - 1) / THREADS;     // vectors per thread for a full chunk
            const int nvec = chunk_len * 8 * VPT;
            uint4 raw[MAXV];
#pragma unroll
            for (int n = 0; n < MAXV; ++n) {
                const int idx = tid + n * THREADS;
                raw[n] = make_uint4(0, 0, 0, 0);
                if (idx < nvec) {
                    const int cv = idx % VPT, tensor = (idx / VPT) % 8, tt = idx / (8 * VPT);
                    const void *src = tensor == VR ? p.r : tensor == VD ? p.w : tensor == VK ? p.k : tensor == VV ? p.v
                                    : tensor == VA ? p.a : tensor == VB ? p.b : tensor == VSA ? p.state_replacement
                                                                                             : p.output_grad;
                    raw[n] = __ldg(reinterpret_cast<const uint4 *>(
                        reinterpret_cast<const T *>(src) + seq_base + (size_t)(t0 + tt) * tok_stride + cv * EPV));
                }
            }
#pragma unroll
            for (int n = 0; n < MAXV; ++n) {
                const int idx = tid + n * THREADS;
                if (idx < nvec) {
                    const int cv = idx % VPT, tensor = (idx / VPT) % 8, tt = idx / (8 * VPT);
                    float f[EPV];
                    if constexpr (sizeof(T) == 4) {
                        f[0] = __uint_as_float(raw[n].x); f[1] = __uint_as_float(raw[n].y);
                        f[2] = __uint_as_float(raw[n].z); f[3] = __uint_as_float(raw[n].w);
                    } else {
                        const unsigned wds[4] = {raw[n].x, raw[n].y, raw[n].z, raw[n].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            f[2 * i] = __uint_as_float(wds[i] << 16);
                            f[2 * i + 1] = __uint_as_float(wds[i] & 0xffff0000u);
                        }
                    }
                    float *v_t = vec + (size_t)tt * kVecs * N;
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        float x = f[e];
                        if (tensor == VD) {
                            const float ew = __expf(x);
                            v_t[VEW * N + cv * EPV + e] = ew;
                            x = __expf(-ew);
                        }
                        v_t[tensor * N + cv * EPV + e] = x;
                    }
                }
            }
        }
        // state at the start of the chunk, transposed: S^T[j][c] = S[c][j]
        float st_cur[R][E];
        {
            const float *start = chunk > 0 ? p.snapshots + ((size_t)bh * nchunks + chunk - 1) * N * N
                                           : (p.initial_state ? p.initial_state + state_base : nullptr);
#pragma unroll
            for (int rho = 0; rho < R; ++rho)
#pragma unroll
                for (int e = 0; e < E; ++e) st_cur[rho][e] = start ? start[(size_t)(c0 + e) * N + row0 + rho] : 0.f;
        }
        __syncthreads();
        // replay the chunk forwards; slot g keeps the state before token kGroup * g
        for (int tt = 0; tt < chunk_len; ++tt) {
            if (tt % kGroup == 0) keep_store(tt / kGroup, st_cur);
            replay(st_cur, vec + (size_t)tt * kVecs * N);
        }
        float s_new[R][E];   // state after the token being differentiated
#pragma unroll
        for (int rho = 0; rho < R; ++rho)
#pragma unroll
            for (int e = 0; e < E; ++e) s_new[rho][e] = st_cur[rho][e];

        for (int g = ngroups - 1; g >= 0; --g) {
            // states before tokens kGroup*g + 1 .. kGroup*g + kGroup - 1 go to slots kMaxChunk/kGroup + u
            {
                float x[R][E];
                keep_load(g, x);
                for (int u = 0; u + 1 < kGroup; ++u) {
                    replay(x, vec + (size_t)(g * kGroup + u) * kVecs * N);
                    keep_store(kMaxChunk / kGroup + u, x);
                }
            }
            for (int u = kGroup - 1; u >= 0; --u) {
                const int tt = g * kGroup + u;
                const size_t o = seq_base + (size_t)(t0 + tt) * tok_stride;
                const float *v_t = vec + (size_t)tt * kVecs * N;
                // dsa and the output staging alternate between two buffers, so that one barrier
                // per token is enough: a buffer is rewritten two tokens later, after the barrier
                // of the token in between, which every thread reaches only after reading it.
                float *dsa = dsa2 + (tt & 1) * N, *outs = outs2 + (tt & 1) * kOuts * N;
                float s_old[R][E];   // state before the token
                keep_load(u == 0 ? g : kMaxChunk / kGroup + u - 1, s_old);
                float dyv[E], rv[E], vv[E], sav[E], kv[E], bv[E];
                ldv(v_t + VDY * N, dyv);
                ldv(v_t + VR * N, rv);
                ldv(v_t + VV * N, vv);
                ldv(v_t + VSA * N, sav);
                ldv(v_t + VK * N, kv);
                ldv(v_t + VB * N, bv);
                float dsa_i[R];
#pragma unroll
                for (int rho = 0; rho < R; ++rho) {
                    const int row = row0 + rho;
                    const float r_j = v_t[VR * N + row], dy_i = v_t[VDY * N + row];
                    float dr = 0.f, dd = 0.f, dk = 0.f, db = 0.f, dv = 0.f, ds = 0.f;
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        dr = fmaf(s_new[rho][e], dyv[e], dr);
                        dS[rho][e] = fmaf(dy_i, rv[e], dS[rho][e]);
                        dSt[rho][e] = fmaf(r_j, dyv[e], dSt[rho][e]);
                        dd = fmaf(dSt[rho][e], s_old[rho][e], dd);
                        dk = fmaf(dSt[rho][e], vv[e], dk);
                        db = fmaf(dSt[rho][e], sav[e], db);
                        dv = fmaf(dS[rho][e], kv[e], dv);
                        ds = fmaf(dS[rho][e], bv[e], ds);
                    }
                    dr = row_sum<TPR>(dr); dd = row_sum<TPR>(dd); dk = row_sum<TPR>(dk); db = row_sum<TPR>(db);
                    dv = row_sum<TPR>(dv); ds = row_sum<TPR>(ds);
                    dsa_i[rho] = ds;
                    if (q == 0) {
                        outs[OR_ * N + row] = dr;
                        outs[OW * N + row] = dd * (-v_t[VEW * N + row] * v_t[VD * N + row]);
                        outs[OK_ * N + row] = dk;
                        outs[OB * N + row] = db;
                        outs[OV * N + row] = dv;
                        dsa[row] = ds;
                    }
                }
                __syncthreads();
                if (tid < N) {
                    st<T>(p.receptance_grad, o + tid, outs[OR_ * N + tid]);
                    st<T>(p.weight_decay_grad, o + tid, outs[OW * N + tid]);
                    st<T>(p.replacement_key_grad, o + tid, outs[OK_ * N + tid]);
                    st<T>(p.replacement_grad, o + tid, outs[OB * N + tid]);
                    st<T>(p.value_grad, o + tid, outs[OV * N + tid]);
                }
                float dsav[E], dv_[E], av[E];
                ldv(dsa, dsav);
                ldv(v_t + VD * N, dv_);
                ldv(v_t + VA * N, av);
#pragma unroll
                for (int rho = 0; rho < R; ++rho) {
                    const int row = row0 + rho;
                    const float d_j = v_t[VD * N + row], a_j = v_t[VA * N + row];
                    float da = 0.f;
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        da = fmaf(s_old[rho][e], dsav[e], da);
                        dS[rho][e] = fmaf(dS[rho][e], dv_[e], dsa_i[rho] * av[e]);
                        dSt[rho][e] = fmaf(dSt[rho][e], d_j, a_j * dsav[e]);
                        s_new[rho][e] = s_old[rho][e];
                    }
                    da = row_sum<TPR>(da);
                    if (q == 0) st<T>(p.removal_key_normalized_grad, o + row, da);
                }
            }
        }
    }
    if (p.initial_state_grad) {
#pragma unroll
        for (int rho = 0; rho < R; ++rho)
#pragma unroll
            for (int e4 = 0; e4 < E / 4; ++e4)
                *reinterpret_cast<float4 *>(p.initial_state_grad + state_base + (size_t)(row0 + rho) * N + c0 + 4 * e4) =
                    make_float4(dS[rho][4 * e4], dS[rho][4 * e4 + 1], dS[rho][4 * e4 + 2], dS[rho][4 * e4 + 3]);
    }
}

}  // namespace

int launch_wkv7_backward(const Wkv7BackwardArgs &p, cudaStream_t stream) {
    if (p.B * p.H == 0 || p.T == 0) return 0;
    const int N = (int)p.N;
    if (N == 64) {
        constexpr int R = RWKV7_BWD_ROWS, E = RWKV7_BWD_COLS;   // rows x columns of every work matrix per thread
        constexpr int THREADS = 64 * 64 / (R * E);
        const size_t smem64 = sizeof(float) * ((size_t)(kMaxChunk * kVecs + 2 + 2 * kOuts) * 64 + (size_t)(kStates - 1) * 64 * 64);
        cudaError_t e64;
        if (p.bf16) {
            e64 = cudaFuncSetAttribute(wkv7_backward64_kernel<__nv_bfloat16, R, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem64);
            if (e64 != cudaSuccess) return (int)e64;
            wkv7_backward64_kernel<__nv_bfloat16, R, E><<<(unsigned)(p.B * p.H), THREADS, smem64, stream>>>(p);
        } else {
            e64 = cudaFuncSetAttribute(wkv7_backward64_kernel<float, R, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem64);
            if (e64 != cudaSuccess) return (int)e64;
            wkv7_backward64_kernel<float, R, E><<<(unsigned)(p.B * p.H), THREADS, smem64, stream>>>(p);
        }
        count_launch();
        return (int)cudaGetLastError();
    }
    const size_t smem = sizeof(float) * ((kStates + 2) * (size_t)N * (N + 4) + (size_t)(kMaxChunk * kVecs + 1 + kOuts) * N);
    const int threads = ((4 * N + 31) / 32) * 32;
    cudaError_t e;
    if (p.bf16) {
        e = cudaFuncSetAttribute(wkv7_backward_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        wkv7_backward_kernel<__nv_bfloat16><<<(unsigned)(p.B * p.H), threads, smem, stream>>>(p);
    } else {
        e = cudaFuncSetAttribute(wkv7_backward_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        wkv7_backward_kernel<float><<<(unsigned)(p.B * p.H), threads, smem, stream>>>(p);
    }
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace rwkv7
