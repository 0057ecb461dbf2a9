// Sequential WKV7 scan and decode sweep.
//
// Semantics: crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:179-242 of
// the reference (per token: sa = S a; S = S diag(d) + sa b^T + v k^T; y = S r,
// d = exp(-exp(w))).  Unlike the reference kernel (kernel.rs:82-195), which
// re-reads its state row from global memory every token, the fp32 state here
// stays in registers for the whole call and is read from / written to HBM once.
//
// N == 64: a CTA owns ROWS value rows of one (b,h); 4 threads share a row, each
// holding 16 key columns (interleaved in groups of 4 so that the per-token
// vectors are read from shared memory with conflict-free 128-bit loads).  Token
// vectors are staged 16 tokens at a time through a double-buffered shared tile,
// converted to fp32 once (decay computed once per element).
// Any other N <= 128: one thread per row, state in shared memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "kernels.h"

namespace rwkv7 {
namespace {

constexpr int kN = 64;
constexpr int kTile = 16;  // tokens staged per shared tile

enum { VR = 0, VD = 1, VK = 2, VV = 3, VA = 4, VB = 5 };

struct SeqPtrs {
    const void *in[6];  // r, w, k, v, a, b
};

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
    static constexpr int kElems = 4;
    static __device__ __forceinline__ void unpack(const uint4 &u, float *f) {
        f[0] = __uint_as_float(u.x);
        f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z);
        f[3] = __uint_as_float(u.w);
    }
};
template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void unpack(const uint4 &u, float *f) {
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// Tensors a training forward saves for the backward pass (wkv7/forward.rs:368-375):
// snapshots [B,H,T/chunk_len,N,N] = the state after the last token of every chunk (fp32 here),
// state_replacement [B,T,H,N] = sa_t = S_{t-1} a_t, in the sequence dtype.
struct SavePtrs {
    float *snapshots;
    void *state_replacement;
    int chunk_len;
};

template <typename T, int ROWS, bool SAVE = false>
__global__ void __launch_bounds__(ROWS * 4)
wkv7_seq64_kernel(SeqPtrs ptrs, const float *s0, T *__restrict__ y,
                  float *s_out, int Tlen, int H, const int *__restrict__ flags, SavePtrs save = SavePtrs{}) {
    constexpr int THREADS = ROWS * 4;
    constexpr int SPLITS = kN / ROWS;
    constexpr int EPV = Vec16<T>::kElems;
    constexpr int VPR = kN / EPV;                 // 16-byte vectors per token row
    constexpr int VECS = kTile * 6 * VPR;         // vectors per tile
    constexpr int NV = (VECS + THREADS - 1) / THREADS;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *vec = reinterpret_cast<float *>(smem_raw);             // [2][kTile][6][kN]
    float *ytile = vec + 2 * kTile * 6 * kN;                      // [2][kTile][ROWS]
    float *satile = ytile + 2 * kTile * ROWS;                     // [2][kTile][ROWS], SAVE only

    const int bh = blockIdx.x / SPLITS;
    // Fallback mode: only the chains another kernel flagged are (re)computed.
    if (flags != nullptr) {
        // (launched right behind the kernel that writes the flags, possibly before it has finished:
        // wait for its memory; a no-op for an ordinary launch)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (flags[bh] == 0) return;
    }
    const int split = blockIdx.x % SPLITS;
    const int bi = bh / H, h = bh % H;
    const int row0 = split * ROWS;
    const int tid = threadIdx.x;
    const int i = tid >> 2, q = tid & 3;

    float S[16];
    if (s0 != nullptr) {
        const float4 *src =
            reinterpret_cast<const float4 *>(s0 + ((size_t)bh * kN + row0 + i) * kN);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const float4 x = src[kk * 4 + q];
            S[kk * 4 + 0] = x.x; S[kk * 4 + 1] = x.y; S[kk * 4 + 2] = x.z; S[kk * 4 + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) S[e] = 0.f;
    }

    const size_t seq_base = ((size_t)bi * Tlen * H + h) * kN;  // element offset of (b, t=0, h, 0)
    const size_t tok_stride = (size_t)H * kN;
    const int ntiles = (Tlen + kTile - 1) / kTile;

    uint4 stage[NV];
    auto issue_loads = [&](int tile) {
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int idx = tid + n * THREADS;
            stage[n] = make_uint4(0, 0, 0, 0);
            if (idx < VECS) {
                const int c = idx % VPR;
                const int tensor = (idx / VPR) % 6;
                const int tok = idx / (VPR * 6);
                const int t = tile * kTile + tok;
                if (t < Tlen) {
                    const T *p = reinterpret_cast<const T *>(ptrs.in[tensor]) + seq_base +
                                 (size_t)t * tok_stride + c * EPV;
                    stage[n] = __ldg(reinterpret_cast<const uint4 *>(p));
                }
            }
        }
    };
    auto commit_stage = [&](int buf) {
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int idx = tid + n * THREADS;
            if (idx < VECS) {
                const int c = idx % VPR;
                const int tensor = (idx / VPR) % 6;
                const int tok = idx / (VPR * 6);
                float f[EPV];
                Vec16<T>::unpack(stage[n], f);
                if (tensor == VD) {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) f[e] = expf(-expf(f[e]));
                }
                float4 *dst = reinterpret_cast<float4 *>(
                    vec + (((size_t)buf * kTile + tok) * 6 + tensor) * kN + c * EPV);
#pragma unroll
                for (int e = 0; e < EPV / 4; ++e)
                    dst[e] = make_float4(f[4 * e], f[4 * e + 1], f[4 * e + 2], f[4 * e + 3]);
            }
        }
    };

    issue_loads(0);
    commit_stage(0);
    __syncthreads();

    for (int tile = 0; tile < ntiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < ntiles) issue_loads(tile + 1);
        const int ntok = min(kTile, Tlen - tile * kTile);
        const float *tv = vec + (size_t)buf * kTile * 6 * kN;
        float *yt = ytile + (size_t)buf * kTile * ROWS;
        float *sat = satile + (size_t)buf * kTile * ROWS;

        for (int tt = 0; tt < ntok; ++tt) {
            const float *base = tv + (size_t)tt * 6 * kN;
            const float4 *a4 = reinterpret_cast<const float4 *>(base + VA * kN);
            float sa0 = 0.f, sa1 = 0.f, sa2 = 0.f, sa3 = 0.f;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float4 x = a4[kk * 4 + q];
                sa0 = fmaf(S[kk * 4 + 0], x.x, sa0);
                sa1 = fmaf(S[kk * 4 + 1], x.y, sa1);
                sa2 = fmaf(S[kk * 4 + 2], x.z, sa2);
                sa3 = fmaf(S[kk * 4 + 3], x.w, sa3);
            }
            float sa = (sa0 + sa1) + (sa2 + sa3);
            sa += __shfl_xor_sync(0xffffffffu, sa, 1);
            sa += __shfl_xor_sync(0xffffffffu, sa, 2);
            if constexpr (SAVE) {
                if (q == 0) sat[tt * ROWS + i] = sa;
            }
            const float vi = base[VV * kN + row0 + i];
            const float4 *d4 = reinterpret_cast<const float4 *>(base + VD * kN);
            const float4 *b4 = reinterpret_cast<const float4 *>(base + VB * kN);
            const float4 *k4 = reinterpret_cast<const float4 *>(base + VK * kN);
            const float4 *r4 = reinterpret_cast<const float4 *>(base + VR * kN);
            float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float4 d = d4[kk * 4 + q], bb = b4[kk * 4 + q], kx = k4[kk * 4 + q],
                             rr = r4[kk * 4 + q];
                float s;
                s = fmaf(S[kk * 4 + 0], d.x, fmaf(sa, bb.x, vi * kx.x)); S[kk * 4 + 0] = s; y0 = fmaf(s, rr.x, y0);
                s = fmaf(S[kk * 4 + 1], d.y, fmaf(sa, bb.y, vi * kx.y)); S[kk * 4 + 1] = s; y1 = fmaf(s, rr.y, y1);
                s = fmaf(S[kk * 4 + 2], d.z, fmaf(sa, bb.z, vi * kx.z)); S[kk * 4 + 2] = s; y2 = fmaf(s, rr.z, y2);
                s = fmaf(S[kk * 4 + 3], d.w, fmaf(sa, bb.w, vi * kx.w)); S[kk * 4 + 3] = s; y3 = fmaf(s, rr.w, y3);
            }
            float yy = (y0 + y1) + (y2 + y3);
            yy += __shfl_xor_sync(0xffffffffu, yy, 1);
            yy += __shfl_xor_sync(0xffffffffu, yy, 2);
            if (q == 0) yt[tt * ROWS + i] = yy;
            if constexpr (SAVE) {
                const int t = tile * kTile + tt;
                if ((t + 1) % save.chunk_len == 0) {   // state after the last token of a chunk
                    const int chunk = t / save.chunk_len, nchunks = Tlen / save.chunk_len;
                    float4 *dst = reinterpret_cast<float4 *>(
                        save.snapshots + (((size_t)bh * nchunks + chunk) * kN + row0 + i) * kN);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        dst[kk * 4 + q] = make_float4(S[kk * 4 + 0], S[kk * 4 + 1], S[kk * 4 + 2], S[kk * 4 + 3]);
                }
            }
        }

        if (tile + 1 < ntiles) commit_stage(buf ^ 1);
        __syncthreads();
        for (int idx = tid; idx < ntok * ROWS; idx += THREADS) {
            const int tt = idx / ROWS, rr = idx % ROWS;
            const size_t o = seq_base + (size_t)(tile * kTile + tt) * tok_stride + row0 + rr;
            y[o] = from_f32<T>(yt[tt * ROWS + rr]);
            if constexpr (SAVE) reinterpret_cast<T *>(save.state_replacement)[o] = from_f32<T>(sat[tt * ROWS + rr]);
        }
    }

    if (s_out != nullptr) {
        float4 *dst = reinterpret_cast<float4 *>(s_out + ((size_t)bh * kN + row0 + i) * kN);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
            dst[kk * 4 + q] = make_float4(S[kk * 4 + 0], S[kk * 4 + 1], S[kk * 4 + 2], S[kk * 4 + 3]);
    }
}

// Any head size N <= 128: thread i owns state row i, kept in shared memory with
// a padded row pitch; the six token vectors are staged per token.
template <typename T, bool SAVE = false>
__global__ void wkv7_seq_generic_kernel(SeqPtrs ptrs, const float *s0,
                                        T *__restrict__ y, float *s_out, int Tlen,
                                        int H, int N, SavePtrs save = SavePtrs{}) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int pitch = N + 1;
    float *S = reinterpret_cast<float *>(smem_raw);  // [N][N+1]
    float *vec = S + (size_t)N * pitch;              // [6][N]
    const int bh = blockIdx.x;
    const int bi = bh / H, h = bh % H;
    const int tid = threadIdx.x;

    for (int idx = tid; idx < N * N; idx += blockDim.x) {
        const int i = idx / N, j = idx % N;
        S[i * pitch + j] = s0 ? s0[(size_t)bh * N * N + idx] : 0.f;
    }
    const size_t seq_base = ((size_t)bi * Tlen * H + h) * N;
    const size_t tok_stride = (size_t)H * N;
    __syncthreads();
    for (int t = 0; t < Tlen; ++t) {
        const size_t o = seq_base + (size_t)t * tok_stride;
        for (int idx = tid; idx < 6 * N; idx += blockDim.x) {
            const int tensor = idx / N, j = idx % N;
            float x = static_cast<float>(reinterpret_cast<const T *>(ptrs.in[tensor])[o + j]);
            if (tensor == VD) x = expf(-expf(x));
            vec[idx] = x;
        }
        __syncthreads();
        if (tid < N) {
            float *Si = S + tid * pitch;
            float sa = 0.f;
            for (int j = 0; j < N; ++j) sa = fmaf(Si[j], vec[VA * N + j], sa);
            const float vi = vec[VV * N + tid];
            float acc = 0.f;
            for (int j = 0; j < N; ++j) {
                const float s = fmaf(Si[j], vec[VD * N + j], fmaf(sa, vec[VB * N + j], vi * vec[VK * N + j]));
                Si[j] = s;
                acc = fmaf(s, vec[VR * N + j], acc);
            }
            y[o + tid] = from_f32<T>(acc);
            if constexpr (SAVE) {
                reinterpret_cast<T *>(save.state_replacement)[o + tid] = from_f32<T>(sa);
                if ((t + 1) % save.chunk_len == 0) {
                    float *dst = save.snapshots +
                                 (((size_t)bh * (Tlen / save.chunk_len) + t / save.chunk_len) * N + tid) * N;
                    for (int j = 0; j < N; ++j) dst[j] = Si[j];
                }
            }
        }
        __syncthreads();
    }
    if (s_out != nullptr)
        for (int idx = tid; idx < N * N; idx += blockDim.x) {
            const int i = idx / N, j = idx % N;
            s_out[(size_t)bh * N * N + idx] = S[i * pitch + j];
        }
}

template <typename T, int ROWS>
int launch_seq64(const Wkv7Args &p, cudaStream_t stream, const int *flags = nullptr) {
    SeqPtrs ptrs{{p.r, p.w, p.k, p.v, p.a, p.b}};
    const size_t smem = sizeof(float) * (2 * kTile * 6 * kN + 4 * kTile * ROWS);
    auto kern = wkv7_seq64_kernel<T, ROWS, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const unsigned grid = (unsigned)(p.B * p.H * (kN / ROWS));
    if (flags != nullptr) {
        // The flagged-chain pass follows the kernel that wrote the flags on the same stream: programmatic
        // dependent launch lets its launch overlap that kernel's tail (the kernel itself waits for the flags).
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(ROWS * 4);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, kern, ptrs, p.s0, reinterpret_cast<T *>(p.y), p.s_out, (int)p.T, (int)p.H, flags,
                               SavePtrs{});
        if (e == cudaSuccess) count_launch();
        return (int)e;
    }
    kern<<<grid, ROWS * 4, smem, stream>>>(ptrs, p.s0, reinterpret_cast<T *>(p.y), p.s_out,
                                           (int)p.T, (int)p.H, flags, SavePtrs{});
    count_launch();
    return (int)cudaGetLastError();
}

template <typename T>
int launch_seq(const Wkv7Args &p, cudaStream_t stream) {
    if (p.N == kN) {
        // Split the 64 value rows of a (b,h) over several CTAs when there are too
        // few (b,h) chains to fill the SMs; rows of S never interact.
        const int64_t chains = p.B * p.H;
        int rows = 64;
        if (chains < 2 * (int64_t)p.num_sms) rows = 32;
        if (chains * 2 < 2 * (int64_t)p.num_sms) rows = 16;
        if (rows == 64) return launch_seq64<T, 64>(p, stream);
        if (rows == 32) return launch_seq64<T, 32>(p, stream);
        return launch_seq64<T, 16>(p, stream);
    }
    SeqPtrs ptrs{{p.r, p.w, p.k, p.v, p.a, p.b}};
    const int N = (int)p.N;
    const size_t smem = sizeof(float) * ((size_t)N * (N + 1) + 6 * N);
    auto kern = wkv7_seq_generic_kernel<T, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int threads = ((N + 31) / 32) * 32;
    kern<<<(unsigned)(p.B * p.H), threads, smem, stream>>>(ptrs, p.s0, reinterpret_cast<T *>(p.y),
                                                          p.s_out, (int)p.T, (int)p.H, N, SavePtrs{});
    count_launch();
    return (int)cudaGetLastError();
}

// Training forward: the scan above, also writing the tensors the backward pass needs.
template <typename T>
int launch_seq_saved(const Wkv7Args &p, float *snapshots, void *state_replacement, int chunk_len,
                     cudaStream_t stream) {
    SeqPtrs ptrs{{p.r, p.w, p.k, p.v, p.a, p.b}};
    SavePtrs save{snapshots, state_replacement, chunk_len};
    if (p.N == kN) {
        constexpr int ROWS = 16;   // four CTAs per chain: rows of S never interact
        const size_t smem = sizeof(float) * (2 * kTile * 6 * kN + 4 * kTile * ROWS);
        auto kern = wkv7_seq64_kernel<T, ROWS, true>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<(unsigned)(p.B * p.H * (kN / ROWS)), ROWS * 4, smem, stream>>>(
            ptrs, p.s0, reinterpret_cast<T *>(p.y), p.s_out, (int)p.T, (int)p.H, nullptr, save);
    } else {
        const int N = (int)p.N;
        const size_t smem = sizeof(float) * ((size_t)N * (N + 1) + 6 * N);
        auto kern = wkv7_seq_generic_kernel<T, true>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<(unsigned)(p.B * p.H), ((N + 31) / 32) * 32, smem, stream>>>(
            ptrs, p.s0, reinterpret_cast<T *>(p.y), p.s_out, (int)p.T, (int)p.H, N, save);
    }
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace

int launch_wkv7_forward_saved(const Wkv7Args &p, float *snapshots, void *state_replacement, int chunk_len,
                              cudaStream_t stream) {
    return p.bf16 ? launch_seq_saved<__nv_bfloat16>(p, snapshots, state_replacement, chunk_len, stream)
                  : launch_seq_saved<float>(p, snapshots, state_replacement, chunk_len, stream);
}

// N == 64 only: the flagged chains again, with the saved tensors of the training forward.
int launch_wkv7_sequential_flagged_saved(const Wkv7Args &p, const int *flags, float *snapshots,
                                         void *state_replacement, int chunk_len, cudaStream_t stream) {
    SeqPtrs ptrs{{p.r, p.w, p.k, p.v, p.a, p.b}};
    SavePtrs save{snapshots, state_replacement, chunk_len};
    constexpr int ROWS = 16;
    const size_t smem = sizeof(float) * (2 * kTile * 6 * kN + 4 * kTile * ROWS);
    const unsigned grid = (unsigned)(p.B * p.H * (kN / ROWS));
    cudaError_t e;
    if (p.bf16) {
        auto kern = wkv7_seq64_kernel<__nv_bfloat16, ROWS, true>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, ROWS * 4, smem, stream>>>(ptrs, p.s0, reinterpret_cast<__nv_bfloat16 *>(p.y), p.s_out, (int)p.T,
                                               (int)p.H, flags, save);
    } else {
        auto kern = wkv7_seq64_kernel<float, ROWS, true>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, ROWS * 4, smem, stream>>>(ptrs, p.s0, reinterpret_cast<float *>(p.y), p.s_out, (int)p.T, (int)p.H,
                                               flags, save);
    }
    count_launch();
    return (int)cudaGetLastError();
}

// N == 64 only: recomputes the chains with flags[b*H+h] != 0, 16 value rows per CTA.
int launch_wkv7_sequential_flagged(const Wkv7Args &p, const int *flags, cudaStream_t stream) {
    return p.bf16 ? launch_seq64<__nv_bfloat16, 16>(p, stream, flags) : launch_seq64<float, 16>(p, stream, flags);
}

int launch_wkv7_sequential(const Wkv7Args &p, cudaStream_t stream) {
    // A handful of tokens per chain is the decode case: the state sweep dominates.
    if (p.N == kN && p.T <= 4) return launch_wkv7_decode(p, stream);
    return p.bf16 ? launch_seq<__nv_bfloat16>(p, stream) : launch_seq<float>(p, stream);
}

}  // namespace rwkv7
