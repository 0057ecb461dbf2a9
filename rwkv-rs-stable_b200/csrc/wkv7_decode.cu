// WKV7 decode sweep (N == 64, T of a few tokens): the memory-bound case where
// every (b,h) state matrix (16 KB fp32) is read once and written once per call.
//
// Semantics: crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:179-242 of
// the reference at T == 1 (its custom kernel rejects T % 16 != 0, wkv7/io.rs:198-201).
//
// One CTA of 128 threads per (b,h); a thread holds a block of R rows x 32/R columns of the
// state in registers, so a warp's loads and stores touch full 32-byte sectors of R rows.  The
// state loads are in flight while the six token vectors are converted and staged in shared
// memory; the two row reductions (S a and S r) end in shuffles among the threads of a row.
// State traffic uses streaming loads and stores since nothing is reused.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels.h"

namespace rwkv7 {
namespace {

constexpr int kN = 64;

struct DecPtrs {
    const void *in[6];  // r, w, k, v, a, b
};

enum { VR = 0, VD = 1, VK = 2, VV = 3, VA = 4, VB = 5 };

template <typename T>
__device__ __forceinline__ float ld_f32(const T *p);
template <>
__device__ __forceinline__ float ld_f32<float>(const float *p) { return __ldg(p); }
template <>
__device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __uint_as_float((unsigned)__ldg(reinterpret_cast<const unsigned short *>(p)) << 16);
}
template <typename T>
__device__ __forceinline__ void st_out(T *p, float x);
template <>
__device__ __forceinline__ void st_out<float>(float *p, float x) { *p = x; }
template <>
__device__ __forceinline__ void st_out<__nv_bfloat16>(__nv_bfloat16 *p, float x) { *p = __float2bfloat16_rn(x); }

#ifndef RWKV7_DECODE_ROWS
#define RWKV7_DECODE_ROWS 8
#endif

// A thread owns R rows x E columns of the state (R * E = 32, 128 threads per (b,h)): the E
// columns of each token vector it needs are read from shared memory once for all R rows, which
// is what keeps the shared-memory port from competing with the HBM stream (with one row of 32
// columns per thread the kernel read 80 KB of shared memory per 32 KB of state traffic).
template <typename T, int R>
__global__ void __launch_bounds__(128, 8)
wkv7_decode_kernel(DecPtrs ptrs, const float *s0, T *__restrict__ y, float *s_out,
                   int Tlen, int H) {
    constexpr int E = 32 / R, TPR = kN / E, Q = E / 4;   // columns per thread, threads per row, float4s per row
    __shared__ __align__(16) float vec[6][kN];
    const int bh = blockIdx.x;
    const int bi = bh / H, h = bh % H;
    const int tid = threadIdx.x;
    const int row0 = (tid / TPR) * R, c0 = (tid % TPR) * E;

    // Launched with programmatic stream serialization: this grid's CTAs may take their places while the kernel
    // before it on the stream (typically the previous layer's sweep) is still draining; nothing is read before
    // that kernel has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float4 S[R][Q];
    if (s0 != nullptr) {
#pragma unroll
        for (int rho = 0; rho < R; ++rho) {
            const float4 *src = reinterpret_cast<const float4 *>(s0 + ((size_t)bh * kN + row0 + rho) * kN + c0);
#pragma unroll
            for (int m = 0; m < Q; ++m) S[rho][m] = __ldcs(src + m);
        }
    } else {
#pragma unroll
        for (int rho = 0; rho < R; ++rho)
#pragma unroll
            for (int m = 0; m < Q; ++m) S[rho][m] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    // (this CTA's state loads are under way: the next kernel on the stream may start taking places)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int t = 0; t < Tlen; ++t) {
        const size_t o = (((size_t)bi * Tlen + t) * H + h) * kN;
        if (t > 0) __syncthreads();  // previous token's vectors fully consumed
        for (int idx = tid; idx < 6 * kN; idx += 128) {
            const int tensor = idx >> 6, j = idx & 63;
            float x = ld_f32(reinterpret_cast<const T *>(ptrs.in[tensor]) + o + j);
            if (tensor == VD) x = expf(-expf(x));
            vec[tensor][j] = x;
        }
        __syncthreads();
        float4 av[Q];
#pragma unroll
        for (int m = 0; m < Q; ++m) av[m] = *reinterpret_cast<const float4 *>(&vec[VA][c0 + 4 * m]);
        float sa[R];
#pragma unroll
        for (int rho = 0; rho < R; ++rho) {
            float s0_ = 0.f, s1_ = 0.f;
#pragma unroll
            for (int m = 0; m < Q; ++m) {
                s0_ = fmaf(S[rho][m].x, av[m].x, s0_);
                s1_ = fmaf(S[rho][m].y, av[m].y, s1_);
                s0_ = fmaf(S[rho][m].z, av[m].z, s0_);
                s1_ = fmaf(S[rho][m].w, av[m].w, s1_);
            }
            float x = s0_ + s1_;
#pragma unroll
            for (int off = TPR / 2; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
            sa[rho] = x;
        }
        float yy[R];
#pragma unroll
        for (int rho = 0; rho < R; ++rho) yy[rho] = 0.f;
#pragma unroll
        for (int m = 0; m < Q; ++m) {
            const float4 d = *reinterpret_cast<const float4 *>(&vec[VD][c0 + 4 * m]);
            const float4 b = *reinterpret_cast<const float4 *>(&vec[VB][c0 + 4 * m]);
            const float4 k = *reinterpret_cast<const float4 *>(&vec[VK][c0 + 4 * m]);
            const float4 r = *reinterpret_cast<const float4 *>(&vec[VR][c0 + 4 * m]);
#pragma unroll
            for (int rho = 0; rho < R; ++rho) {
                const float vi = vec[VV][row0 + rho];
                float4 &x = S[rho][m];
                x.x = fmaf(x.x, d.x, fmaf(sa[rho], b.x, vi * k.x));
                x.y = fmaf(x.y, d.y, fmaf(sa[rho], b.y, vi * k.y));
                x.z = fmaf(x.z, d.z, fmaf(sa[rho], b.z, vi * k.z));
                x.w = fmaf(x.w, d.w, fmaf(sa[rho], b.w, vi * k.w));
                yy[rho] = fmaf(x.x, r.x, fmaf(x.y, r.y, fmaf(x.z, r.z, fmaf(x.w, r.w, yy[rho]))));
            }
        }
#pragma unroll
        for (int rho = 0; rho < R; ++rho) {
            float x = yy[rho];
#pragma unroll
            for (int off = TPR / 2; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
            if (tid % TPR == 0) st_out<T>(y + o + row0 + rho, x);
        }
    }

    if (s_out != nullptr) {
#pragma unroll
        for (int rho = 0; rho < R; ++rho) {
            float4 *dst = reinterpret_cast<float4 *>(s_out + ((size_t)bh * kN + row0 + rho) * kN + c0);
#pragma unroll
            for (int m = 0; m < Q; ++m) __stcs(dst + m, S[rho][m]);
        }
    }
}

}  // namespace

int launch_wkv7_decode(const Wkv7Args &p, cudaStream_t stream) {
    DecPtrs ptrs{{p.r, p.w, p.k, p.v, p.a, p.b}};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.B * p.H));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
    if (p.bf16)
        e = cudaLaunchKernelEx(&cfg, wkv7_decode_kernel<__nv_bfloat16, RWKV7_DECODE_ROWS>, ptrs, p.s0,
                               reinterpret_cast<__nv_bfloat16 *>(p.y), p.s_out, (int)p.T, (int)p.H);
    else
        e = cudaLaunchKernelEx(&cfg, wkv7_decode_kernel<float, RWKV7_DECODE_ROWS>, ptrs, p.s0, reinterpret_cast<float *>(p.y),
                               p.s_out, (int)p.T, (int)p.H);
    if (e == cudaSuccess) count_launch();
    return (int)e;
}

}  // namespace rwkv7
