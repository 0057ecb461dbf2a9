// WKV7 decode sweep (N == 64, T of a few tokens): the memory-bound case where
// every (b,h) state matrix (16 KB fp32) is read once and written once per call.
//
// Semantics: crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:179-242 of
// the reference at T == 1 (its custom kernel rejects T % 16 != 0, wkv7/io.rs:198-201).
//
// One CTA of 128 threads per (b,h): two threads share a state row, each holding
// 32 columns as eight 128-bit pieces interleaved with its partner, so a warp's
// load or store touches sixteen full 32-byte sectors.  The state loads are in
// flight while the six token vectors are converted and staged in shared memory;
// the two row reductions (S a and S r) are 32 FMAs and one shuffle each.  State
// traffic uses streaming loads and stores since nothing is reused.
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

template <typename T>
__global__ void __launch_bounds__(128, 8)
wkv7_decode_kernel(DecPtrs ptrs, const float *s0, T *__restrict__ y, float *s_out,
                   int Tlen, int H) {
    __shared__ __align__(16) float vec[6][kN];
    const int bh = blockIdx.x;
    const int bi = bh / H, h = bh % H;
    const int tid = threadIdx.x;
    const int row = tid >> 1, hf = tid & 1;

    float4 S[8];
    if (s0 != nullptr) {
        const float4 *src = reinterpret_cast<const float4 *>(s0 + ((size_t)bh * kN + row) * kN);
#pragma unroll
        for (int m = 0; m < 8; ++m) S[m] = __ldcs(src + 2 * m + hf);
    } else {
#pragma unroll
        for (int m = 0; m < 8; ++m) S[m] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

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
        const float4 *a4 = reinterpret_cast<const float4 *>(vec[VA]);
        float sa0 = 0.f, sa1 = 0.f;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const float4 a = a4[2 * m + hf];
            sa0 = fmaf(S[m].x, a.x, sa0);
            sa1 = fmaf(S[m].y, a.y, sa1);
            sa0 = fmaf(S[m].z, a.z, sa0);
            sa1 = fmaf(S[m].w, a.w, sa1);
        }
        float sa = sa0 + sa1;
        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
        const float vi = vec[VV][row];
        const float4 *d4 = reinterpret_cast<const float4 *>(vec[VD]);
        const float4 *b4 = reinterpret_cast<const float4 *>(vec[VB]);
        const float4 *k4 = reinterpret_cast<const float4 *>(vec[VK]);
        const float4 *r4 = reinterpret_cast<const float4 *>(vec[VR]);
        float y0 = 0.f, y1 = 0.f;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const float4 d = d4[2 * m + hf], b = b4[2 * m + hf], k = k4[2 * m + hf], r = r4[2 * m + hf];
            S[m].x = fmaf(S[m].x, d.x, fmaf(sa, b.x, vi * k.x));
            S[m].y = fmaf(S[m].y, d.y, fmaf(sa, b.y, vi * k.y));
            S[m].z = fmaf(S[m].z, d.z, fmaf(sa, b.z, vi * k.z));
            S[m].w = fmaf(S[m].w, d.w, fmaf(sa, b.w, vi * k.w));
            y0 = fmaf(S[m].x, r.x, y0);
            y1 = fmaf(S[m].y, r.y, y1);
            y0 = fmaf(S[m].z, r.z, y0);
            y1 = fmaf(S[m].w, r.w, y1);
        }
        float yy = y0 + y1;
        yy += __shfl_xor_sync(0xffffffffu, yy, 1);
        if (hf == 0) st_out<T>(y + o + row, yy);
    }

    if (s_out != nullptr) {
        float4 *dst = reinterpret_cast<float4 *>(s_out + ((size_t)bh * kN + row) * kN);
#pragma unroll
        for (int m = 0; m < 8; ++m) __stcs(dst + 2 * m + hf, S[m]);
    }
}

}  // namespace

int launch_wkv7_decode(const Wkv7Args &p, cudaStream_t stream) {
    DecPtrs ptrs{{p.r, p.w, p.k, p.v, p.a, p.b}};
    const unsigned grid = (unsigned)(p.B * p.H);
    if (p.bf16)
        wkv7_decode_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(ptrs, p.s0, reinterpret_cast<__nv_bfloat16 *>(p.y),
                                                                    p.s_out, (int)p.T, (int)p.H);
    else
        wkv7_decode_kernel<float><<<grid, 128, 0, stream>>>(ptrs, p.s0, reinterpret_cast<float *>(p.y), p.s_out,
                                                            (int)p.T, (int)p.H);
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace rwkv7
