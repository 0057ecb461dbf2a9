// Token-shift mixing kernels: mix6, addcmul / addcmul5, token_shift_diff.
//
// All three are pure streaming kernels bound by HBM bandwidth.  A CTA owns a
// block of consecutive token rows; a thread owns one 16-byte channel vector of
// every row in the block, keeps the per-channel scales in registers for the
// whole block and carries the previous row in registers, so each input element
// is read from memory once (plus one halo row per block) and every access is a
// coalesced 128-bit load or store.  Arithmetic is fp32, rounded once on store.
//
// Reference semantics (paths inside the rwkv-rs repository):
//   mix6              crates/rwkv-nn/src/kernels/train/time_mixer/mix6/kernel.rs:25-57
//   addcmul/addcmul5  crates/rwkv-nn/src/kernels/template/addcmul/kernel.rs:4-65
//   token_shift_diff  crates/rwkv-nn/src/kernels/template/token_shift_diff/kernel.rs:16-45
//                     (there one thread walks T serially; here T is parallel and
//                     only the t == 0 row touches the carried state)
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "rwkv7_b200.h"

namespace rwkv7 {
namespace {

constexpr int kRowsPerBlock = 16;

__host__ __device__ __forceinline__ int64_t imin(int64_t a, int64_t b) { return a < b ? a : b; }

// EPV elements per vector: 8 (bf16, 16 B), 4 (f32, 16 B) or 1 (scalar fallback
// for channel counts or pointers that are not 16-byte aligned).
template <typename T, int EPV>
struct Pack {
    float f[EPV];
    __device__ __forceinline__ void load(const T *p) {
        if constexpr (EPV == 1) {
            f[0] = static_cast<float>(*p);
        } else if constexpr (sizeof(T) == 4) {
            const float4 x = *reinterpret_cast<const float4 *>(p);
            f[0] = x.x; f[1] = x.y; f[2] = x.z; f[3] = x.w;
        } else {
            const uint4 u = *reinterpret_cast<const uint4 *>(p);
            const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                f[2 * i] = __uint_as_float(w[i] << 16);
                f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < EPV; ++i) f[i] = 0.f;
    }
    __device__ __forceinline__ void store(T *p) const {
        if constexpr (EPV == 1) {
            if constexpr (sizeof(T) == 4) *p = f[0];
            else *p = __float2bfloat16_rn(f[0]);
        } else if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
        } else {
            uint4 u;
            unsigned *w = &u.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                w[i] = *reinterpret_cast<const unsigned *>(&h);
            }
            *reinterpret_cast<uint4 *>(p) = u;
        }
    }
};

struct Mix6Ptrs {
    const void *mu[6];
    void *out[6];
};

template <typename T, int EPV>
__global__ void __launch_bounds__(256)
mix6_kernel(const T *__restrict__ x, Mix6Ptrs ptrs, int64_t rows, int64_t Tlen, int64_t C) {
    const int64_t CV = C / EPV;
    const int64_t row_begin = (int64_t)blockIdx.x * kRowsPerBlock;
    const int64_t row_end = imin(rows, row_begin + kRowsPerBlock);
    for (int64_t cv = threadIdx.x; cv < CV; cv += blockDim.x) {
        const int64_t c = cv * EPV;
        Pack<T, EPV> mu[6];
#pragma unroll
        for (int s = 0; s < 6; ++s) mu[s].load(reinterpret_cast<const T *>(ptrs.mu[s]) + c);
        Pack<T, EPV> prev;
        if (row_begin % Tlen == 0) prev.zero();
        else prev.load(x + (row_begin - 1) * C + c);
#pragma unroll 4
        for (int64_t row = row_begin; row < row_end; ++row) {
            Pack<T, EPV> cur;
            cur.load(x + row * C + c);
            if (row % Tlen == 0) prev.zero();  // first token of a sequence: x_{-1} = 0
#pragma unroll
            for (int s = 0; s < 6; ++s) {
                Pack<T, EPV> o;
#pragma unroll
                for (int e = 0; e < EPV; ++e)
                    o.f[e] = fmaf(prev.f[e] - cur.f[e], mu[s].f[e], cur.f[e]);
                o.store(reinterpret_cast<T *>(ptrs.out[s]) + row * C + c);
            }
            prev = cur;
        }
    }
}

struct AddcmulPtrs {
    const void *scale[5];
    void *out[5];
};

template <typename T, int EPV, int NS>
__global__ void __launch_bounds__(256)
addcmul_kernel(const T *base, const T *__restrict__ diff, AddcmulPtrs ptrs, int64_t rows, int64_t C) {
    const int64_t CV = C / EPV;
    const int64_t row_begin = (int64_t)blockIdx.x * kRowsPerBlock;
    const int64_t row_end = imin(rows, row_begin + kRowsPerBlock);
    for (int64_t cv = threadIdx.x; cv < CV; cv += blockDim.x) {
        const int64_t c = cv * EPV;
        Pack<T, EPV> sc[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) sc[s].load(reinterpret_cast<const T *>(ptrs.scale[s]) + c);
        // five scale vectors already fill 40 registers: a shorter unroll keeps three CTAs per SM
#pragma unroll(NS == 1 ? 4 : 2)
        for (int64_t row = row_begin; row < row_end; ++row) {
            Pack<T, EPV> bs, df;
            if constexpr (NS == 1) {
                bs.load(base + row * C + c);  // `out[0]` may alias `base`: read before write, same thread
            } else {
                // the five outputs never alias the inputs: let loads of later rows pass earlier stores
                const T *__restrict__ base_noalias = base;
                bs.load(base_noalias + row * C + c);
            }
            df.load(diff + row * C + c);
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                Pack<T, EPV> o;
#pragma unroll
                for (int e = 0; e < EPV; ++e) o.f[e] = fmaf(df.f[e], sc[s].f[e], bs.f[e]);
                o.store(reinterpret_cast<T *>(ptrs.out[s]) + row * C + c);
            }
        }
    }
}

__device__ __forceinline__ int64_t load_id(const void *ids, int dtype, int64_t b) {
    if (dtype == RWKV7_I64) return reinterpret_cast<const int64_t *>(ids)[b];
    if (dtype == RWKV7_U32) return (int64_t) reinterpret_cast<const uint32_t *>(ids)[b];
    return (int64_t) reinterpret_cast<const int32_t *>(ids)[b];
}

template <typename T, int EPV>
__global__ void __launch_bounds__(256)
token_shift_diff_kernel(const T *__restrict__ x, T *state, const void *__restrict__ ids,
                        int ids_dtype, T *__restrict__ diff, int64_t B, int64_t Tlen, int64_t C,
                        int64_t S, int *status) {
    const int64_t CV = C / EPV;
    const int64_t blocks_per_seq = (Tlen + kRowsPerBlock - 1) / kRowsPerBlock;
    const int64_t b = blockIdx.x / blocks_per_seq;
    const int64_t t_begin = (blockIdx.x % blocks_per_seq) * kRowsPerBlock;
    const int64_t t_end = imin(Tlen, t_begin + kRowsPerBlock);
    const int64_t slot = load_id(ids, ids_dtype, b);
    const bool slot_ok = slot >= 0 && slot < S;
    if (!slot_ok && threadIdx.x == 0 && t_begin == 0) atomicExch(status, (int)kDevBadIndex);
    const T *xb = x + b * Tlen * C;
    T *db = diff + b * Tlen * C;
    for (int64_t cv = threadIdx.x; cv < CV; cv += blockDim.x) {
        const int64_t c = cv * EPV;
        Pack<T, EPV> prev;
        if (t_begin == 0) {
            if (slot_ok) prev.load(state + slot * C + c);
            else prev.zero();
        } else {
            prev.load(xb + (t_begin - 1) * C + c);
        }
#pragma unroll 4
        for (int64_t t = t_begin; t < t_end; ++t) {
            Pack<T, EPV> cur, o;
            cur.load(xb + t * C + c);
#pragma unroll
            for (int e = 0; e < EPV; ++e) o.f[e] = prev.f[e] - cur.f[e];
            o.store(db + t * C + c);
            prev = cur;
        }
        // The thread that read the carried token of this (slot, channel vector)
        // is the only one that overwrites it, after its read.
        if (t_begin == 0 && slot_ok) {
            Pack<T, EPV> last;
            if (t_end == Tlen) last = prev;
            else last.load(xb + (Tlen - 1) * C + c);
            last.store(state + slot * C + c);
        }
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int pick_threads(int64_t CV) {
    int t = 32;
    while (t < 256 && t < CV) t <<= 1;
    return t;
}

}  // namespace

int launch_mix6(const MixArgs &p, cudaStream_t stream) {
    const int64_t rows = p.B * p.T;
    if (rows == 0 || p.C == 0) return 0;
    Mix6Ptrs ptrs;
    bool vec_ok = aligned16(p.x);
    for (int s = 0; s < 6; ++s) {
        ptrs.mu[s] = p.mu[s];
        ptrs.out[s] = p.out[s];
        vec_ok = vec_ok && aligned16(p.mu[s]) && aligned16(p.out[s]);
    }
    const unsigned grid = (unsigned)((rows + kRowsPerBlock - 1) / kRowsPerBlock);
    if (p.bf16) {
        using T = __nv_bfloat16;
        if (vec_ok && p.C % 8 == 0)
            mix6_kernel<T, 8><<<grid, pick_threads(p.C / 8), 0, stream>>>((const T *)p.x, ptrs, rows, p.T, p.C);
        else
            mix6_kernel<T, 1><<<grid, pick_threads(p.C), 0, stream>>>((const T *)p.x, ptrs, rows, p.T, p.C);
    } else {
        if (vec_ok && p.C % 4 == 0)
            mix6_kernel<float, 4><<<grid, pick_threads(p.C / 4), 0, stream>>>((const float *)p.x, ptrs, rows, p.T, p.C);
        else
            mix6_kernel<float, 1><<<grid, pick_threads(p.C), 0, stream>>>((const float *)p.x, ptrs, rows, p.T, p.C);
    }
    count_launch();
    return (int)cudaGetLastError();
}

template <typename T, int EPV>
static void launch_addcmul_t(const AddcmulArgs &p, const AddcmulPtrs &ptrs, unsigned grid,
                             cudaStream_t stream) {
    const int threads = pick_threads(p.C / EPV);
    if (p.nscale == 1)
        addcmul_kernel<T, EPV, 1><<<grid, threads, 0, stream>>>((const T *)p.base, (const T *)p.diff, ptrs, p.rows, p.C);
    else
        addcmul_kernel<T, EPV, 5><<<grid, threads, 0, stream>>>((const T *)p.base, (const T *)p.diff, ptrs, p.rows, p.C);
}

int launch_addcmul(const AddcmulArgs &p, cudaStream_t stream) {
    if (p.rows == 0 || p.C == 0) return 0;
    AddcmulPtrs ptrs{};
    bool vec_ok = aligned16(p.base) && aligned16(p.diff);
    for (int s = 0; s < p.nscale; ++s) {
        ptrs.scale[s] = p.scale[s];
        ptrs.out[s] = p.out[s];
        vec_ok = vec_ok && aligned16(p.scale[s]) && aligned16(p.out[s]);
    }
    const unsigned grid = (unsigned)((p.rows + kRowsPerBlock - 1) / kRowsPerBlock);
    if (p.bf16) {
        if (vec_ok && p.C % 8 == 0) launch_addcmul_t<__nv_bfloat16, 8>(p, ptrs, grid, stream);
        else launch_addcmul_t<__nv_bfloat16, 1>(p, ptrs, grid, stream);
    } else {
        if (vec_ok && p.C % 4 == 0) launch_addcmul_t<float, 4>(p, ptrs, grid, stream);
        else launch_addcmul_t<float, 1>(p, ptrs, grid, stream);
    }
    count_launch();
    return (int)cudaGetLastError();
}

int launch_token_shift_diff(const TokenShiftArgs &p, cudaStream_t stream) {
    if (p.B == 0 || p.T == 0 || p.C == 0) return 0;  // T == 0: diff empty, state unchanged
    const int64_t blocks_per_seq = (p.T + kRowsPerBlock - 1) / kRowsPerBlock;
    const unsigned grid = (unsigned)(p.B * blocks_per_seq);
    const bool vec_ok = aligned16(p.x) && aligned16(p.state) && aligned16(p.diff);
    if (p.bf16) {
        using T = __nv_bfloat16;
        if (vec_ok && p.C % 8 == 0)
            token_shift_diff_kernel<T, 8><<<grid, pick_threads(p.C / 8), 0, stream>>>(
                (const T *)p.x, (T *)p.state, p.ids, p.ids_dtype, (T *)p.diff, p.B, p.T, p.C, p.S, p.status);
        else
            token_shift_diff_kernel<T, 1><<<grid, pick_threads(p.C), 0, stream>>>(
                (const T *)p.x, (T *)p.state, p.ids, p.ids_dtype, (T *)p.diff, p.B, p.T, p.C, p.S, p.status);
    } else {
        if (vec_ok && p.C % 4 == 0)
            token_shift_diff_kernel<float, 4><<<grid, pick_threads(p.C / 4), 0, stream>>>(
                (const float *)p.x, (float *)p.state, p.ids, p.ids_dtype, (float *)p.diff, p.B, p.T, p.C, p.S, p.status);
        else
            token_shift_diff_kernel<float, 1><<<grid, pick_threads(p.C), 0, stream>>>(
                (const float *)p.x, (float *)p.state, p.ids, p.ids_dtype, (float *)p.diff, p.B, p.T, p.C, p.S, p.status);
    }
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace rwkv7
