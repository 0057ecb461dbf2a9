// Elementwise-plus-head-reduction kernels on either side of the WKV7 recurrence.
//
//   weight_prepare_kernel   the tail of WeightPrepare::forward
//       (crates/rwkv-nn/src/modules/time_mixer/weight_prepare.rs:252-287 with
//        crates/rwkv-nn/src/functions/normalize.rs:9-41 and functions/lerp.rs:4-10):
//       everything after the dense projections and LoRA products, i.e. the ~10
//       tensor ops that turn key_precursor, the learning-rate LoRA output, the
//       decay LoRA output (and the value-residual inputs) into the WKV7-ready
//       weight_decay, replacement_key, removal_key_normalized, replacement, value.
//   gated_readout_kernel    the body of GatedReadout::forward between the gate LoRA
//       and the output projection
//       (crates/rwkv-nn/src/modules/time_mixer/gated_readout.rs:110-145):
//       per-head GroupNorm of the WKV7 output, the receptance-key bonus, the gate.
//
// Both are HBM-bound streaming kernels with one reduction over the head per
// (b,t,h) row.  [B,T,C] and [B,T,H,N] are the same memory (C = H*N), so a row is N
// contiguous elements.  Fast path (N == 64, 16-byte aligned): a group of 64/EPV lanes
// owns a row, each lane one 16-byte vector of every tensor; the reductions are
// shuffles inside the group; every element is read and written exactly once.
// Generic path (any N): one warp per row, scalar accesses.  Arithmetic is fp32
// and each result is rounded once on store (the reference rounds to the storage
// type after every tensor op).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "rwkv7_b200.h"

namespace rwkv7 {
namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T *p) {
    return static_cast<float>(*p);
}
template <typename T>
__device__ __forceinline__ void stf(T *p, float x) {
    if constexpr (sizeof(T) == 4) *p = x;
    else *p = __float2bfloat16_rn(x);
}

// 16-byte vector of EPV elements as floats.
template <typename T, int EPV>
struct Vec {
    float f[EPV];
    __device__ __forceinline__ void load(const T *p) {
        if constexpr (sizeof(T) == 4) {
            const float4 x = __ldg(reinterpret_cast<const float4 *>(p));
            f[0] = x.x; f[1] = x.y; f[2] = x.z; f[3] = x.w;
        } else {
            const uint4 u = __ldg(reinterpret_cast<const uint4 *>(p));
            const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                f[2 * i] = __uint_as_float(w[i] << 16);
                f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    }
    // streaming variants: data that is touched once should not displace the parameters in L1/L2
    __device__ __forceinline__ void load_stream(const T *p) {
        if constexpr (sizeof(T) == 4) {
            const float4 x = __ldcs(reinterpret_cast<const float4 *>(p));
            f[0] = x.x; f[1] = x.y; f[2] = x.z; f[3] = x.w;
        } else {
            const uint4 u = __ldcs(reinterpret_cast<const uint4 *>(p));
            const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                f[2 * i] = __uint_as_float(w[i] << 16);
                f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    }
    __device__ __forceinline__ void store(T *p) const {
        if constexpr (sizeof(T) == 4) {
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

// Fast-math forms: the kernels are close to issue-bound on the special-function unit, and
// the absolute error of these forms (~1e-7) is far below one bf16 or fp32-output tolerance.
__device__ __forceinline__ float sigmoidf(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// -softplus(-d) - 0.5, softplus(z) = log(1 + e^z) evaluated without overflow
__device__ __forceinline__ float decay_precursor(float d) {
    const float z = -d;
    const float sp = fmaxf(z, 0.f) + __logf(1.f + __expf(-fabsf(z)));
    return -sp - 0.5f;
}

template <int LANES>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// ---- weight_prepare ----------------------------------------------------------------

template <typename T, int EPV>
__global__ void __launch_bounds__(256)
weight_prepare_vec_kernel(WeightPrepareArgs p) {
    constexpr int kN = 64, LANES = kN / EPV, ROWS_PER_WARP = 32 / LANES;
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const bool with_value = p.value != nullptr;
    // The loop bound is uniform across the warp (the shuffles below need every lane); a lane
    // group past the last row recomputes that row and skips its stores.
    for (int64_t row0 = warp * ROWS_PER_WARP; row0 < p.rows; row0 += nwarps * ROWS_PER_WARP) {
        const bool active = row0 + lane / LANES < p.rows;
        const int64_t row = active ? row0 + lane / LANES : p.rows - 1;
        const int64_t off = row * kN + sub * EPV;
        const int64_t c = (row % p.H) * kN + sub * EPV;
        Vec<T, EPV> k, lr, d, xi, al;
        k.load_stream((const T *)p.key_precursor + off);
        lr.load_stream((const T *)p.learning_rate_lora + off);
        d.load_stream((const T *)p.weight_decay_lora + off);
        xi.load((const T *)p.key_removal + c);
        al.load((const T *)p.key_replacement + c);
        Vec<T, EPV> w, kt, a, b;
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            lr.f[e] = sigmoidf(lr.f[e]);
            kt.f[e] = k.f[e] * fmaf(al.f[e], lr.f[e] - 1.f, 1.f);
            w.f[e] = decay_precursor(d.f[e]);
            a.f[e] = k.f[e] * xi.f[e];          // removal key before normalisation
            ss = fmaf(a.f[e], a.f[e], ss);
        }
        ss = group_sum<LANES>(ss);
        const float inv = fminf(rsqrtf(ss), 1e12f);   // 1 / max(||.||, 1e-12)
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            const float kappa = a.f[e] * inv;
            a.f[e] = -kappa;
            b.f[e] = kappa * lr.f[e];
        }
        if (!active) continue;
        w.store((T *)p.weight_decay + off);
        kt.store((T *)p.replacement_key + off);
        a.store((T *)p.removal_key_normalized + off);
        b.store((T *)p.replacement + off);
        if (with_value) {
            // loaded only now: holding three more vectors across the reduction costs a CTA per SM
            Vec<T, EPV> vp, vf, nu;
            vp.load_stream((const T *)p.value_precursor + off);
            vf.load_stream((const T *)p.value_from_first_cell + off);
            nu.load_stream((const T *)p.value_residual_lora + off);
#pragma unroll
            for (int e = 0; e < EPV; ++e) vp.f[e] = fmaf(vf.f[e] - vp.f[e], sigmoidf(nu.f[e]), vp.f[e]);
            vp.store((T *)p.value + off);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
weight_prepare_generic_kernel(WeightPrepareArgs p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t N = p.N;
    for (int64_t row = warp; row < p.rows; row += nwarps) {
        const int64_t base = row * N, cbase = (row % p.H) * N;
        float ss = 0.f;
        for (int64_t e = lane; e < N; e += 32) {
            const float rk = ldf((const T *)p.key_precursor + base + e) * ldf((const T *)p.key_removal + cbase + e);
            ss = fmaf(rk, rk, ss);
        }
        ss = group_sum<32>(ss);
        const float inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
        for (int64_t e = lane; e < N; e += 32) {
            const float k = ldf((const T *)p.key_precursor + base + e);
            const float lr = sigmoidf(ldf((const T *)p.learning_rate_lora + base + e));
            const float kappa = k * ldf((const T *)p.key_removal + cbase + e) * inv;
            stf((T *)p.weight_decay + base + e, decay_precursor(ldf((const T *)p.weight_decay_lora + base + e)));
            stf((T *)p.replacement_key + base + e, k * fmaf(ldf((const T *)p.key_replacement + cbase + e), lr - 1.f, 1.f));
            stf((T *)p.removal_key_normalized + base + e, -kappa);
            stf((T *)p.replacement + base + e, kappa * lr);
            if (p.value != nullptr) {
                const float vp = ldf((const T *)p.value_precursor + base + e);
                const float vf = ldf((const T *)p.value_from_first_cell + base + e);
                stf((T *)p.value + base + e, fmaf(vf - vp, sigmoidf(ldf((const T *)p.value_residual_lora + base + e)), vp));
            }
        }
    }
}

// ---- gated_readout -----------------------------------------------------------------

template <typename T, int EPV>
__global__ void __launch_bounds__(256)
gated_readout_vec_kernel(GatedReadoutArgs p) {
    constexpr int kN = 64, LANES = kN / EPV, ROWS_PER_WARP = 32 / LANES;
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    // The loop bound is uniform across the warp (the shuffles below need every lane); a lane
    // group past the last row recomputes that row and skips its stores.
    for (int64_t row0 = warp * ROWS_PER_WARP; row0 < p.rows; row0 += nwarps * ROWS_PER_WARP) {
        const bool active = row0 + lane / LANES < p.rows;
        const int64_t row = active ? row0 + lane / LANES : p.rows - 1;
        const int64_t off = row * kN + sub * EPV;
        const int64_t c = (row % p.H) * kN + sub * EPV;
        Vec<T, EPV> y, r, k, v, g, gamma, beta, rho;
        y.load_stream((const T *)p.wkv7_output + off);
        r.load_stream((const T *)p.receptance + off);
        k.load_stream((const T *)p.replacement_key + off);
        v.load_stream((const T *)p.value + off);
        g.load_stream((const T *)p.gate + off);
        gamma.load((const T *)p.gamma + c);
        beta.load((const T *)p.beta + c);
        rho.load((const T *)p.bonus + c);
        float s1 = 0.f, dot = 0.f;
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            s1 += y.f[e];
            dot = fmaf(r.f[e] * k.f[e], rho.f[e], dot);
        }
        s1 = group_sum<LANES>(s1);
        dot = group_sum<LANES>(dot);
        const float mean = s1 * (1.f / kN);
        float s2 = 0.f;
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            y.f[e] -= mean;
            s2 = fmaf(y.f[e], y.f[e], s2);
        }
        s2 = group_sum<LANES>(s2);
        const float rstd = rsqrtf(s2 * (1.f / kN) + p.epsilon);
        Vec<T, EPV> o;
#pragma unroll
        for (int e = 0; e < EPV; ++e)
            o.f[e] = (fmaf(y.f[e] * rstd, gamma.f[e], beta.f[e]) + dot * v.f[e]) * g.f[e];
        if (active) o.store((T *)p.output + off);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_readout_generic_kernel(GatedReadoutArgs p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t N = p.N;
    for (int64_t row = warp; row < p.rows; row += nwarps) {
        const int64_t base = row * N, cbase = (row % p.H) * N;
        float s1 = 0.f, dot = 0.f;
        for (int64_t e = lane; e < N; e += 32) {
            s1 += ldf((const T *)p.wkv7_output + base + e);
            dot = fmaf(ldf((const T *)p.receptance + base + e) * ldf((const T *)p.replacement_key + base + e),
                       ldf((const T *)p.bonus + cbase + e), dot);
        }
        s1 = group_sum<32>(s1);
        dot = group_sum<32>(dot);
        const float mean = s1 / (float)N;
        float s2 = 0.f;
        for (int64_t e = lane; e < N; e += 32) {
            const float dlt = ldf((const T *)p.wkv7_output + base + e) - mean;
            s2 = fmaf(dlt, dlt, s2);
        }
        s2 = group_sum<32>(s2);
        const float rstd = rsqrtf(s2 / (float)N + p.epsilon);
        for (int64_t e = lane; e < N; e += 32) {
            const float nrm = fmaf((ldf((const T *)p.wkv7_output + base + e) - mean) * rstd,
                                   ldf((const T *)p.gamma + cbase + e), ldf((const T *)p.beta + cbase + e));
            stf((T *)p.output + base + e,
                (nrm + dot * ldf((const T *)p.value + base + e)) * ldf((const T *)p.gate + base + e));
        }
    }
}

inline bool aligned16(const void *p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// A grid that fills every SM a few times over; the kernels stride over the rows.
inline unsigned pick_grid(int64_t rows, int rows_per_block, int num_sms) {
    const int64_t need = (rows + rows_per_block - 1) / rows_per_block;
    const int64_t cap = (int64_t)num_sms * 16;
    return (unsigned)(need < cap ? (need > 0 ? need : 1) : cap);
}

}  // namespace

int launch_weight_prepare(const WeightPrepareArgs &p, cudaStream_t stream) {
    if (p.rows == 0 || p.N == 0) return 0;
    const bool vec_ok = p.N == 64 && aligned16(p.key_precursor) && aligned16(p.learning_rate_lora) &&
                        aligned16(p.weight_decay_lora) && aligned16(p.key_removal) && aligned16(p.key_replacement) &&
                        aligned16(p.value_precursor) && aligned16(p.value_from_first_cell) &&
                        aligned16(p.value_residual_lora) && aligned16(p.weight_decay) &&
                        aligned16(p.replacement_key) && aligned16(p.removal_key_normalized) &&
                        aligned16(p.replacement) && aligned16(p.value);
    constexpr int kThreads = 256;
    if (p.bf16) {
        using T = __nv_bfloat16;
        if (vec_ok) weight_prepare_vec_kernel<T, 8><<<pick_grid(p.rows, kThreads / 8, p.num_sms), kThreads, 0, stream>>>(p);
        else weight_prepare_generic_kernel<T><<<pick_grid(p.rows, kThreads / 32, p.num_sms), kThreads, 0, stream>>>(p);
    } else {
        if (vec_ok) weight_prepare_vec_kernel<float, 4><<<pick_grid(p.rows, kThreads / 16, p.num_sms), kThreads, 0, stream>>>(p);
        else weight_prepare_generic_kernel<float><<<pick_grid(p.rows, kThreads / 32, p.num_sms), kThreads, 0, stream>>>(p);
    }
    count_launch();
    return (int)cudaGetLastError();
}

int launch_gated_readout(const GatedReadoutArgs &p, cudaStream_t stream) {
    if (p.rows == 0 || p.N == 0) return 0;
    const bool vec_ok = p.N == 64 && aligned16(p.wkv7_output) && aligned16(p.receptance) &&
                        aligned16(p.replacement_key) && aligned16(p.value) && aligned16(p.gate) &&
                        aligned16(p.gamma) && aligned16(p.beta) && aligned16(p.bonus) && aligned16(p.output);
    constexpr int kThreads = 256;
    if (p.bf16) {
        using T = __nv_bfloat16;
        if (vec_ok) gated_readout_vec_kernel<T, 8><<<pick_grid(p.rows, kThreads / 8, p.num_sms), kThreads, 0, stream>>>(p);
        else gated_readout_generic_kernel<T><<<pick_grid(p.rows, kThreads / 32, p.num_sms), kThreads, 0, stream>>>(p);
    } else {
        if (vec_ok) gated_readout_vec_kernel<float, 4><<<pick_grid(p.rows, kThreads / 16, p.num_sms), kThreads, 0, stream>>>(p);
        else gated_readout_generic_kernel<float><<<pick_grid(p.rows, kThreads / 32, p.num_sms), kThreads, 0, stream>>>(p);
    }
    count_launch();
    return (int)cudaGetLastError();
}

}  // namespace rwkv7
