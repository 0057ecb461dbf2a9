// Internal launch interface between the C ABI (abi.cpp) and the CUDA kernels.
// Plain pointers and sizes; every launcher enqueues on `stream` and returns the
// cudaError_t of the launch as an int (0 = success).
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime_api.h>

namespace rwkv7 {

// Device status word values (see rwkv7_read_device_status).
enum DeviceStatus : int { kDevOk = 0, kDevTimeout = 1, kDevBadIndex = 2, kDevInternal = 3 };
// Address of the per-device status word, resolved once per device.
int device_status_ptr(int device, int **out);
// One bounded wait on a barrier nobody signals: records kDevTimeout and returns (test hook).
int launch_bounded_wait_selftest(int device, unsigned max_polls, cudaStream_t stream);
// Process-wide count of kernel launches (rwkv7_kernel_launch_count).
void count_launch(int n = 1);
int64_t launch_count();

struct Wkv7Args {
    const void *r, *w, *k, *v, *a, *b;  // [B,T,H,N], bf16 or f32
    const float *s0;                    // [B,H,N,N] or null (zero state)
    void *y;                            // [B,T,H,N]
    float *s_out;                       // [B,H,N,N] or null
    int64_t B, T, H, N;
    bool bf16;
    int device;
    int num_sms;
};

// Token-by-token scan, fp32 state in registers (N == 64) or shared memory (any
// N <= 128).  Also the decode (T == 1) sweep.
int launch_wkv7_sequential(const Wkv7Args &p, cudaStream_t stream);
// Decode sweep (N == 64, a few tokens): one pass over the fp32 state per call.
int launch_wkv7_decode(const Wkv7Args &p, cudaStream_t stream);

// Training forward: the sequential scan, also writing snapshots [B,H,T/chunk_len,N,N] (fp32 state
// after the last token of every chunk) and state_replacement [B,T,H,N] (sa_t, sequence dtype).
int launch_wkv7_forward_saved(const Wkv7Args &p, float *snapshots, void *state_replacement, int chunk_len,
                              cudaStream_t stream);

// Backward pass over the tensors the training forward saved.
struct Wkv7BackwardArgs {
    const void *r, *w, *k, *v, *a, *b;          // [B,T,H,N]
    const float *snapshots;                      // [B,H,T/chunk_len,N,N]
    const void *state_replacement, *output_grad; // [B,T,H,N]
    const float *initial_state;                  // [B,H,N,N] or null (zero): the state the forward started from
    const float *next_state_grad;                // [B,H,N,N] or null (zero)
    void *receptance_grad, *weight_decay_grad, *replacement_key_grad, *value_grad,
        *removal_key_normalized_grad, *replacement_grad;   // [B,T,H,N]
    float *initial_state_grad;                   // [B,H,N,N] or null
    int64_t B, T, H, N, chunk_len;
    bool bf16;
};
int launch_wkv7_backward(const Wkv7BackwardArgs &p, cudaStream_t stream);

// Time-parallel backward (N == 64, bf16, chunk_len 16, T >= 64): the gradient recurrence runs as a
// forward pass of the tensor-core prefill kernel over the reversed sequence, everything else per
// 16-token chunk.  Needs wkv7_backward_parallel_workspace_bytes of workspace.
bool wkv7_backward_parallel_supported(const Wkv7BackwardArgs &p);
size_t wkv7_backward_parallel_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N);
int launch_wkv7_backward_parallel(const Wkv7BackwardArgs &p, void *workspace, int device, int num_sms,
                                  cudaStream_t stream);

// Chunked tensor-core prefill (N == 64): tcgen05 MMAs with TMEM accumulators.
size_t wkv7_chunked_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N);
bool wkv7_chunked_supported(const Wkv7Args &p);
int launch_wkv7_chunked(const Wkv7Args &p, void *workspace, size_t workspace_bytes,
                        cudaStream_t stream);

// Two-kernel tensor-core prefill (N == 64, bf16, fp16 operands): the operator of every 64-token chunk
// is built for all chunks in parallel, then one scan per chain applies them.  The workspace holds the
// per-chain fallback flags (first B*H ints), a carried state per chain and the operators of one
// segment of chunks; `wkv7_split_workspace_bytes` is the size the launcher prefers (fewest segments
// within its operator budget), `wkv7_split_min_workspace_bytes` the least it can work with.
// Chains it cannot resolve (decay range, non-finite operators) are left flagged for the caller.
size_t wkv7_split_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N, int num_sms);
// With at most as many chains as SMs the scan of a segment of chunks runs on a second stream beside the
// operator kernel of the next segment (1, default) or after it on the caller's stream (0).
int wkv7_split_overlap();
void wkv7_set_split_overlap(int on);
size_t wkv7_split_min_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N);
bool wkv7_split_supported(const Wkv7Args &p);
int launch_wkv7_split(const Wkv7Args &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
// The flagged chains only, by the tf32 chunked kernel (one CTA per chain), then by the sequential scan
// for those that are still flagged afterwards.
int launch_wkv7_chunked_flagged(const Wkv7Args &p, void *workspace, cudaStream_t stream);
// Sequential recomputation of the chains whose flag is set (exits at once for the others).
int launch_wkv7_sequential_flagged(const Wkv7Args &p, const int *flags, cudaStream_t stream);

// Cluster size of the chunked kernel: 0 = by the number of chains (default), else 1, 2 or 4.
int wkv7_cluster_override();
void wkv7_set_cluster_override(int k);

// Training forward on the tensor cores (N == 64, bf16, chunk_len 16): the chunked kernel also
// writing snapshots and state_replacement; same workspace as launch_wkv7_chunked.
int launch_wkv7_chunked_saved(const Wkv7Args &p, void *workspace, float *snapshots, void *state_replacement,
                              cudaStream_t stream);

// Fixed flag array inside the library image, usable in place of a workspace by
// callers that must not allocate: device address (resolved on first use per
// device, which must be current) and capacity.
int wkv7_static_scratch(int device, void **ptr, size_t *bytes);
int64_t wkv7_static_scratch_max_chains();

struct MixArgs {
    const void *x;        // [B,T,C]
    const void *mu[6];    // [C] each
    void *out[6];         // [B,T,C] each
    int64_t B, T, C;
    bool bf16;
    int num_sms;
};
int launch_mix6(const MixArgs &p, cudaStream_t stream);

struct AddcmulArgs {
    const void *base, *diff;  // [rows,C]
    const void *scale[5];     // [C] each
    void *out[5];             // [rows,C] each
    int nscale;               // 1 or 5
    int64_t rows, C;
    bool bf16;
    int num_sms;
};
int launch_addcmul(const AddcmulArgs &p, cudaStream_t stream);

// Tail of WeightPrepare::forward: rows = B*T*H head rows of N elements; parameters are [H*N].
struct WeightPrepareArgs {
    const void *key_precursor, *learning_rate_lora, *weight_decay_lora;   // [rows,N]
    const void *key_removal, *key_replacement;                             // [H*N]
    const void *value_precursor, *value_from_first_cell, *value_residual_lora;   // [rows,N] or all null
    void *weight_decay, *replacement_key, *removal_key_normalized, *replacement;  // [rows,N]
    void *value;                                                           // [rows,N] or null
    int64_t rows, H, N;
    bool bf16;
    int num_sms;
};
int launch_weight_prepare(const WeightPrepareArgs &p, cudaStream_t stream);

// Body of GatedReadout::forward between the gate LoRA and the output projection.
struct GatedReadoutArgs {
    const void *wkv7_output, *receptance, *replacement_key, *value, *gate;   // [rows,N]
    const void *gamma, *beta, *bonus;                                        // [H*N]
    void *output;                                                            // [rows,N]
    float epsilon;
    int64_t rows, H, N;
    bool bf16;
    int num_sms;
};
int launch_gated_readout(const GatedReadoutArgs &p, cudaStream_t stream);

// Channel mixer: x [B,T,C] bf16, key_scale [C], key_weight [F,C], value_weight [C,F], out [B,T,C].
struct ChannelMixerArgs {
    const void *x, *key_scale, *key_weight, *value_weight;
    void *out;
    int64_t B, T, C, F;
    int *status;   // device status word
    int num_sms;
};
size_t channel_mixer_workspace_bytes(int64_t rows, int64_t C, int64_t F);
int launch_channel_mixer(const ChannelMixerArgs &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);

struct TokenShiftArgs {
    const void *x;     // [B,T,C]
    void *state;       // [S,C], updated in place
    const void *ids;   // [B]
    int ids_dtype;     // RWKV7_I32 / RWKV7_I64 / RWKV7_U32
    void *diff;        // [B,T,C]
    int64_t B, T, C, S;
    bool bf16;
    int *status;       // device status word
    int num_sms;
};
int launch_token_shift_diff(const TokenShiftArgs &p, cudaStream_t stream);

struct LmHeadArgs {
    const void *x;        // [R,C] bf16
    const void *w;        // [V,C] bf16
    const void *targets;  // [R]
    int targets_dtype;
    int64_t vocab_offset;
    float *partials;      // [R,3]
    int64_t R, C, V;
    int device;
    int num_sms;
    int *status;
};
size_t lm_head_ce_workspace_bytes(int64_t R, int64_t C, int64_t V);
int launch_lm_head_ce_partial(const LmHeadArgs &p, void *workspace, size_t workspace_bytes,
                              cudaStream_t stream);
int launch_lm_head_ce_finalize(const float *partials_all, int num_shards, const void *targets,
                               int targets_dtype, float *lse, float *loss, int64_t R,
                               cudaStream_t stream);

}  // namespace rwkv7
