// rwkv7_b200.hpp — C++ host-side mirror of the reference's operator interface,
// header-only, over the C ABI of rwkv7_b200.h.
//
// Names and argument meaning follow the reference's public wrappers and I/O
// structs: Wkv7PretrainForwardInputs / wkv7_pretrain_custom / wkv7_statetune_custom /
// wkv7_statepass_custom (crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/io.rs:20-173,
// mod.rs:105-150), mix6_custom (.../mix6/mod.rs:76-108), addcmul_custom /
// addcmul5_custom (crates/rwkv-nn/src/kernels/template/addcmul/mod.rs:100-157),
// token_shift_diff_custom (.../token_shift_diff/mod.rs:82-111).  Where the reference
// panics (`inputs.check().unwrap()`, `assert!`), these functions throw
// KernelInputsError carrying the same message text.  Unlike the reference there
// is no allocator behind this layer: the caller passes the output tensors.
#ifndef RWKV7_B200_HPP_
#define RWKV7_B200_HPP_

#include <array>
#include <vector>
#include <cstdint>
#include <initializer_list>
#include <stdexcept>
#include <string>

#include "rwkv7_b200.h"

namespace rwkv7b200 {

// The reference's KernelInputsError (kernels/check.rs:34-73) plus the ABI's own codes.
class KernelInputsError : public std::runtime_error {
   public:
    KernelInputsError(int status, const std::string &message) : std::runtime_error(message), status_(status) {}
    int status() const { return status_; }
    const char *kind() const { return rwkv7_status_string(status_); }

   private:
    int status_;
};

inline void check_status(int status) {
    if (status != RWKV7_OK) throw KernelInputsError(status, rwkv7_last_error_message());
}

// Borrowed, contiguous row-major view of device memory.
struct TensorView {
    rwkv7_tensor t{};
    TensorView() = default;
    TensorView(void *data, rwkv7_dtype dtype, int device, std::initializer_list<int64_t> shape) {
        t.data = data;
        t.dtype = dtype;
        t.device = device;
        t.ndim = (int32_t)shape.size();
        int i = 0;
        for (int64_t d : shape) t.shape[i++] = d;
        int64_t stride = 1;
        for (int k = t.ndim - 1; k >= 0; --k) {
            t.stride[k] = stride;
            stride *= t.shape[k];
        }
    }
    const rwkv7_tensor *c() const { return &t; }
    rwkv7_tensor *m() { return &t; }
};

// wkv7/io.rs:20-66
struct Wkv7PretrainForwardInputs {
    TensorView receptance, weight_decay, replacement_key, value, removal_key_normalized, replacement;
    int64_t chunk_len = 16;

    // The two assertions that precede the reference's shape checks (wkv7/io.rs:187,198-201).
    // The C ABI itself accepts any T >= 1; pass reference_contract = false for decode steps.
    void check(bool reference_contract = true) const {
        if (!reference_contract) return;
        if (chunk_len != 16) throw KernelInputsError(RWKV7_ERR_BAD_CHUNK, "wkv7 currently supports chunk_len=16");
        if (receptance.t.ndim == 4 && receptance.t.shape[1] % chunk_len != 0)
            throw KernelInputsError(RWKV7_ERR_BAD_CHUNK, "context_len must be a multiple of chunk_len");
    }
};

// wkv7/io.rs:122-164
struct Wkv7StatepassForwardInputs {
    TensorView initial_state;
    Wkv7PretrainForwardInputs sequence;
};
struct Wkv7StatepassForwardOutput {
    TensorView output, next_state;
};

struct Workspace {
    void *data = nullptr;
    size_t bytes = 0;
};

inline size_t wkv7_workspace_bytes(const Wkv7PretrainForwardInputs &in) {
    const rwkv7_tensor &r = in.receptance.t;
    return r.ndim == 4 ? rwkv7_wkv7_workspace_bytes(r.shape[0], r.shape[1], r.shape[2], r.shape[3], r.dtype) : 0;
}

// wkv7_pretrain_custom (wkv7/mod.rs:105-110)
inline void wkv7_pretrain_custom(const Wkv7PretrainForwardInputs &in, TensorView &output, Workspace ws = {},
                                 rwkv7_stream stream = nullptr, bool reference_contract = true) {
    in.check(reference_contract);
    check_status(rwkv7_fused_wkv7_pretrain(in.receptance.c(), in.weight_decay.c(), in.replacement_key.c(),
                                           in.value.c(), in.removal_key_normalized.c(), in.replacement.c(),
                                           in.chunk_len, output.m(), ws.data, ws.bytes, stream));
}

// wkv7_statetune_custom (wkv7/mod.rs:113-120)
inline void wkv7_statetune_custom(const Wkv7StatepassForwardInputs &in, TensorView &output, Workspace ws = {},
                                  rwkv7_stream stream = nullptr, bool reference_contract = true) {
    in.sequence.check(reference_contract);
    const auto &s = in.sequence;
    check_status(rwkv7_fused_wkv7_statetune(in.initial_state.c(), s.receptance.c(), s.weight_decay.c(),
                                            s.replacement_key.c(), s.value.c(), s.removal_key_normalized.c(),
                                            s.replacement.c(), s.chunk_len, output.m(), ws.data, ws.bytes, stream));
}

// wkv7_statepass_custom (wkv7/mod.rs:123-133); out.next_state may view the same memory as in.initial_state.
inline void wkv7_statepass_custom(const Wkv7StatepassForwardInputs &in, Wkv7StatepassForwardOutput &out,
                                  Workspace ws = {}, rwkv7_stream stream = nullptr, bool reference_contract = true) {
    in.sequence.check(reference_contract);
    const auto &s = in.sequence;
    check_status(rwkv7_fused_wkv7_statepass(in.initial_state.c(), s.receptance.c(), s.weight_decay.c(),
                                            s.replacement_key.c(), s.value.c(), s.removal_key_normalized.c(),
                                            s.replacement.c(), s.chunk_len, out.output.m(), out.next_state.m(),
                                            ws.data, ws.bytes, stream));
}

// Statepass over tensors in pinned HOST memory (views with device = RWKV7_HOST): rwkv7_wkv7_statepass_host.
// `staging` is device memory of wkv7_host_staging_bytes(...) bytes, `streams` the caller's worker streams;
// with join = false the caller issues several passes back to back and calls wkv7_host_join once.
struct Wkv7HostPipeline {
    int32_t device = 0, slices = 1;
    Workspace staging;
    std::vector<rwkv7_stream> streams;
};
inline size_t wkv7_host_staging_bytes(const Wkv7PretrainForwardInputs &in, int32_t slices, int32_t n_streams) {
    const rwkv7_tensor &r = in.receptance.t;
    return r.ndim == 4 ? rwkv7_wkv7_host_staging_bytes(r.shape[0], r.shape[1], r.shape[2], r.shape[3], r.dtype, slices,
                                                       n_streams)
                       : 0;
}
inline void wkv7_statepass_host(const Wkv7StatepassForwardInputs &in, Wkv7StatepassForwardOutput &out,
                                const Wkv7HostPipeline &pipe, rwkv7_stream caller_stream = nullptr, bool join = true,
                                bool reference_contract = true) {
    in.sequence.check(reference_contract);
    const auto &s = in.sequence;
    const rwkv7_tensor *six[6] = {s.receptance.c(), s.weight_decay.c(), s.replacement_key.c(),
                                  s.value.c(), s.removal_key_normalized.c(), s.replacement.c()};
    check_status(rwkv7_wkv7_statepass_host(in.initial_state.c(), six, s.chunk_len, out.output.m(), out.next_state.m(),
                                           pipe.device, pipe.slices, pipe.staging.data, pipe.staging.bytes,
                                           pipe.streams.data(), (int32_t)pipe.streams.size(), caller_stream,
                                           join ? 0 : RWKV7_HOST_NO_JOIN));
}
inline void wkv7_host_join(const Wkv7HostPipeline &pipe, rwkv7_stream caller_stream = nullptr) {
    check_status(rwkv7_wkv7_host_join(pipe.device, pipe.streams.data(), (int32_t)pipe.streams.size(), caller_stream));
}

// ---- training: the tensors the autodiff nodes keep, and the backward pass ---------------------
// What launch_wkv7_*_forward returns under autodiff (wkv7/forward.rs:290-302) and what
// Wkv7BackwardState keeps (wkv7/backward.rs:549-559).
struct Wkv7SavedForward {
    TensorView output, next_state;             // next_state may be empty (pretrain, statetune)
    TensorView snapshots, state_replacement;   // F32 [B,H,T/chunk_len,N,N]; [B,T,H,N] like the inputs
};

// Forward pass of an autodiff node; initial_state may be empty (pretrain: S0 = 0).
inline void wkv7_forward_saved(const Wkv7StatepassForwardInputs &in, Wkv7SavedForward &out, Workspace ws = {},
                               rwkv7_stream stream = nullptr) {
    const auto &s = in.sequence;
    check_status(rwkv7_fused_wkv7_forward_saved(
        in.initial_state.t.data ? in.initial_state.c() : nullptr, s.receptance.c(), s.weight_decay.c(),
        s.replacement_key.c(), s.value.c(), s.removal_key_normalized.c(), s.replacement.c(), s.chunk_len,
        out.output.m(), out.next_state.t.data ? out.next_state.m() : nullptr, out.snapshots.m(),
        out.state_replacement.m(), ws.data, ws.bytes, stream));
}

// Wkv7BackwardPrimitiveOutputs (wkv7/backward.rs:567-575); initial_state_grad may be empty.
struct Wkv7BackwardOutputs {
    TensorView receptance_grad, weight_decay_grad, replacement_key_grad, value_grad, removal_key_normalized_grad,
        replacement_grad, initial_state_grad;
};

inline size_t wkv7_backward_workspace_bytes(const Wkv7PretrainForwardInputs &in) {
    const rwkv7_tensor &r = in.receptance.t;
    return r.ndim == 4 ? rwkv7_wkv7_backward_workspace_bytes(r.shape[0], r.shape[1], r.shape[2], r.shape[3]) : 0;
}

// launch_wkv7_backward (wkv7/backward.rs:583-703).  in.initial_state is the state the forward started from
// (empty = zero); next_state_grad may be empty (zero).  With a workspace of wkv7_backward_workspace_bytes the
// time-parallel form is used where it applies; without one, the token-by-token kernel.
inline void wkv7_backward(const Wkv7StatepassForwardInputs &in, const Wkv7SavedForward &saved,
                          const TensorView &output_grad, const TensorView &next_state_grad, Wkv7BackwardOutputs &out,
                          Workspace ws = {}, rwkv7_stream stream = nullptr) {
    const auto &s = in.sequence;
    rwkv7_tensor *grads[6] = {out.receptance_grad.m(), out.weight_decay_grad.m(), out.replacement_key_grad.m(),
                              out.value_grad.m(), out.removal_key_normalized_grad.m(), out.replacement_grad.m()};
    const rwkv7_tensor *s0 = in.initial_state.t.data ? in.initial_state.c() : nullptr;
    const rwkv7_tensor *dst = next_state_grad.t.data ? next_state_grad.c() : nullptr;
    rwkv7_tensor *ds0 = out.initial_state_grad.t.data ? out.initial_state_grad.m() : nullptr;
    if (ws.data != nullptr)
        check_status(rwkv7_fused_wkv7_backward_parallel(
            s0, s.receptance.c(), s.weight_decay.c(), s.replacement_key.c(), s.value.c(), s.removal_key_normalized.c(),
            s.replacement.c(), saved.snapshots.c(), saved.state_replacement.c(), s.chunk_len, output_grad.c(), dst,
            grads, ds0, ws.data, ws.bytes, stream));
    else
        check_status(rwkv7_fused_wkv7_backward(
            s0, s.receptance.c(), s.weight_decay.c(), s.replacement_key.c(), s.value.c(), s.removal_key_normalized.c(),
            s.replacement.c(), saved.snapshots.c(), saved.state_replacement.c(), s.chunk_len, output_grad.c(), dst,
            grads, ds0, stream));
}

// mix6/io.rs:20-46, 110-124: scales and outputs in the order receptance, weight_decay, key, value,
// learning_rate, gate.
struct Mix6ForwardInputs {
    TensorView embedded_context;
    std::array<TensorView, 6> scales;
};
struct Mix6ForwardOutput {
    std::array<TensorView, 6> inputs;
};

// mix6_custom (mix6/mod.rs:76-108)
inline void mix6_custom(const Mix6ForwardInputs &in, Mix6ForwardOutput &out, rwkv7_stream stream = nullptr) {
    const rwkv7_tensor *sc[6];
    rwkv7_tensor *o[6];
    for (int i = 0; i < 6; ++i) {
        sc[i] = in.scales[i].c();
        o[i] = out.inputs[i].m();
    }
    check_status(rwkv7_fused_mix6(in.embedded_context.c(), sc, o, stream));
}

// addcmul_custom (addcmul/mod.rs:100-105); `output` may view the same memory as `base`.
inline void addcmul_custom(const TensorView &base, const TensorView &diff, const TensorView &scale,
                           TensorView &output, rwkv7_stream stream = nullptr) {
    check_status(rwkv7_fused_addcmul(base.c(), diff.c(), scale.c(), output.m(), stream));
}

// addcmul5_custom (addcmul/mod.rs:138-157)
inline void addcmul5_custom(const TensorView &base, const TensorView &diff, const std::array<TensorView, 5> &scales,
                            std::array<TensorView, 5> &outputs, rwkv7_stream stream = nullptr) {
    const rwkv7_tensor *sc[5];
    rwkv7_tensor *o[5];
    for (int i = 0; i < 5; ++i) {
        sc[i] = scales[i].c();
        o[i] = outputs[i].m();
    }
    check_status(rwkv7_fused_addcmul5(base.c(), diff.c(), sc, o, stream));
}

// token_shift_diff_custom (token_shift_diff/mod.rs:82-111): `embedded_token_shift` is updated in place.
inline void token_shift_diff_custom(const TensorView &embedded_context, TensorView &embedded_token_shift,
                                    const TensorView &batch_ids, TensorView &token_shifted_diff,
                                    rwkv7_stream stream = nullptr) {
    check_status(rwkv7_fused_token_shift_diff(embedded_context.c(), embedded_token_shift.m(), batch_ids.c(),
                                              token_shifted_diff.m(), stream));
}

// Tail of WeightPrepare::forward (modules/time_mixer/weight_prepare.rs:252-287); field names
// follow WeightPrepareOutput (:289-297).  Leave the three value inputs and `value` default-constructed
// for the first cell.
struct WeightPrepareEpilogueInputs {
    TensorView key_precursor, learning_rate_lora, weight_decay_lora, key_removal, key_replacement;
    TensorView value_precursor, value_from_first_cell, value_residual_lora;
    int64_t num_heads = 0;
};
struct WeightPrepareEpilogueOutput {
    TensorView weight_decay, replacement_key, value, removal_key_normalized, replacement;
};
inline void weight_prepare_epilogue(const WeightPrepareEpilogueInputs &in, WeightPrepareEpilogueOutput &out,
                                    rwkv7_stream stream = nullptr) {
    const bool with_value = in.value_precursor.t.data != nullptr;
    check_status(rwkv7_fused_weight_prepare(
        in.key_precursor.c(), in.learning_rate_lora.c(), in.weight_decay_lora.c(), in.key_removal.c(),
        in.key_replacement.c(), with_value ? in.value_precursor.c() : nullptr,
        with_value ? in.value_from_first_cell.c() : nullptr, with_value ? in.value_residual_lora.c() : nullptr,
        in.num_heads, out.weight_decay.m(), out.replacement_key.m(), out.removal_key_normalized.m(),
        out.replacement.m(), with_value ? out.value.m() : nullptr, stream));
}

// GatedReadout::forward between the gate LoRA and the output projection
// (modules/time_mixer/gated_readout.rs:123-141); names follow GatedReadoutInput.
struct GatedReadoutEpilogueInputs {
    TensorView gate, wkv7_forward_output, wkv7_forward_input_receptance, wkv7_forward_input_replacement_key,
        wkv7_forward_input_value;
    TensorView group_norm_gamma, group_norm_beta, receptance_key_bonus;
    double epsilon = 64e-5;
    int64_t num_heads = 0;
};
inline void gated_readout_epilogue(const GatedReadoutEpilogueInputs &in, TensorView &output,
                                   rwkv7_stream stream = nullptr) {
    check_status(rwkv7_fused_gated_readout(
        in.wkv7_forward_output.c(), in.wkv7_forward_input_receptance.c(),
        in.wkv7_forward_input_replacement_key.c(), in.wkv7_forward_input_value.c(), in.gate.c(),
        in.group_norm_gamma.c(), in.group_norm_beta.c(), in.receptance_key_bonus.c(), in.epsilon, in.num_heads,
        output.m(), stream));
}

// ChannelMixerForwardInputs (kernels/train/channel_mixer/io.rs:17-22) and channel_mixer_custom
// (mod.rs:80-94).
struct ChannelMixerForwardInputs {
    TensorView embedded_context, key_scale, key_weight, value_weight;
};
inline size_t channel_mixer_workspace_bytes(const ChannelMixerForwardInputs &in) {
    const rwkv7_tensor &x = in.embedded_context.t;
    return x.ndim == 3 && in.key_weight.t.ndim == 2
               ? rwkv7_channel_mixer_workspace_bytes(x.shape[0], x.shape[1], x.shape[2], in.key_weight.t.shape[0])
               : 0;
}
inline void channel_mixer_custom(const ChannelMixerForwardInputs &in, TensorView &output, Workspace ws,
                                 rwkv7_stream stream = nullptr) {
    check_status(rwkv7_fused_channel_mixer(in.embedded_context.c(), in.key_scale.c(), in.key_weight.c(),
                                           in.value_weight.c(), output.m(), ws.data, ws.bytes, stream));
}

}  // namespace rwkv7b200

#endif  // RWKV7_B200_HPP_
