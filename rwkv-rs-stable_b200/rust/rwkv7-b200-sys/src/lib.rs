//! Raw declarations of `include/rwkv7_b200.h` (ABI version 1).
//!
//! Every entry borrows device pointers for the duration of the work it enqueues on `stream`,
//! allocates nothing, never synchronises the device, and returns an `rwkv7_status` code; codes
//! 1..=5 are `KernelInputsError` of `crates/rwkv-nn/src/kernels/check.rs:34-73` in declaration
//! order, and `rwkv7_last_error_message()` gives the text the reference's `Display` prints, which
//! is what the safe layer panics with (the public wrappers `unwrap()` the check,
//! `crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:106,116,126`).
#![no_std]
#![allow(non_camel_case_types)]

#[cfg(feature = "std")]
extern crate std;

use core::ffi::{c_char, c_int, c_void};

pub const RWKV7_MAX_DIMS: usize = 5;
pub const RWKV7_ABI_VERSION: c_int = 1;

/// `cudaStream_t`.
pub type rwkv7_stream = *mut c_void;

// rwkv7_dtype
pub const RWKV7_F32: i32 = 0;
pub const RWKV7_BF16: i32 = 1;
pub const RWKV7_F16: i32 = 2;
pub const RWKV7_I32: i32 = 3;
pub const RWKV7_I64: i32 = 4;
pub const RWKV7_U32: i32 = 5;

// rwkv7_status
pub const RWKV7_OK: c_int = 0;
pub const RWKV7_ERR_AXIS_MISMATCH: c_int = 1;
pub const RWKV7_ERR_SHAPE_MISMATCH: c_int = 2;
pub const RWKV7_ERR_DTYPE_MISMATCH: c_int = 3;
pub const RWKV7_ERR_DEVICE_MISMATCH: c_int = 4;
pub const RWKV7_ERR_EMPTY_AXIS: c_int = 5;
pub const RWKV7_ERR_NOT_CONTIGUOUS: c_int = 6;
pub const RWKV7_ERR_BAD_CHUNK: c_int = 7;
pub const RWKV7_ERR_UNSUPPORTED: c_int = 8;
pub const RWKV7_ERR_NULL_POINTER: c_int = 9;
pub const RWKV7_ERR_WORKSPACE_TOO_SMALL: c_int = 10;
pub const RWKV7_ERR_CUDA: c_int = 11;
pub const RWKV7_ERR_TIMEOUT: c_int = 12;
pub const RWKV7_ERR_BAD_INDEX: c_int = 13;
pub const RWKV7_ERR_BAD_ARGUMENT: c_int = 14;

// rwkv7_wkv7_path
pub const RWKV7_WKV7_AUTO: c_int = 0;
pub const RWKV7_WKV7_SEQUENTIAL: c_int = 1;
pub const RWKV7_WKV7_CHUNKED: c_int = 2;
pub const RWKV7_WKV7_SPLIT: c_int = 3;

/// `device` value of a tensor descriptor that lives in pinned host memory.
pub const RWKV7_HOST: i32 = -1;
/// `flags` bit of `rwkv7_wkv7_statepass_host`: leave the caller's stream unjoined.
pub const RWKV7_HOST_NO_JOIN: i32 = 1;

/// A borrowed tensor: what the safe layer fills from a `CubeTensor` (`handle` -> device pointer,
/// `meta.shape`, `meta.strides` in elements, `dtype`, device ordinal).
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rwkv7_tensor {
    pub data: *mut c_void,
    pub dtype: i32,
    pub device: i32,
    pub ndim: i32,
    pub reserved: i32,
    pub shape: [i64; RWKV7_MAX_DIMS],
    pub stride: [i64; RWKV7_MAX_DIMS],
}

impl rwkv7_tensor {
    /// Descriptor of a contiguous row-major tensor.
    pub fn contiguous(data: *mut c_void, dtype: i32, device: i32, dims: &[i64]) -> Self {
        assert!(dims.len() <= RWKV7_MAX_DIMS);
        let mut shape = [0i64; RWKV7_MAX_DIMS];
        let mut stride = [0i64; RWKV7_MAX_DIMS];
        let mut run = 1i64;
        for (i, &d) in dims.iter().enumerate().rev() {
            shape[i] = d;
            stride[i] = run;
            run *= d;
        }
        Self { data, dtype, device, ndim: dims.len() as i32, reserved: 0, shape, stride }
    }
}

type T = *const rwkv7_tensor;
type TM = *mut rwkv7_tensor;

extern "C" {
    // ---- library state and diagnostics
    pub fn rwkv7_abi_version() -> c_int;
    pub fn rwkv7_build_features() -> c_int;
    pub fn rwkv7_status_string(status: c_int) -> *const c_char;
    pub fn rwkv7_last_error_message() -> *const c_char;
    pub fn rwkv7_set_wkv7_path(path: c_int) -> c_int;
    pub fn rwkv7_get_wkv7_path() -> c_int;
    pub fn rwkv7_set_wkv7_cluster(cluster_size: c_int) -> c_int;
    pub fn rwkv7_set_wkv7_overlap(on: c_int) -> c_int;
    pub fn rwkv7_kernel_launch_count() -> i64;
    pub fn rwkv7_read_device_status(device: c_int, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_selftest_bounded_wait(device: c_int, max_polls: i64, stream: rwkv7_stream) -> c_int;

    // ---- Wkv7Backend (wkv7/mod.rs:29-41)
    pub fn rwkv7_wkv7_workspace_bytes(b: i64, t: i64, h: i64, n: i64, dtype: i32) -> usize;
    pub fn rwkv7_fused_wkv7_pretrain(receptance: T, weight_decay: T, replacement_key: T, value: T,
        removal_key_normalized: T, replacement: T, chunk_len: i64, output: TM,
        workspace: *mut c_void, workspace_bytes: usize, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_wkv7_statetune(initial_state: T, receptance: T, weight_decay: T, replacement_key: T,
        value: T, removal_key_normalized: T, replacement: T, chunk_len: i64, output: TM,
        workspace: *mut c_void, workspace_bytes: usize, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_wkv7_statepass(initial_state: T, receptance: T, weight_decay: T, replacement_key: T,
        value: T, removal_key_normalized: T, replacement: T, chunk_len: i64, output: TM, next_state: TM,
        workspace: *mut c_void, workspace_bytes: usize, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_wkv7_statepass_noalloc(initial_state: T, receptance: T, weight_decay: T,
        replacement_key: T, value: T, removal_key_normalized: T, replacement: T, chunk_len: i64,
        output: TM, next_state: TM, stream: rwkv7_stream) -> c_int;

    // ---- the same call over pinned host tensors (copies pipelined with the kernels)
    pub fn rwkv7_wkv7_host_staging_bytes(b: i64, t: i64, h: i64, n: i64, dtype: i32, slices: i32,
        n_streams: i32) -> usize;
    pub fn rwkv7_wkv7_statepass_host(host_initial_state: T, host_six: *const T, chunk_len: i64,
        host_output: TM, host_next_state: TM, device: i32, slices: i32, device_staging: *mut c_void,
        staging_bytes: usize, streams: *const rwkv7_stream, n_streams: i32, caller_stream: rwkv7_stream,
        flags: i32) -> c_int;
    pub fn rwkv7_wkv7_host_join(device: i32, streams: *const rwkv7_stream, n_streams: i32,
        caller_stream: rwkv7_stream) -> c_int;

    // ---- training (wkv7/forward.rs:290-302, wkv7/backward.rs:158-527)
    pub fn rwkv7_fused_wkv7_forward_saved(initial_state: T, receptance: T, weight_decay: T,
        replacement_key: T, value: T, removal_key_normalized: T, replacement: T, chunk_len: i64,
        output: TM, next_state: TM, snapshots: TM, state_replacement: TM, workspace: *mut c_void,
        workspace_bytes: usize, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_wkv7_backward(initial_state: T, receptance: T, weight_decay: T, replacement_key: T,
        value: T, removal_key_normalized: T, replacement: T, snapshots: T, state_replacement: T,
        chunk_len: i64, output_grad: T, next_state_grad: T, sequence_grads: *const TM,
        initial_state_grad: TM, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_wkv7_backward_workspace_bytes(b: i64, t: i64, h: i64, n: i64) -> usize;
    pub fn rwkv7_fused_wkv7_backward_parallel(initial_state: T, receptance: T, weight_decay: T,
        replacement_key: T, value: T, removal_key_normalized: T, replacement: T, snapshots: T,
        state_replacement: T, chunk_len: i64, output_grad: T, next_state_grad: T,
        sequence_grads: *const TM, initial_state_grad: TM, workspace: *mut c_void,
        workspace_bytes: usize, stream: rwkv7_stream) -> c_int;

    // ---- Mix6Backend, AddcmulBackend, TokenShiftDiffBackend
    pub fn rwkv7_fused_mix6(embedded_context: T, scales: *const T, outputs: *const TM,
        stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_mix6_stacked(embedded_context: T, scales: *const T, stacked_output: TM,
        stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_addcmul(base: T, diff: T, scale: T, output: TM, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_addcmul5(base: T, diff: T, scales: *const T, outputs: *const TM,
        stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_token_shift_diff(embedded_context: T, embedded_token_shift: TM, batch_ids: T,
        token_shifted_diff: TM, stream: rwkv7_stream) -> c_int;

    // ---- time-mixer epilogues and the channel mixer
    pub fn rwkv7_fused_weight_prepare(key_precursor: T, learning_rate_lora: T, weight_decay_lora: T,
        key_removal: T, key_replacement: T, value_precursor: T, value_from_first_cell: T,
        value_residual_lora: T, num_heads: i64, weight_decay: TM, replacement_key: TM,
        removal_key_normalized: TM, replacement: TM, value: TM, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_fused_gated_readout(wkv7_output: T, receptance: T, replacement_key: T, value: T, gate: T,
        group_norm_gamma: T, group_norm_beta: T, receptance_key_bonus: T, epsilon: f64, num_heads: i64,
        output: TM, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_channel_mixer_workspace_bytes(b: i64, t: i64, c: i64, f: i64) -> usize;
    pub fn rwkv7_fused_channel_mixer(embedded_context: T, key_scale: T, key_weight: T, value_weight: T,
        output: TM, workspace: *mut c_void, workspace_bytes: usize, stream: rwkv7_stream) -> c_int;

    // ---- LM-head cross-entropy (vocabulary shards; combine on the caller's side)
    pub fn rwkv7_lm_head_ce_workspace_bytes(r: i64, c: i64, v_shard: i64) -> usize;
    pub fn rwkv7_fused_lm_head_ce_partial(x: T, weight_shard: T, targets: T, vocab_offset: i64,
        partials: TM, workspace: *mut c_void, workspace_bytes: usize, stream: rwkv7_stream) -> c_int;
    pub fn rwkv7_lm_head_ce_finalize(partials_all: T, targets: T, lse: TM, loss: TM,
        stream: rwkv7_stream) -> c_int;
}

/// The message a failed call left for this thread, as the reference's error `Display` prints it.
///
/// # Safety
/// Calls into the library; the returned text is copied out before any other call can replace it.
#[cfg(feature = "std")]
pub unsafe fn last_error() -> std::string::String {
    std::ffi::CStr::from_ptr(rwkv7_last_error_message()).to_string_lossy().into_owned()
}
