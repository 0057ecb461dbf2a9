/*
 * rwkv7_b200.h — C ABI of the B200 (sm_100a) implementation of the rwkv-rs WKV7
 * hot path: the fused WKV7 forward recurrence, the token-shift mixing kernels
 * (mix6, addcmul, addcmul5, token_shift_diff) and the fused LM-head cross
 * entropy.
 *
 * Every entry point replaces the body of one backend-extension trait function
 * of the reference (paths inside the rwkv-rs repository are cited per function).
 * Conventions shared by all entry points:
 *
 *  - Tensors are BORROWED: `data` is a device pointer owned by the caller, valid
 *    until the work enqueued on `stream` has completed.  The library allocates
 *    no tensor memory; outputs and workspaces are caller-allocated (the
 *    reference allocates outputs with `empty_device` inside the op,
 *    wkv7/forward.rs:368-375 — the Rust shim does that before calling in).
 *  - Work is enqueued on `stream` and is asynchronous with respect to the host
 *    (the reference enqueues on the CubeCL client's stream).  No entry point
 *    synchronises the device, except rwkv7_read_device_status.
 *  - The return value is a status code.  Non-zero codes 1..5 map 1:1 onto the
 *    reference's `KernelInputsError` variants (kernels/check.rs:34-73) and
 *    rwkv7_last_error_message() returns the same Display text the reference
 *    would panic with; the reference's wrappers `check().unwrap()` and panic, a
 *    Rust shim does `panic!("{}", rwkv7_last_error_message())` on non-zero.
 *  - All tensors must be contiguous row-major (the reference asserts
 *    `is_contiguous()`, wkv7/mod.rs:56-76).
 *  - The compute entry points are re-entrant: a call keeps no state of its own
 *    beyond a thread-local error message and a per-device status word.  Two
 *    process-wide switches exist for tests and benchmarks, rwkv7_set_wkv7_path
 *    and rwkv7_set_wkv7_cluster; they are atomics read once per call, they
 *    change which kernel a later call on ANY thread takes (and, for the path,
 *    what rwkv7_wkv7_workspace_bytes reports), and a process that never calls
 *    them gets the automatic choice everywhere.  Per-device caches (SM count,
 *    resident-cluster counts, the status word, the address of the fixed scratch
 *    array) are filled once under a mutex.
 */
#ifndef RWKV7_B200_H_
#define RWKV7_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RWKV7_MAX_DIMS 5
#define RWKV7_ABI_VERSION 1

/* Opaque CUDA stream handle (cudaStream_t); NULL is the legacy default stream. */
typedef void *rwkv7_stream;

typedef enum rwkv7_dtype {
    RWKV7_F32 = 0,
    RWKV7_BF16 = 1,
    RWKV7_F16 = 2, /* recognised, not computed: returns RWKV7_ERR_UNSUPPORTED */
    RWKV7_I32 = 3,
    RWKV7_I64 = 4,
    RWKV7_U32 = 5
} rwkv7_dtype;

typedef enum rwkv7_status {
    RWKV7_OK = 0,
    /* 1..5: KernelInputsError variants, kernels/check.rs:34-73 */
    RWKV7_ERR_AXIS_MISMATCH = 1,
    RWKV7_ERR_SHAPE_MISMATCH = 2,
    RWKV7_ERR_DTYPE_MISMATCH = 3,
    RWKV7_ERR_DEVICE_MISMATCH = 4,
    RWKV7_ERR_EMPTY_AXIS = 5,
    /* assertions of the reference's CubeBackend impl and io.rs */
    RWKV7_ERR_NOT_CONTIGUOUS = 6, /* wkv7/mod.rs:56-76 */
    RWKV7_ERR_BAD_CHUNK = 7,      /* wkv7/io.rs:187,198-201 (only chunk_len <= 0 here) */
    /* conditions that have no counterpart in the reference */
    RWKV7_ERR_UNSUPPORTED = 8,
    RWKV7_ERR_NULL_POINTER = 9,
    RWKV7_ERR_WORKSPACE_TOO_SMALL = 10,
    RWKV7_ERR_CUDA = 11,
    RWKV7_ERR_TIMEOUT = 12,    /* a bounded device-side wait expired */
    RWKV7_ERR_BAD_INDEX = 13,  /* a device-side index (batch_ids, target) was out of range */
    RWKV7_ERR_BAD_ARGUMENT = 14
} rwkv7_status;

/* Borrowed tensor view.  `stride` is in elements; `device` is the CUDA ordinal. */
typedef struct rwkv7_tensor {
    void *data;
    int32_t dtype; /* rwkv7_dtype */
    int32_t device;
    int32_t ndim;
    int32_t reserved;
    int64_t shape[RWKV7_MAX_DIMS];
    int64_t stride[RWKV7_MAX_DIMS];
} rwkv7_tensor;

/* Which kernel the WKV7 entry points dispatch to.  AUTO picks the decode sweep for T <= 4; for N == 64 and
 * BF16 or F32 tensors the two-kernel tensor-core prefill (SPLIT: per-chunk operators in fp16, then one scan per
 * chain) from 512 tokens on when the workspace holds at least one chunk of operators per chain; for BF16 tensors
 * otherwise the fused tf32 chunked kernel (CHUNKED) from 64 tokens on; the sequential kernel for everything else
 * (F32 tensors under 512 tokens, other head sizes).  Chains that the fp16 operators of SPLIT cannot resolve (a
 * chunk's log-decay beyond 18 in some channel, or a non-finite operator) are recomputed by CHUNKED (BF16 tensors),
 * and chains beyond its range (80), or flagged chains of F32 tensors, by SEQUENTIAL, inside the same call; a final
 * state that aliases the initial state is only written once a chain's result is final. */
typedef enum rwkv7_wkv7_path {
    RWKV7_WKV7_AUTO = 0,
    RWKV7_WKV7_SEQUENTIAL = 1,
    RWKV7_WKV7_CHUNKED = 2,
    RWKV7_WKV7_SPLIT = 3
} rwkv7_wkv7_path;

int rwkv7_abi_version(void);
/* Bit 0: built with -DRWKV7_NVTX (every compute entry point opens an NVTX range named after the reference's
 * tracing span of the calling module, e.g. "rwkv.infer.model.time_mixer.wkv7" for
 * crates/rwkv-nn/src/modules/time_mixer/mod.rs:153-156).  Bit 1: built with -DRWKV7_CHECKED (device code
 * verifies tile rows, output rows and workspace slots before using them and reports RWKV7_ERR_BAD_INDEX
 * through rwkv7_read_device_status instead of performing a bad access).  The product build returns 0. */
int rwkv7_build_features(void);
const char *rwkv7_status_string(int status);
/* Thread-local text of the last non-zero status returned on this thread. */
const char *rwkv7_last_error_message(void);
/* Process-wide override of the WKV7 kernel choice (tests and benchmarks).  It also changes
 * what rwkv7_wkv7_workspace_bytes reports (the sequential path needs none), so size the
 * workspace after setting it, and do not flip it while calls are in flight on other threads. */
int rwkv7_set_wkv7_path(int path);
int rwkv7_get_wkv7_path(void);

/* The chunked prefill kernel gives a chain to a thread-block cluster of 2 or 4 CTAs when there
 * are at most half / a quarter as many (b,h) chains as SMs (small-batch prefill): the CTAs take
 * the chunks in turn, prepare everything that does not depend on the state ahead of time and
 * pass only the state through distributed shared memory.  With more chains than SMs the chains
 * of a last, at most half-full wave are launched the same way (a second launch on the same
 * stream).  Results of a chain depend on its cluster size in the last bits (a few 1e-5 to 1e-4 of
 * the largest entry).  0 restores that automatic choice; 1, 2 or 4 force a cluster size for every
 * chain (1 makes results independent of how many chains a call holds).  Process-wide. */
int rwkv7_set_wkv7_cluster(int cluster_size);
/* The two-kernel prefill cuts a long call into segments of chunks.  With few chains (at most 27 % as many as
 * SMs) and at least 192 chunks (128 with very few chains), the scan of a segment (one latency-bound CTA per chain) runs beside the operator
 * kernel of the next segment: the device's SMs are split once into two partitions (CUDA green contexts: the
 * scans on as many SMs as chains, rounded up to eight, the operator kernels on the rest), each with a
 * library-owned stream; events order the two streams and the caller's stream continues after the last scan, so
 * the call keeps its stream semantics.  Where the driver offers no partitions, or a profiler is injected into the
 * process (Nsight Compute cannot profile kernels in green contexts), calls of 24 to 40 chains (on 148
 * SMs) use a second stream of the primary context instead, the scan CTAs beside operator CTAs.  Partitions,
 * streams and events are created per device on the first such call and kept until the process exits; the
 * enqueueing of overlapped calls is serialised per process.  0 puts every kernel on the caller's stream (same
 * results, bitwise), 1 is the schedule described (default), 2 forces the second-stream schedule without
 * partitions.  Process-wide. */
int rwkv7_set_wkv7_overlap(int on);
/* Number of kernels this library has launched in this process (all devices,
 * all threads).  Benchmarks read it before and after a timed region. */
int64_t rwkv7_kernel_launch_count(void);

/*
 * Reads and clears the status word that kernels on `device` set instead of
 * trapping (expired bounded wait, out-of-range index).  Synchronises `stream`.
 * Returns RWKV7_OK, RWKV7_ERR_TIMEOUT or RWKV7_ERR_BAD_INDEX.
 */
int rwkv7_read_device_status(int device, rwkv7_stream stream);

/* No counterpart in the reference.  Launches one thread that waits, for at most max_polls
 * polls (1 .. 1000000), on a barrier that nothing signals, records the time-out in the device
 * status word and returns: the error path of every bounded wait in this library, exercised
 * without hanging or faulting anything.  rwkv7_read_device_status then returns
 * RWKV7_ERR_TIMEOUT once, and the device stays usable. */
int rwkv7_selftest_bounded_wait(int device, int64_t max_polls, rwkv7_stream stream);

/* ------------------------------------------------------------------ WKV7 -- */
/*
 * Per (b,h), state S[i][j] (i value row, j key column), t = 0..T-1:
 *   d_j = exp(-exp(w[b,t,h,j]));  sa_i = sum_j S[i][j] a[b,t,h,j];
 *   S[i][j] = S[i][j] d_j + sa_i b[b,t,h,j] + v[b,t,h,i] k[b,t,h,j];
 *   y[b,t,h,i] = sum_j S[i][j] r[b,t,h,j].
 * r,w,k,v,a,b,y are [B,T,H,N] (receptance, weight_decay, replacement_key, value,
 * removal_key_normalized, replacement), all F32 or all BF16; states are
 * [B,H,N,N] F32.  Accumulation and the carried state are fp32.
 *
 * `chunk_len` is the reference's snapshot cadence (wkv7/io.rs:187); here it must
 * only be positive, any T >= 1 is accepted (T == 1 is the decode step).
 * `workspace` may be NULL when rwkv7_wkv7_workspace_bytes() returns 0.
 */

/* Scratch bytes the WKV7 entry points prefer for this shape (0 for the sequential and decode kernels; B*H*4
 * for the tf32 chunked kernel; for the two-kernel prefill the flags, 1024 work counters, a carried state per
 * chain and 32.5 KB per 64-token chunk of a segment of the call, at most 768 MB of operators).  A smaller
 * workspace is accepted: the call is cut into more segments, and below one chunk per chain the tf32 kernel
 * (BF16 tensors) or the sequential scan runs instead.  The size depends on the SM count of the calling thread's
 * current device. */
size_t rwkv7_wkv7_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N, int32_t dtype);

/* Replaces Wkv7Backend::fused_wkv7_pretrain (wkv7/mod.rs:31, impl :55-79;
 * host wkv7/forward.rs:348-435; kernel wkv7/kernel.rs:60-196): S0 = 0 -> y. */
int rwkv7_fused_wkv7_pretrain(const rwkv7_tensor *receptance, const rwkv7_tensor *weight_decay,
                              const rwkv7_tensor *replacement_key, const rwkv7_tensor *value,
                              const rwkv7_tensor *removal_key_normalized,
                              const rwkv7_tensor *replacement, int64_t chunk_len,
                              rwkv7_tensor *output, void *workspace, size_t workspace_bytes,
                              rwkv7_stream stream);

/* Replaces Wkv7Backend::fused_wkv7_statetune (wkv7/mod.rs:34-35, impl :81-90;
 * wkv7/forward.rs:205-223): S0 given -> y, final state dropped. */
int rwkv7_fused_wkv7_statetune(const rwkv7_tensor *initial_state, const rwkv7_tensor *receptance,
                               const rwkv7_tensor *weight_decay,
                               const rwkv7_tensor *replacement_key, const rwkv7_tensor *value,
                               const rwkv7_tensor *removal_key_normalized,
                               const rwkv7_tensor *replacement, int64_t chunk_len,
                               rwkv7_tensor *output, void *workspace, size_t workspace_bytes,
                               rwkv7_stream stream);

/* Replaces Wkv7Backend::fused_wkv7_statepass (wkv7/mod.rs:38-40, impl :92-101;
 * wkv7/forward.rs:245-267,437-530; kernel wkv7/kernel.rs:198-364):
 * S0 given -> (y, S_T).  `next_state` may alias `initial_state`. */
int rwkv7_fused_wkv7_statepass(const rwkv7_tensor *initial_state, const rwkv7_tensor *receptance,
                               const rwkv7_tensor *weight_decay,
                               const rwkv7_tensor *replacement_key, const rwkv7_tensor *value,
                               const rwkv7_tensor *removal_key_normalized,
                               const rwkv7_tensor *replacement, int64_t chunk_len,
                               rwkv7_tensor *output, rwkv7_tensor *next_state, void *workspace,
                               size_t workspace_bytes, rwkv7_stream stream);

/* This entry point has no counterpart in the reference.  It is
 * rwkv7_fused_wkv7_statepass for callers that cannot allocate device memory at
 * the moment they call in and therefore have no workspace to pass: for example a
 * serving process whose own memory pool has already claimed the whole GPU, so that
 * a cudaMalloc at call time would fail, or a host runtime in which a device
 * allocation is not allowed on the calling thread because it would stall every
 * stream of the device.  The per-chain fallback flags of the chunked kernel live
 * in a fixed array inside the library image instead (256 KiB, held by every GPU
 * that loads the library until the process exits), so the call itself performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * Limits and rules:
 *  - B*H must not exceed 65536 chains; larger shapes return RWKV7_ERR_UNSUPPORTED.
 *  - The first call on each device resolves the array's device address
 *    (cudaGetSymbolAddress, with that device made current for the call); make
 *    that first call before starting any stream capture on the device.
 *  - All calls on a device share the one array and it keeps the previous call's
 *    contents.  Nothing in it has to start at zero (every call overwrites the
 *    flags of its own chains before reading them), but two calls whose GPU work
 *    overlaps (different streams, or different host threads) race on it:
 *    serialise calls to this entry point per device.
 * Inputs, outputs and results are those of rwkv7_fused_wkv7_statepass. */
int rwkv7_fused_wkv7_statepass_noalloc(const rwkv7_tensor *initial_state,
                                       const rwkv7_tensor *receptance,
                                       const rwkv7_tensor *weight_decay,
                                       const rwkv7_tensor *replacement_key,
                                       const rwkv7_tensor *value,
                                       const rwkv7_tensor *removal_key_normalized,
                                       const rwkv7_tensor *replacement, int64_t chunk_len,
                                       rwkv7_tensor *output, rwkv7_tensor *next_state,
                                       rwkv7_stream stream);

/* ---------------------------------------------- wkv7 from host buffers -- */
/*
 * Statepass for callers whose six sequence tensors, y and the states live in
 * PINNED HOST memory (an inference server that receives activations from another
 * process; the end-to-end leg of the benchmark).  No counterpart in the reference,
 * whose tensors are device-resident; the arithmetic is rwkv7_fused_wkv7_statepass.
 *
 * The batch is cut into `slices` equal parts.  Slice i uses streams[i % n_streams]
 * for its host-to-device copies (one cudaMemcpyAsync per tensor), its kernels and its
 * device-to-host copies, so the copies of one slice overlap the kernels and the
 * copy-back of the slices before it.  (b,h) chains are independent, so slicing the
 * batch changes no arithmetic.
 *
 * Host tensors are described like device tensors, with `device` = RWKV7_HOST and a
 * pointer that the CUDA device can copy from asynchronously (page-locked memory).
 * host_initial_state may be NULL (zero state).  `device_staging` is caller-allocated
 * device memory of rwkv7_wkv7_host_staging_bytes(...) bytes, 256-byte aligned,
 * borrowed until the enqueued work has run; it holds n_streams sets of slice
 * tensors and the kernels' workspace.  The library creates and destroys a few CUDA
 * events per call and allocates nothing else.
 *
 * Ordering: the work is ordered after everything enqueued on `caller_stream` so far.
 * Without RWKV7_HOST_NO_JOIN, `caller_stream` is made to wait for all of it, so a
 * synchronisation on `caller_stream` marks completion.  With the flag the caller
 * issues several passes back to back (each pass still starts after the previous
 * one's work on the same stream set, so host buffers are written in order) and calls
 * rwkv7_wkv7_host_join once at the end.
 */
#define RWKV7_HOST (-1)
#define RWKV7_HOST_NO_JOIN 1
size_t rwkv7_wkv7_host_staging_bytes(int64_t B, int64_t T, int64_t H, int64_t N, int32_t dtype,
                                     int32_t slices, int32_t n_streams);
int rwkv7_wkv7_statepass_host(const rwkv7_tensor *host_initial_state,
                              const rwkv7_tensor *const host_six[6], int64_t chunk_len,
                              rwkv7_tensor *host_output, rwkv7_tensor *host_next_state,
                              int32_t device, int32_t slices, void *device_staging,
                              size_t staging_bytes, const rwkv7_stream *streams, int32_t n_streams,
                              rwkv7_stream caller_stream, int32_t flags);
/* Makes `caller_stream` wait for everything enqueued so far on the given streams. */
int rwkv7_wkv7_host_join(int32_t device, const rwkv7_stream *streams, int32_t n_streams,
                         rwkv7_stream caller_stream);

/* ------------------------------------------------------- wkv7 training -- */
/*
 * The forward pass as the reference runs it under autodiff: the recurrence of
 * rwkv7_fused_wkv7_statepass plus the two tensors its backward pass consumes
 * (wkv7/forward.rs:368-375,460-472; written by kernel.rs:60-196,198-364):
 *   snapshots         [B, H, T/chunk_len, N, N]  the state after the last token of every chunk
 *                     (index order kernel.rs:40-53); F32 here, where the reference stores
 *                     the sequence dtype
 *   state_replacement [B, T, H, N]  sa_t = S_{t-1} a_t, sequence dtype.
 * initial_state may be NULL (pretrain: S0 = 0) and next_state may be NULL (pretrain,
 * statetune).  T must be a multiple of chunk_len (the reference also asserts chunk_len == 16;
 * any positive value is accepted here).  With chunk_len 16, N = 64 and BF16 tensors the
 * tensor-core prefill kernel computes the saved tensors as well (state_replacement is its U,
 * the snapshots are partial sums of its state update); it needs the workspace of
 * rwkv7_wkv7_workspace_bytes.  Everything else takes the sequential scan.
 */
int rwkv7_fused_wkv7_forward_saved(const rwkv7_tensor *initial_state, const rwkv7_tensor *receptance,
                                   const rwkv7_tensor *weight_decay,
                                   const rwkv7_tensor *replacement_key, const rwkv7_tensor *value,
                                   const rwkv7_tensor *removal_key_normalized,
                                   const rwkv7_tensor *replacement, int64_t chunk_len,
                                   rwkv7_tensor *output, rwkv7_tensor *next_state,
                                   rwkv7_tensor *snapshots, rwkv7_tensor *state_replacement,
                                   void *workspace, size_t workspace_bytes, rwkv7_stream stream);

/*
 * Replaces launch_wkv7_backward / wkv7_backward_kernel (wkv7/backward.rs:583-703,
 * kernel.rs:395-690): gradients of the six sequence tensors and of the initial state, given
 * the gradient of y (output_grad) and of the final state (next_state_grad, NULL = zero).
 * sequence_grads are in the order receptance, weight_decay, replacement_key, value,
 * removal_key_normalized, replacement (Wkv7BackwardPrimitiveOutputs, backward.rs:567-575);
 * state gradients are F32 [B,H,N,N]; initial_state_grad may be NULL.  initial_state is the
 * state the forward started from (NULL = zero): the reference rebuilds the state before each
 * token by dividing by the decay going backwards (kernel.rs:516-521), which loses all accuracy
 * for small decays; here each chunk is replayed forwards from the snapshot at its start
 * instead, which needs the initial state for the first chunk.  N <= 64; chunk_len 4, 8, 12 or 16.
 */
int rwkv7_fused_wkv7_backward(const rwkv7_tensor *initial_state, const rwkv7_tensor *receptance,
                              const rwkv7_tensor *weight_decay, const rwkv7_tensor *replacement_key,
                              const rwkv7_tensor *value,
                              const rwkv7_tensor *removal_key_normalized,
                              const rwkv7_tensor *replacement, const rwkv7_tensor *snapshots,
                              const rwkv7_tensor *state_replacement, int64_t chunk_len,
                              const rwkv7_tensor *output_grad, const rwkv7_tensor *next_state_grad,
                              rwkv7_tensor *const sequence_grads[6],
                              rwkv7_tensor *initial_state_grad, rwkv7_stream stream);

/*
 * The same gradients in time-parallel form; no counterpart in the reference, whose backward
 * kernel takes T dependent steps per (b,h) chain.  The recurrence of the state gradient is a
 * forward WKV7 recurrence over the reversed sequence (decay w_t, removal key b_t, replacement
 * a_t, value dy_t, key r_t d_t + (r_t.b_t) a_t, starting from next_state_grad), so it runs on
 * the tensor-core prefill kernel; its saved tensors then let every 16-token chunk be finished
 * independently of all others.  Taken for BF16 tensors with N = 64, chunk_len 16 and T >= 64;
 * any other shape is handled exactly like rwkv7_fused_wkv7_backward and needs no workspace.
 * workspace: rwkv7_wkv7_backward_workspace_bytes(B,T,H,N) bytes, 256-byte aligned, borrowed
 * until the enqueued work has finished (0 is returned for shapes that need none).
 */
size_t rwkv7_wkv7_backward_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t N);
int rwkv7_fused_wkv7_backward_parallel(const rwkv7_tensor *initial_state, const rwkv7_tensor *receptance,
                                       const rwkv7_tensor *weight_decay, const rwkv7_tensor *replacement_key,
                                       const rwkv7_tensor *value,
                                       const rwkv7_tensor *removal_key_normalized,
                                       const rwkv7_tensor *replacement, const rwkv7_tensor *snapshots,
                                       const rwkv7_tensor *state_replacement, int64_t chunk_len,
                                       const rwkv7_tensor *output_grad, const rwkv7_tensor *next_state_grad,
                                       rwkv7_tensor *const sequence_grads[6],
                                       rwkv7_tensor *initial_state_grad, void *workspace,
                                       size_t workspace_bytes, rwkv7_stream stream);

/* ------------------------------------------------------------------ mix6 -- */
/* Replaces Mix6Backend::fused_mix6 (mix6/mod.rs:25-28, impl :42-73; kernel
 * mix6/kernel.rs:25-57): prev = x[b,t-1,:] (0 at t == 0);
 * out_i = x + (prev - x) * scale_i for i in receptance, weight_decay, key,
 * value, learning_rate, gate.  x and out_i are [B,T,C], scale_i [1,1,C]. */
int rwkv7_fused_mix6(const rwkv7_tensor *embedded_context, const rwkv7_tensor *const scales[6],
                     rwkv7_tensor *const outputs[6], rwkv7_stream stream);

/* Same arithmetic into one stacked tensor [6,B,T,C] (the reference's
 * mix6_stacked_forward_kernel, mix6/kernel.rs:64-98, used under autodiff). */
int rwkv7_fused_mix6_stacked(const rwkv7_tensor *embedded_context,
                             const rwkv7_tensor *const scales[6], rwkv7_tensor *stacked_output,
                             rwkv7_stream stream);

/* --------------------------------------------------------------- addcmul -- */
/* Replaces AddcmulBackend::fused_addcmul (addcmul/mod.rs:27-35, impl :49-66;
 * kernel addcmul/kernel.rs:4-20): out = base + diff * scale; base, diff, out
 * [B,T,C], scale [1,1,C].  `output` may alias `base` (the reference writes in
 * place when the buffer is uniquely owned, addcmul/forward.rs:547-598). */
int rwkv7_fused_addcmul(const rwkv7_tensor *base, const rwkv7_tensor *diff,
                        const rwkv7_tensor *scale, rwkv7_tensor *output, rwkv7_stream stream);

/* Replaces AddcmulBackend::fused_addcmul5 (addcmul/mod.rs:27-35, impl :68-84;
 * kernel addcmul/kernel.rs:42-65): five outputs sharing base and diff, scale
 * order receptance, weight_decay, key, value, learning_rate. */
int rwkv7_fused_addcmul5(const rwkv7_tensor *base, const rwkv7_tensor *diff,
                         const rwkv7_tensor *const scales[5], rwkv7_tensor *const outputs[5],
                         rwkv7_stream stream);

/* ------------------------------------------------------ token_shift_diff -- */
/* Replaces TokenShiftDiffBackend::fused_token_shift_diff
 * (token_shift_diff/mod.rs:27-32, impl :42-63; kernel kernel.rs:16-45):
 *   prev[b,0,:] = state[ids[b],:]; prev[b,t,:] = x[b,t-1,:]; diff = prev - x;
 *   state[ids[b],:] = x[b,T-1,:]   (in place; other rows untouched; T == 0: no-op).
 * x, diff [B,T,C]; state [S,C]; batch_ids [B] of I32, I64 or U32, values valid
 * and unique.  An out-of-range id is skipped and reported through
 * rwkv7_read_device_status (the reference does not check). */
int rwkv7_fused_token_shift_diff(const rwkv7_tensor *embedded_context,
                                 rwkv7_tensor *embedded_token_shift,
                                 const rwkv7_tensor *batch_ids, rwkv7_tensor *token_shifted_diff,
                                 rwkv7_stream stream);

/* -------------------------------------------------- time-mixer epilogues -- */
/*
 * The tail of WeightPrepare::forward (modules/time_mixer/weight_prepare.rs:252-287,
 * functions/normalize.rs:9-41, functions/lerp.rs:4-10) in one pass.  The reference
 * has no single operator for it: these are the tensor ops between the dense
 * projections / LoRA products and the WKV7 call.  With lr = sigmoid(learning_rate_lora):
 *   replacement_key        = key_precursor * (key_replacement * (lr - 1) + 1)
 *   weight_decay           = -softplus(-weight_decay_lora) - 0.5
 *   removal_key_normalized = -(key_precursor * key_removal) / max(||.||_2 over the head, 1e-12)
 *   replacement            = -removal_key_normalized * lr
 *   value                  = value_precursor + (value_from_first_cell - value_precursor)
 *                            * sigmoid(value_residual_lora)       (cells after the first)
 * The big tensors are [B,T,C] (or [B,T,H,N], the same memory) with C = num_heads * N;
 * key_removal and key_replacement hold C elements ([1,1,C]).  The three value inputs
 * and `value` are either all given or all NULL (first cell: value = value_precursor,
 * nothing to compute).  Arithmetic is fp32, each output rounded once.
 */
int rwkv7_fused_weight_prepare(const rwkv7_tensor *key_precursor,
                               const rwkv7_tensor *learning_rate_lora,
                               const rwkv7_tensor *weight_decay_lora,
                               const rwkv7_tensor *key_removal,
                               const rwkv7_tensor *key_replacement,
                               const rwkv7_tensor *value_precursor,
                               const rwkv7_tensor *value_from_first_cell,
                               const rwkv7_tensor *value_residual_lora, int64_t num_heads,
                               rwkv7_tensor *weight_decay, rwkv7_tensor *replacement_key,
                               rwkv7_tensor *removal_key_normalized, rwkv7_tensor *replacement,
                               rwkv7_tensor *value, rwkv7_stream stream);

/*
 * The body of GatedReadout::forward between the gate LoRA and the output projection
 * (modules/time_mixer/gated_readout.rs:110-145) in one pass:
 *   norm   = GroupNorm(num_groups = num_heads, eps = epsilon; the module uses 64e-5)
 *            of wkv7_output per (b,t): (y - mean_h) / sqrt(var_h + eps) * gamma + beta,
 *            mean and (biased) variance over the N channels of head h
 *   bonus  = (sum_n receptance * replacement_key * receptance_key_bonus[h,n]) * value
 *   output = (norm + bonus) * gate
 * Big tensors [B,T,C] or [B,T,H,N]; group_norm_gamma, group_norm_beta and
 * receptance_key_bonus ([H,N]) hold C elements each.
 */
int rwkv7_fused_gated_readout(const rwkv7_tensor *wkv7_output, const rwkv7_tensor *receptance,
                              const rwkv7_tensor *replacement_key, const rwkv7_tensor *value,
                              const rwkv7_tensor *gate, const rwkv7_tensor *group_norm_gamma,
                              const rwkv7_tensor *group_norm_beta,
                              const rwkv7_tensor *receptance_key_bonus, double epsilon,
                              int64_t num_heads, rwkv7_tensor *output, rwkv7_stream stream);

/* --------------------------------------------------------- channel mixer -- */
/*
 * Replaces ChannelMixerBackend::fused_channel_mixer (kernels/train/channel_mixer/mod.rs,
 * host forward.rs:52-88, definition channel_mixer_reference mod.rs:96-128):
 *   shifted[b,t,:] = x[b,t-1,:] (zero at t == 0); key_input = x + (shifted - x) * key_scale;
 *   output = relu(key_input . key_weight^T)^2 . value_weight^T.
 * embedded_context and output [B,T,C], key_scale [C], key_weight [F,C], value_weight [C,F];
 * checks in the order of ChannelMixerForwardInputs::check (channel_mixer/io.rs:40-62).
 * Both projections run on the tensor cores in BF16 with fp32 accumulation; the
 * activation is part of the first projection's epilogue.  BF16 tensors only (F32 returns
 * RWKV7_ERR_UNSUPPORTED); C and F must be multiples of 8.  The workspace holds key_input
 * and the activated hidden tensor: rwkv7_channel_mixer_workspace_bytes(B, T, C, F).
 */
size_t rwkv7_channel_mixer_workspace_bytes(int64_t B, int64_t T, int64_t C, int64_t F);

int rwkv7_fused_channel_mixer(const rwkv7_tensor *embedded_context, const rwkv7_tensor *key_scale,
                              const rwkv7_tensor *key_weight, const rwkv7_tensor *value_weight,
                              rwkv7_tensor *output, void *workspace, size_t workspace_bytes,
                              rwkv7_stream stream);

/* ------------------------------------------------------------ lm_head_ce -- */
/*
 * Fused LM-head cross entropy.  The reference only reserves the module
 * (kernels/train/lm_head_l2wrap_ce/mod.rs is empty; config switch
 * rwkv-config/src/raw/train.rs:59-60), so this entry point defines the
 * operator: z = x W^T with x [R,C] and W [V_shard,C] (BF16, fp32 accumulate);
 * per row the partial triple over this vocabulary shard
 *   row_max = max_v z_v, row_sumexp = sum_v exp(z_v - row_max),
 *   row_target = z[target - vocab_offset] if the target falls in the shard else 0.
 * Logits are never written to memory.  targets [R] are I32 or I64; a negative
 * target marks an ignored row.  L2Wrap is a backward-only regulariser and is the
 * identity here.  partials is [R,3] F32 (max, sumexp, target logit).
 */
size_t rwkv7_lm_head_ce_workspace_bytes(int64_t R, int64_t C, int64_t V_shard);

int rwkv7_fused_lm_head_ce_partial(const rwkv7_tensor *x, const rwkv7_tensor *weight_shard,
                                   const rwkv7_tensor *targets, int64_t vocab_offset,
                                   rwkv7_tensor *partials, void *workspace,
                                   size_t workspace_bytes, rwkv7_stream stream);

/* Combines `num_shards` partial tensors laid out [num_shards,R,3] into per-row
 * lse [R] and loss [R] (F32): M = max_g m_g; lse = M + log sum_g s_g exp(m_g-M);
 * loss = lse - sum_g target_g (0 for ignored rows). */
int rwkv7_lm_head_ce_finalize(const rwkv7_tensor *partials_all, const rwkv7_tensor *targets,
                              rwkv7_tensor *lse, rwkv7_tensor *loss, rwkv7_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* RWKV7_B200_H_ */
