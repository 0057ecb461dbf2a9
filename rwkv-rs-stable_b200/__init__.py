"""Host-side mirror of the rwkv-rs WKV7 operator interface over the C ABI.

The directory name carries a hyphen, so the package is loaded under the module
name ``rwkv_rs_stable_b200`` (``__graft_entry__.load_package()`` does that with
:mod:`importlib`).

Function and argument names follow the reference's public wrappers
(``crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:105-150``,
``.../mix6/mod.rs:159-177``, ``crates/rwkv-nn/src/kernels/template/addcmul/mod.rs:100-114``,
``.../token_shift_diff/mod.rs:82-168``).  Like the reference's wrappers, which
``check().unwrap()`` and panic, every function raises :class:`KernelInputsError`
with the reference's message text when the input contract is violated.

All arithmetic happens in ``librwkv7_b200.so`` (hand-written sm_100a CUDA, see
``csrc/``); torch only owns device memory and streams here.  There is no CPU
fallback: importing works without a GPU, calling an operator does not.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# RWKV7_B200_LIB selects another build of the same library (e.g. an instrumented one).
LIB_PATH = os.environ.get("RWKV7_B200_LIB") or os.path.join(_HERE, "librwkv7_b200.so")

MAX_DIMS = 5
F32, BF16, F16, I32, I64, U32 = 0, 1, 2, 3, 4, 5
WKV7_AUTO, WKV7_SEQUENTIAL, WKV7_CHUNKED, WKV7_SPLIT = 0, 1, 2, 3

_DTYPES = {
    torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16,
    torch.int32: I32, torch.int64: I64,
}

STATUS_NAMES = {
    0: "Ok", 1: "AxisMismatch", 2: "ShapeMismatch", 3: "DTypeMismatch", 4: "DeviceMismatch",
    5: "EmptyAxis", 6: "NotContiguous", 7: "BadChunk", 8: "Unsupported", 9: "NullPointer",
    10: "WorkspaceTooSmall", 11: "CudaError", 12: "Timeout", 13: "BadIndex", 14: "BadArgument",
}


class KernelInputsError(RuntimeError):
    """Raised where the reference panics (``kernels/check.rs:34-73``)."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.kind = STATUS_NAMES.get(status, "Unknown")


class Tensor(ctypes.Structure):
    """``rwkv7_tensor`` of ``include/rwkv7_b200.h``."""

    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("device", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("shape", ctypes.c_int64 * MAX_DIMS),
        ("stride", ctypes.c_int64 * MAX_DIMS),
    ]


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """Loads the C-ABI library; fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}`. "
                "There is no fallback path.")
        L = ctypes.CDLL(LIB_PATH)
        L.rwkv7_status_string.restype = ctypes.c_char_p
        L.rwkv7_last_error_message.restype = ctypes.c_char_p
        L.rwkv7_wkv7_workspace_bytes.restype = ctypes.c_size_t
        L.rwkv7_wkv7_workspace_bytes.argtypes = [ctypes.c_int64] * 4 + [ctypes.c_int32]
        L.rwkv7_kernel_launch_count.restype = ctypes.c_int64
        L.rwkv7_lm_head_ce_workspace_bytes.restype = ctypes.c_size_t
        L.rwkv7_lm_head_ce_workspace_bytes.argtypes = [ctypes.c_int64] * 3
        L.rwkv7_channel_mixer_workspace_bytes.restype = ctypes.c_size_t
        L.rwkv7_channel_mixer_workspace_bytes.argtypes = [ctypes.c_int64] * 4
        L.rwkv7_wkv7_backward_workspace_bytes.restype = ctypes.c_size_t
        L.rwkv7_wkv7_backward_workspace_bytes.argtypes = [ctypes.c_int64] * 4
        _lib = L
    return _lib


def describe(t: Optional[torch.Tensor], device: Optional[int] = None) -> Optional[Tensor]:
    """Builds the borrowed descriptor of a torch tensor (no copy)."""
    if t is None:
        return None
    d = Tensor()
    d.data = t.data_ptr() if t.numel() else None
    if t.dtype not in _DTYPES:
        raise TypeError(f"unsupported torch dtype {t.dtype}")
    d.dtype = _DTYPES[t.dtype]
    d.device = t.device.index if t.device.type == "cuda" else (-1 if device is None else device)
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    return d


def _ref(d: Optional[Tensor]):
    return None if d is None else ctypes.byref(d)


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    if t.device.type != "cuda":
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _check(status: int) -> None:
    if status != 0:
        raise KernelInputsError(status, lib().rwkv7_last_error_message().decode())


def set_wkv7_path(path: int) -> None:
    _check(lib().rwkv7_set_wkv7_path(ctypes.c_int(path)))


def set_wkv7_cluster(cluster_size: int) -> None:
    """0 = automatic (by the number of chains), else the cluster size (1, 2, 4) of the chunked kernel."""
    _check(lib().rwkv7_set_wkv7_cluster(ctypes.c_int(cluster_size)))


def set_wkv7_overlap(on: bool) -> None:
    """``rwkv7_set_wkv7_overlap``: scans of the two-kernel prefill beside the next segment's operator kernel
    on the library's second stream (default) or everything on the caller's stream."""
    _check(lib().rwkv7_set_wkv7_overlap(int(on)))


def get_wkv7_path() -> int:
    return int(lib().rwkv7_get_wkv7_path())


def kernel_launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib().rwkv7_kernel_launch_count())


def read_device_status(device: int = 0) -> int:
    """Reads and clears the device status word; returns the status code."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    return int(lib().rwkv7_read_device_status(ctypes.c_int(device), stream))


def selftest_bounded_wait(device: int = 0, max_polls: int = 1000) -> None:
    """Runs the library's bounded-wait error path once (``rwkv7_selftest_bounded_wait``); the
    time-out is then reported by :func:`read_device_status`."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    _check(lib().rwkv7_selftest_bounded_wait(ctypes.c_int(device), ctypes.c_int64(max_polls), stream))


# ---------------------------------------------------------------------- WKV7 --


@dataclass
class Wkv7PretrainForwardInputs:
    """``wkv7/io.rs:20-66``: six ``[batch, context_len, num_heads, head_size]`` tensors."""

    receptance: torch.Tensor
    weight_decay: torch.Tensor
    replacement_key: torch.Tensor
    value: torch.Tensor
    removal_key_normalized: torch.Tensor
    replacement: torch.Tensor
    chunk_len: int = 16

    def six(self):
        return (self.receptance, self.weight_decay, self.replacement_key, self.value,
                self.removal_key_normalized, self.replacement)

    def check(self, reference_contract: bool = True) -> None:
        """The reference's assertions that precede its shape checks
        (``wkv7/io.rs:187,198-201``): ``chunk_len == 16`` and
        ``context_len % chunk_len == 0``.  The C ABI itself accepts any ``T >= 1``."""
        if not reference_contract:
            return
        if self.chunk_len != 16:
            raise KernelInputsError(7, "wkv7 currently supports chunk_len=16")
        if self.receptance.dim() == 4 and self.receptance.shape[1] % self.chunk_len != 0:
            raise KernelInputsError(7, "context_len must be a multiple of chunk_len")


@dataclass
class Wkv7StatepassForwardOutput:
    """``wkv7/io.rs:157-164``."""

    output: torch.Tensor
    next_state: torch.Tensor


def _wkv7_workspace(r: torch.Tensor) -> tuple[Optional[torch.Tensor], int]:
    if r.dim() != 4:
        return None, 0
    B, T, H, N = r.shape
    n = int(lib().rwkv7_wkv7_workspace_bytes(B, T, H, N, _DTYPES.get(r.dtype, 0)))
    if n == 0:
        return None, 0
    return torch.empty(n, dtype=torch.uint8, device=r.device), n


def _wkv7_call(inputs: Wkv7PretrainForwardInputs, initial_state, want_state: bool,
               next_state: Optional[torch.Tensor] = None, output: Optional[torch.Tensor] = None,
               workspace: Optional[torch.Tensor] = None):
    r = inputs.receptance
    six = [describe(t) for t in inputs.six()]
    y = torch.empty_like(r) if output is None else output
    yd = describe(y)
    if workspace is None:
        workspace, ws_bytes = _wkv7_workspace(r)
    else:
        ws_bytes = workspace.numel() * workspace.element_size()
    ws_ptr = ctypes.c_void_p(workspace.data_ptr() if workspace is not None else 0)
    stream = _stream(r)
    L = lib()
    cl = ctypes.c_int64(inputs.chunk_len)
    if initial_state is None:
        st = L.rwkv7_fused_wkv7_pretrain(*[_ref(d) for d in six], cl, _ref(yd), ws_ptr,
                                         ctypes.c_size_t(ws_bytes), stream)
        _check(st)
        return y, None
    s0d = describe(initial_state)
    if not want_state:
        st = L.rwkv7_fused_wkv7_statetune(_ref(s0d), *[_ref(d) for d in six], cl, _ref(yd), ws_ptr,
                                          ctypes.c_size_t(ws_bytes), stream)
        _check(st)
        return y, None
    s_out = torch.empty_like(initial_state) if next_state is None else next_state
    sod = describe(s_out)
    st = L.rwkv7_fused_wkv7_statepass(_ref(s0d), *[_ref(d) for d in six], cl, _ref(yd), _ref(sod),
                                      ws_ptr, ctypes.c_size_t(ws_bytes), stream)
    _check(st)
    return y, s_out


def wkv7_pretrain_custom(inputs: Wkv7PretrainForwardInputs, *, reference_contract: bool = True,
                         output=None, workspace=None) -> torch.Tensor:
    """``wkv7_pretrain_custom`` (``wkv7/mod.rs:105-110``): zero initial state -> y."""
    inputs.check(reference_contract)
    return _wkv7_call(inputs, None, False, output=output, workspace=workspace)[0]


def wkv7_statetune_custom(initial_state: torch.Tensor, sequence: Wkv7PretrainForwardInputs, *,
                          reference_contract: bool = True, output=None, workspace=None) -> torch.Tensor:
    """``wkv7_statetune_custom`` (``wkv7/mod.rs:113-120``): given state -> y."""
    sequence.check(reference_contract)
    return _wkv7_call(sequence, initial_state, False, output=output, workspace=workspace)[0]


def wkv7_statepass_custom(initial_state: torch.Tensor, sequence: Wkv7PretrainForwardInputs, *,
                          reference_contract: bool = True, next_state=None, output=None,
                          workspace=None) -> Wkv7StatepassForwardOutput:
    """``wkv7_statepass_custom`` (``wkv7/mod.rs:123-133``): given state -> (y, S_T).
    With ``reference_contract=False`` any ``T >= 1`` is accepted (``T == 1`` is decode);
    ``next_state`` may be the same tensor as ``initial_state`` (in-place update)."""
    sequence.check(reference_contract)
    y, s = _wkv7_call(sequence, initial_state, True, next_state=next_state, output=output,
                      workspace=workspace)
    return Wkv7StatepassForwardOutput(output=y, next_state=s)


class Wkv7StatepassCall:
    """A statepass call with its descriptors built once, for callers that repeat the
    same call on fixed buffers (decode loops, benchmarks): ``call()`` is one FFI
    call with no per-call allocation.  The tensors must stay alive and unmoved."""

    def __init__(self, initial_state, sequence: Wkv7PretrainForwardInputs, output, next_state,
                 workspace=None):
        self._keep = (initial_state, sequence, output, next_state, workspace)
        self._desc = [describe(initial_state)] + [describe(t) for t in sequence.six()]
        self._y, self._s = describe(output), describe(next_state)
        self._args = [_ref(d) for d in self._desc] + [ctypes.c_int64(sequence.chunk_len), _ref(self._y),
                                                      _ref(self._s)]
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        self._args += [ctypes.c_void_p(workspace.data_ptr() if workspace is not None else 0),
                       ctypes.c_size_t(ws_bytes)]
        self._device = sequence.receptance.device
        self._fn = lib().rwkv7_fused_wkv7_statepass

    def __call__(self):
        st = self._fn(*self._args, ctypes.c_void_p(torch.cuda.current_stream(self._device).cuda_stream))
        if st:
            _check(st)


@dataclass
class Wkv7SavedForward:
    """Outputs of the training forward: what the reference's forward kernels return under
    autodiff (``wkv7/forward.rs:368-375``)."""

    output: Optional[torch.Tensor]
    next_state: Optional[torch.Tensor]
    snapshots: torch.Tensor            # [B, H, T/chunk_len, N, N] fp32
    state_replacement: torch.Tensor    # [B, T, H, N]


def wkv7_forward_saved(inputs: Wkv7PretrainForwardInputs, initial_state: Optional[torch.Tensor] = None, *,
                       want_state: bool = False) -> Wkv7SavedForward:
    """``rwkv7_fused_wkv7_forward_saved``: the recurrence plus the tensors the backward pass needs."""
    inputs.check(True)
    r = inputs.receptance
    B, T, H, N = r.shape
    y = torch.empty_like(r)
    sa = torch.empty_like(r)
    snaps = torch.empty((B, H, T // inputs.chunk_len, N, N), dtype=torch.float32, device=r.device)
    s_out = torch.empty((B, H, N, N), dtype=torch.float32, device=r.device) if want_state else None
    descs = [describe(initial_state)] + [describe(t) for t in inputs.six()]
    outs = [describe(y), describe(s_out), describe(snaps), describe(sa)]
    workspace, ws_bytes = _wkv7_workspace(r)
    ws_ptr = ctypes.c_void_p(workspace.data_ptr() if workspace is not None else 0)
    _check(lib().rwkv7_fused_wkv7_forward_saved(*[_ref(d) for d in descs], ctypes.c_int64(inputs.chunk_len),
                                                *[_ref(d) for d in outs], ws_ptr, ctypes.c_size_t(ws_bytes), _stream(r)))
    return Wkv7SavedForward(output=y, next_state=s_out, snapshots=snaps, state_replacement=sa)


def wkv7_backward_workspace_bytes(B: int, T: int, H: int, N: int) -> int:
    """``rwkv7_wkv7_backward_workspace_bytes``: workspace of the time-parallel backward (0 when the shape
    takes the token-by-token kernel)."""
    return int(lib().rwkv7_wkv7_backward_workspace_bytes(ctypes.c_int64(B), ctypes.c_int64(T), ctypes.c_int64(H),
                                                         ctypes.c_int64(N)))


def wkv7_backward(inputs: Wkv7PretrainForwardInputs, saved: Wkv7SavedForward, output_grad: torch.Tensor,
                  next_state_grad: Optional[torch.Tensor] = None, *, initial_state: Optional[torch.Tensor] = None,
                  want_state_grad: bool = True, parallel: bool = True, workspace: Optional[torch.Tensor] = None):
    """``rwkv7_fused_wkv7_backward_parallel`` (``parallel=True``: the gradient recurrence as a tensor-core
    forward pass over the reversed sequence, the rest per 16-token chunk; shapes it does not cover fall
    through to the token-by-token kernel) or ``rwkv7_fused_wkv7_backward``.  Returns ``(six sequence
    gradients in input order, initial_state_grad or None)`` (``Wkv7BackwardPrimitiveOutputs``,
    ``wkv7/backward.rs:567-575``).  ``workspace``: a uint8 tensor of ``wkv7_backward_workspace_bytes``;
    allocated here when omitted."""
    r = inputs.receptance
    B, T, H, N = r.shape
    grads = [torch.empty_like(r) for _ in range(6)]
    ds0 = torch.empty((B, H, N, N), dtype=torch.float32, device=r.device) if want_state_grad else None
    gd = [describe(t) for t in grads]
    arr = (ctypes.POINTER(Tensor) * 6)(*[ctypes.pointer(d) for d in gd])
    descs = [describe(initial_state)] + [describe(t) for t in inputs.six()] + [describe(saved.snapshots),
                                                                            describe(saved.state_replacement)]
    dyd, dsd, ds0d = describe(output_grad.contiguous()), describe(next_state_grad), describe(ds0)
    if parallel and r.dtype == torch.bfloat16:
        need = wkv7_backward_workspace_bytes(B, T, H, N)
        if workspace is None:
            workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=r.device)
        _check(lib().rwkv7_fused_wkv7_backward_parallel(
            *[_ref(d) for d in descs], ctypes.c_int64(inputs.chunk_len), _ref(dyd), _ref(dsd), arr, _ref(ds0d),
            ctypes.c_void_p(workspace.data_ptr()), ctypes.c_size_t(workspace.numel()), _stream(r)))
        return grads, ds0
    _check(lib().rwkv7_fused_wkv7_backward(*[_ref(d) for d in descs], ctypes.c_int64(inputs.chunk_len), _ref(dyd),
                                           _ref(dsd), arr, _ref(ds0d), _stream(r)))
    return grads, ds0


class _Wkv7Function(torch.autograd.Function):
    """The autodiff node of the reference (``Wkv7StatepassBackward``, ``wkv7/backward.rs:381-533``):
    forward saves snapshots and state_replacement, backward runs the reverse kernel."""

    @staticmethod
    def forward(ctx, r, w, k, v, a, b, s0, chunk_len):
        inputs = Wkv7PretrainForwardInputs(r, w, k, v, a, b, chunk_len=chunk_len)
        saved = wkv7_forward_saved(inputs, s0, want_state=True)
        # Only what the backward pass reads is kept, and through save_for_backward: the node then
        # holds no reference to its own outputs (no cycle) and autograd's version counters catch an
        # in-place change of an input between forward and backward.
        keep = [r, w, k, v, a, b, saved.snapshots, saved.state_replacement]
        if s0 is not None:
            keep.append(s0)
        ctx.save_for_backward(*keep)
        ctx.has_state, ctx.chunk_len = s0 is not None, chunk_len
        return saved.output, saved.next_state

    @staticmethod
    def backward(ctx, dy, ds):
        t = ctx.saved_tensors
        inputs = Wkv7PretrainForwardInputs(*t[:6], chunk_len=ctx.chunk_len)
        saved = Wkv7SavedForward(output=None, next_state=None, snapshots=t[6], state_replacement=t[7])
        s0 = t[8] if ctx.has_state else None
        grads, ds0 = wkv7_backward(inputs, saved, dy, None if ds is None else ds.contiguous(),
                                   initial_state=s0, want_state_grad=ctx.has_state)
        return (*grads, ds0, None)


def wkv7_statepass_autograd(initial_state: Optional[torch.Tensor], sequence: Wkv7PretrainForwardInputs):
    """Differentiable statepass: ``(output, next_state)`` with gradients to the six sequence tensors and
    the initial state, like ``wkv7_statepass_custom`` on the reference's Autodiff backend."""
    return _Wkv7Function.apply(*[t.contiguous() for t in sequence.six()], initial_state, sequence.chunk_len)


class Wkv7HostStatepass:
    """``rwkv7_wkv7_statepass_host``: statepass for callers whose six sequence tensors, y and
    S_T live in pinned host memory (an inference server that receives activations from
    another process, a benchmark that counts the copies).  The library cuts the batch into
    equal slices; slice ``i`` uses stream ``i % n_streams`` for its host-to-device copies,
    its kernels and its device-to-host copies, so the copy of one slice overlaps the kernels
    and the copy-back of the slices before it.  (b,h) chains are independent, so slicing the
    batch changes no arithmetic: results are bitwise those of one call on the whole batch
    whenever both run the same variant of the kernel.

    ``host_state_in`` may be None (S0 = 0).  The device staging buffer and the worker streams
    are created once, here; ``__call__`` allocates nothing.  The call is asynchronous: work is
    ordered after the caller's current stream, and (unless ``join=False``) the current stream
    waits for it, so ``torch.cuda.current_stream().synchronize()`` marks completion."""

    def __init__(self, host_six: Sequence[torch.Tensor], host_state_in: Optional[torch.Tensor],
                 host_output: torch.Tensor, host_state_out: torch.Tensor, *, device,
                 slices: Optional[int] = None, n_streams: int = 3, chunk_len: int = 16):
        r = host_six[0]
        if r.dim() != 4:
            raise KernelInputsError(1, "AxisMismatch: expected [B, T, H, N] host tensors")
        B, T, H, N = r.shape
        for t in list(host_six) + [host_output, host_state_out] + ([host_state_in] if host_state_in is not None else []):
            if t.is_cuda or not t.is_pinned() or not t.is_contiguous():
                raise KernelInputsError(6, "NotContiguous: host tensors must be contiguous pinned CPU tensors")
        if slices is None:
            slices = next(s for s in (8, 4, 2, 1) if B % s == 0)
        if slices < 1 or B % slices:
            raise KernelInputsError(2, f"ShapeMismatch: {slices} slices do not divide B={B}")
        self._device = torch.device(device)
        self._index = self._device.index if self._device.index is not None else torch.cuda.current_device()
        self._slices = slices
        n_streams = max(1, min(n_streams, slices))
        self._streams = [torch.cuda.Stream(self._device) for _ in range(n_streams)]
        self._stream_array = (ctypes.c_void_p * n_streams)(*[st.cuda_stream for st in self._streams])
        self._host = (list(host_six), host_state_in, host_output, host_state_out)
        L = lib()
        L.rwkv7_wkv7_host_staging_bytes.restype = ctypes.c_size_t
        L.rwkv7_wkv7_host_staging_bytes.argtypes = [ctypes.c_int64] * 4 + [ctypes.c_int32] * 3
        nbytes = int(L.rwkv7_wkv7_host_staging_bytes(B, T, H, N, _DTYPES.get(r.dtype, 0), slices, n_streams))
        self._staging = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self._device)
        self._desc = [describe(t, device=-1) for t in host_six]
        self._six = (ctypes.POINTER(Tensor) * 6)(*[ctypes.pointer(d) for d in self._desc])
        self._s_in = describe(host_state_in, device=-1)
        self._y, self._s_out = describe(host_output, device=-1), describe(host_state_out, device=-1)
        self._chunk_len = chunk_len

    def __call__(self, join: bool = True) -> None:
        """Enqueues one pass.  With ``join=False`` the caller's stream is not made to wait for the
        pass: a caller that issues passes back to back (a server draining a queue) lets the
        copy-in of the next pass overlap the tail of this one, and calls :meth:`join` (or a last
        pass with ``join=True``) before it reads the host outputs.  Passes always execute in
        issue order slice by slice, so the host buffers are never written out of order."""
        cur = torch.cuda.current_stream(self._device)
        _check(lib().rwkv7_wkv7_statepass_host(
            _ref(self._s_in), self._six, ctypes.c_int64(self._chunk_len), _ref(self._y), _ref(self._s_out),
            ctypes.c_int32(self._index), ctypes.c_int32(self._slices), ctypes.c_void_p(self._staging.data_ptr()),
            ctypes.c_size_t(self._staging.numel()), self._stream_array, ctypes.c_int32(len(self._streams)),
            ctypes.c_void_p(cur.cuda_stream), ctypes.c_int32(0 if join else 1)))

    def join(self) -> None:
        """Makes the caller's current stream wait for every pass issued so far."""
        cur = torch.cuda.current_stream(self._device)
        _check(lib().rwkv7_wkv7_host_join(ctypes.c_int32(self._index), self._stream_array,
                                          ctypes.c_int32(len(self._streams)), ctypes.c_void_p(cur.cuda_stream)))

    def bytes_per_call(self) -> tuple[int, int]:
        """(host-to-device, device-to-host) bytes one call moves."""
        host_six, host_s_in, host_y, host_s_out = self._host
        h2d = sum(t.numel() * t.element_size() for t in host_six)
        if host_s_in is not None:
            h2d += host_s_in.numel() * host_s_in.element_size()
        d2h = host_y.numel() * host_y.element_size() + host_s_out.numel() * host_s_out.element_size()
        return h2d, d2h


def wkv7_statepass_noalloc(initial_state: torch.Tensor, sequence: Wkv7PretrainForwardInputs,
                           output: torch.Tensor, next_state: torch.Tensor) -> Wkv7StatepassForwardOutput:
    """``rwkv7_fused_wkv7_statepass_noalloc``: the statepass for callers that must
    not allocate device memory while calling (a server whose memory pool already
    owns the GPU, a thread on which a device allocation would stall the device).
    The caller passes every buffer, ``output`` and ``next_state`` included, and no
    workspace: the library's own fixed 256 KiB flag array is used instead, which
    limits ``B*H`` to 65536 chains.  Calls on one device must not overlap on the
    GPU, since they share that array.  Nothing is allocated here either: the
    descriptors are plain ctypes structures on the host."""
    desc = [describe(initial_state)] + [describe(t) for t in sequence.six()]
    yd, sd = describe(output), describe(next_state)
    st = lib().rwkv7_fused_wkv7_statepass_noalloc(*[_ref(d) for d in desc], ctypes.c_int64(sequence.chunk_len),
                                                  _ref(yd), _ref(sd), _stream(sequence.receptance))
    _check(st)
    return Wkv7StatepassForwardOutput(output=output, next_state=next_state)


wkv7_pretrain = wkv7_pretrain_custom
wkv7_statetune = wkv7_statetune_custom
wkv7_statepass = wkv7_statepass_custom

# ---------------------------------------------------------------------- mix6 --

MIX6_BRANCHES = ("receptance_input", "weight_decay_input", "key_input", "value_input",
                 "learning_rate_input", "gate_input")


def _ptr_array(descs: Sequence[Optional[Tensor]]):
    arr = (ctypes.POINTER(Tensor) * len(descs))()
    for i, d in enumerate(descs):
        arr[i] = ctypes.pointer(d) if d is not None else None
    return arr


def mix6_custom(embedded_context: torch.Tensor, receptance_scale, weight_decay_scale, key_scale,
                value_scale, learning_rate_scale, gate_scale, *, stacked: bool = False):
    """``mix6_custom`` (``mix6/mod.rs:76-108``).  Returns a dict of the six
    ``[B,T,C]`` outputs, or one ``[6,B,T,C]`` tensor when ``stacked``."""
    x = embedded_context
    scales = [receptance_scale, weight_decay_scale, key_scale, value_scale, learning_rate_scale, gate_scale]
    xd = describe(x)
    sd = [describe(s) for s in scales]
    L = lib()
    if stacked:
        out = torch.empty((6,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        od = describe(out)
        _check(L.rwkv7_fused_mix6_stacked(_ref(xd), _ptr_array(sd), _ref(od), _stream(x)))
        return out
    outs = [torch.empty_like(x) for _ in range(6)]
    od = [describe(o) for o in outs]
    _check(L.rwkv7_fused_mix6(_ref(xd), _ptr_array(sd), _ptr_array(od), _stream(x)))
    return dict(zip(MIX6_BRANCHES, outs))


mix6 = mix6_custom

# ------------------------------------------------------------------- addcmul --


def addcmul_custom(base: torch.Tensor, diff: torch.Tensor, scale: torch.Tensor, *,
                   inplace: bool = False) -> torch.Tensor:
    """``addcmul_custom`` (``addcmul/mod.rs:100-105``): ``base + diff * scale``.
    ``inplace`` writes over ``base`` like the reference does for a uniquely owned buffer."""
    out = base if inplace else torch.empty_like(base)
    bd, dd, sd, od = describe(base), describe(diff), describe(scale), describe(out)
    _check(lib().rwkv7_fused_addcmul(_ref(bd), _ref(dd), _ref(sd), _ref(od), _stream(base)))
    return out


def addcmul5_custom(base: torch.Tensor, diff: torch.Tensor, receptance_scale, weight_decay_scale,
                    key_scale, value_scale, learning_rate_scale):
    """``addcmul5_custom`` (``addcmul/mod.rs:138-157``): five outputs sharing base and diff."""
    scales = [receptance_scale, weight_decay_scale, key_scale, value_scale, learning_rate_scale]
    outs = [torch.empty_like(base) for _ in range(5)]
    bd, dd = describe(base), describe(diff)
    sd = [describe(s) for s in scales]
    od = [describe(o) for o in outs]
    _check(lib().rwkv7_fused_addcmul5(_ref(bd), _ref(dd), _ptr_array(sd), _ptr_array(od), _stream(base)))
    return dict(zip(MIX6_BRANCHES[:5], outs))


addcmul = addcmul_custom
addcmul5 = addcmul5_custom

# ---------------------------------------------------------- token_shift_diff --


@dataclass
class TokenShiftDiffForwardOutput:
    """``token_shift_diff/io.rs:77-83``."""

    token_shifted_diff: torch.Tensor
    next_token_shift: torch.Tensor


def token_shift_diff_custom(embedded_context: torch.Tensor, embedded_token_shift: torch.Tensor,
                            batch_ids: torch.Tensor, *, inplace_state: bool = False
                            ) -> TokenShiftDiffForwardOutput:
    """``token_shift_diff_custom`` (``token_shift_diff/mod.rs:82-111``).  The state
    buffer is updated in place by the kernel; unless ``inplace_state`` the caller's
    tensor is cloned first so that the call is functional like the reference's."""
    state = embedded_token_shift if inplace_state else embedded_token_shift.clone()
    diff = torch.empty_like(embedded_context)
    xd, sd, idd, dd = describe(embedded_context), describe(state), describe(batch_ids), describe(diff)
    _check(lib().rwkv7_fused_token_shift_diff(_ref(xd), _ref(sd), _ref(idd), _ref(dd),
                                              _stream(embedded_context)))
    return TokenShiftDiffForwardOutput(token_shifted_diff=diff, next_token_shift=state)


token_shift_diff = token_shift_diff_custom

# ---------------------------------------------------------------- lm_head_ce --


@dataclass
class WeightPrepareEpilogueOutput:
    """The WKV7-ready fields of ``WeightPrepareOutput``
    (``modules/time_mixer/weight_prepare.rs:289-297``) that the epilogue computes."""

    weight_decay: torch.Tensor
    replacement_key: torch.Tensor
    value: Optional[torch.Tensor]
    removal_key_normalized: torch.Tensor
    replacement: torch.Tensor


def weight_prepare_epilogue(key_precursor: torch.Tensor, learning_rate_lora: torch.Tensor,
                            weight_decay_lora: torch.Tensor, key_removal: torch.Tensor,
                            key_replacement: torch.Tensor, num_heads: int, *,
                            value_precursor: Optional[torch.Tensor] = None,
                            value_from_first_cell: Optional[torch.Tensor] = None,
                            value_residual_lora: Optional[torch.Tensor] = None) -> WeightPrepareEpilogueOutput:
    """The tail of ``WeightPrepare::forward`` (``weight_prepare.rs:252-287``) in one kernel.
    ``learning_rate_lora``, ``weight_decay_lora`` and ``value_residual_lora`` are the LoRA
    modules' outputs, before the sigmoid / softplus that ``forward`` applies to them; the three value tensors are given for every
    cell but the first (there ``value`` is ``value_precursor`` and is returned as is)."""
    outs = [torch.empty_like(key_precursor) for _ in range(4)]
    with_value = value_precursor is not None
    value = torch.empty_like(key_precursor) if with_value else None
    descs = [describe(t) for t in (key_precursor, learning_rate_lora, weight_decay_lora, key_removal,
                                   key_replacement, value_precursor, value_from_first_cell,
                                   value_residual_lora)]
    od = [describe(t) for t in outs] + [describe(value)]
    _check(lib().rwkv7_fused_weight_prepare(*[_ref(d) for d in descs], ctypes.c_int64(num_heads),
                                            *[_ref(d) for d in od], _stream(key_precursor)))
    return WeightPrepareEpilogueOutput(weight_decay=outs[0], replacement_key=outs[1],
                                       value=value if with_value else None,
                                       removal_key_normalized=outs[2], replacement=outs[3])


def gated_readout_epilogue(wkv7_output: torch.Tensor, receptance: torch.Tensor, replacement_key: torch.Tensor,
                           value: torch.Tensor, gate: torch.Tensor, group_norm_gamma: torch.Tensor,
                           group_norm_beta: torch.Tensor, receptance_key_bonus: torch.Tensor,
                           num_heads: int, epsilon: float = 64e-5) -> torch.Tensor:
    """``GatedReadout::forward`` between the gate LoRA and the output projection
    (``gated_readout.rs:123-141``): per-head GroupNorm of the WKV7 output, the
    receptance-key bonus and the gate, in one kernel.  Returns ``[B,T,C]``-shaped
    like ``wkv7_output``; ``gate`` is the gate LoRA's output as it is (``gated_readout.rs:121``)."""
    out = torch.empty_like(wkv7_output)
    descs = [describe(t) for t in (wkv7_output, receptance, replacement_key, value, gate, group_norm_gamma,
                                   group_norm_beta, receptance_key_bonus)]
    od = describe(out)
    _check(lib().rwkv7_fused_gated_readout(*[_ref(d) for d in descs], ctypes.c_double(epsilon),
                                           ctypes.c_int64(num_heads), _ref(od), _stream(wkv7_output)))
    return out


def channel_mixer_custom(embedded_context: torch.Tensor, key_scale: torch.Tensor, key_weight: torch.Tensor,
                         value_weight: torch.Tensor, *, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``channel_mixer`` (``kernels/train/channel_mixer/mod.rs:130-144``): token-shift mix, key
    projection with relu^2 in its epilogue, value projection; bf16 tensors."""
    out = torch.empty_like(embedded_context)
    ws_ptr, ws_bytes = ctypes.c_void_p(0), 0
    if embedded_context.dim() == 3 and key_weight.dim() == 2:
        B, T, C = embedded_context.shape
        ws_bytes = int(lib().rwkv7_channel_mixer_workspace_bytes(B, T, C, key_weight.shape[0]))
        if workspace is None and ws_bytes:
            workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=embedded_context.device)
        if workspace is not None:
            ws_ptr, ws_bytes = ctypes.c_void_p(workspace.data_ptr()), workspace.numel() * workspace.element_size()
    descs = [describe(t) for t in (embedded_context, key_scale, key_weight, value_weight)]
    od = describe(out)
    _check(lib().rwkv7_fused_channel_mixer(*[_ref(d) for d in descs], _ref(od), ws_ptr, ctypes.c_size_t(ws_bytes),
                                           _stream(embedded_context)))
    return out


channel_mixer = channel_mixer_custom


def lm_head_ce_partial(x: torch.Tensor, weight_shard: torch.Tensor, targets: torch.Tensor,
                       vocab_offset: int = 0) -> torch.Tensor:
    """Per-row ``(max, sumexp, target logit)`` of ``x @ weight_shard.T`` over one
    vocabulary shard, ``[R,3]`` fp32; logits are never materialised."""
    R = x.shape[0]
    partials = torch.empty((R, 3), dtype=torch.float32, device=x.device)
    n = int(lib().rwkv7_lm_head_ce_workspace_bytes(R, x.shape[1], weight_shard.shape[0]))
    ws = torch.empty(max(n, 1), dtype=torch.uint8, device=x.device)
    xd, wd, td, pd = describe(x), describe(weight_shard), describe(targets), describe(partials)
    _check(lib().rwkv7_fused_lm_head_ce_partial(_ref(xd), _ref(wd), _ref(td), ctypes.c_int64(vocab_offset),
                                                _ref(pd), ctypes.c_void_p(ws.data_ptr()),
                                                ctypes.c_size_t(n), _stream(x)))
    return partials


def lm_head_ce_finalize(partials_all: torch.Tensor, targets: torch.Tensor):
    """Combines ``[num_shards,R,3]`` partials into per-row ``(lse, loss)``."""
    R = partials_all.shape[1]
    lse = torch.empty(R, dtype=torch.float32, device=partials_all.device)
    loss = torch.empty(R, dtype=torch.float32, device=partials_all.device)
    pd, td, ld, sd = describe(partials_all), describe(targets), describe(lse), describe(loss)
    _check(lib().rwkv7_lm_head_ce_finalize(_ref(pd), _ref(td), _ref(ld), _ref(sd), _stream(partials_all)))
    return lse, loss


def lm_head_ce(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor):
    """Single-GPU fused LM-head cross entropy: per-row ``(lse, loss)``."""
    p = lm_head_ce_partial(x, weight, targets, 0)
    return lm_head_ce_finalize(p.unsqueeze(0), targets)
