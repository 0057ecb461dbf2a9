"""ctypes loader for the CPU oracle (``oracle/rwkv7_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The
product package never imports this module.  Parity unpinned (see the header of
``rwkv7_oracle.c``): the reference has no golden vectors and cannot be built.

Every function takes and returns numpy arrays; sequence tensors are
``[B, T, H, N]`` and states ``[B, H, N, N]`` exactly as in the reference
(``crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/io.rs``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` next to the source (gcc -O3 -fopenmp)."""
    src = os.path.join(_HERE, "rwkv7_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "liboracle.so"])
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Sets the OpenMP thread count to the cores this process may run on (launchers such as
    torchrun export OMP_NUM_THREADS=1); returns the count in force."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    return int(lib().oracle_set_num_threads(ctypes.c_int(cores)))


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def wkv7(r, w, k, v, a, b, s0=None, *, precision="f64", want_state=True):
    """WKV7 recurrence. Returns ``(y, s_out)``; ``s_out`` is None when not wanted.

    ``precision="f32"`` follows the reference kernel's f32 accumulation order;
    ``"f64"`` evaluates the same definition in double on the same inputs.
    """
    r, w, k, v, a, b = (_f32(t) for t in (r, w, k, v, a, b))
    B, T, H, N = r.shape
    dt = np.float64 if precision == "f64" else np.float32
    s0c = None if s0 is None else np.ascontiguousarray(s0, dtype=dt)
    y = np.empty((B, T, H, N), dtype=dt)
    s_out = np.empty((B, H, N, N), dtype=dt) if want_state else None
    fn = lib().oracle_wkv7_f64 if precision == "f64" else lib().oracle_wkv7_f32
    fn(_p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(s0c), _p(y), _p(s_out),
       ctypes.c_int64(B), ctypes.c_int64(T), ctypes.c_int64(H), ctypes.c_int64(N))
    return y, s_out


def wkv7_train(r, w, k, v, a, b, s0=None, chunk_len=16):
    """Training forward in float64: ``(y, s_out, snapshots [B,H,T/chunk_len,N,N], state_replacement)``."""
    r, w, k, v, a, b = (_f32(t) for t in (r, w, k, v, a, b))
    B, T, H, N = r.shape
    s0d = None if s0 is None else np.ascontiguousarray(s0, dtype=np.float64)
    y = np.empty((B, T, H, N), dtype=np.float64)
    sa = np.empty((B, T, H, N), dtype=np.float64)
    s_out = np.empty((B, H, N, N), dtype=np.float64)
    snaps = np.empty((B, H, T // chunk_len, N, N), dtype=np.float64)
    lib().oracle_wkv7_train_f64(_p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(s0d), _p(y), _p(s_out), _p(snaps),
                                _p(sa), *[ctypes.c_int64(x) for x in (B, T, H, N, chunk_len)])
    return y, s_out, snaps, sa


def wkv7_backward(r, w, k, v, a, b, dy, s0=None, ds_out=None):
    """Exact reverse-mode gradients in float64: ``dict(r, w, k, v, a, b, s0)``."""
    r, w, k, v, a, b = (_f32(t) for t in (r, w, k, v, a, b))
    B, T, H, N = r.shape
    s0d = None if s0 is None else np.ascontiguousarray(s0, dtype=np.float64)
    dyd = np.ascontiguousarray(dy, dtype=np.float64)
    dsd = None if ds_out is None else np.ascontiguousarray(ds_out, dtype=np.float64)
    g = {n: np.empty((B, T, H, N), dtype=np.float64) for n in "rwkvab"}
    g["s0"] = np.empty((B, H, N, N), dtype=np.float64)
    lib().oracle_wkv7_backward_f64(_p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(s0d), _p(dyd), _p(dsd),
                                   _p(g["r"]), _p(g["w"]), _p(g["k"]), _p(g["v"]), _p(g["a"]), _p(g["b"]),
                                   _p(g["s0"]), *[ctypes.c_int64(x) for x in (B, T, H, N)])
    return g


def mix6(x, mus):
    """Six token-shift mixes; returns a float64 array ``[6, B, T, C]``."""
    x = _f32(x)
    B, T, C = x.shape
    mus = [_f32(m).reshape(C) for m in mus]
    arr = (ctypes.c_void_p * 6)(*[m.ctypes.data for m in mus])
    out = np.empty((6, B, T, C), dtype=np.float64)
    lib().oracle_mix6_f64(_p(x), arr, _p(out), ctypes.c_int64(B), ctypes.c_int64(T), ctypes.c_int64(C))
    return out


def addcmul(base, diff, scales):
    """``base + diff * scale`` for 1 or 5 scales; returns float64 ``[n, B, T, C]``."""
    base, diff = _f32(base), _f32(diff)
    B, T, C = base.shape
    scales = [_f32(s).reshape(C) for s in scales]
    n = len(scales)
    arr = (ctypes.c_void_p * n)(*[s.ctypes.data for s in scales])
    out = np.empty((n, B, T, C), dtype=np.float64)
    lib().oracle_addcmul_f64(_p(base), _p(diff), arr, ctypes.c_int(n), _p(out),
                             ctypes.c_int64(B * T), ctypes.c_int64(C))
    return out


def weight_prepare(key_precursor, learning_rate_lora, weight_decay_lora, key_removal, key_replacement,
                   num_heads, value_precursor=None, value_from_first_cell=None, value_residual_lora=None):
    """Tail of ``WeightPrepare::forward``; returns float64 ``dict(weight_decay, replacement_key,
    removal_key_normalized, replacement, value)`` (``value`` None without the value inputs)."""
    k = _f32(key_precursor)
    shape = k.shape
    C = int(np.prod(shape[2:]))
    H = int(num_heads)
    N = C // H
    rows = shape[0] * shape[1] * H
    lr, d = _f32(learning_rate_lora), _f32(weight_decay_lora)
    xi, al = _f32(key_removal).reshape(C), _f32(key_replacement).reshape(C)
    with_value = value_precursor is not None
    vp = _f32(value_precursor) if with_value else None
    vf = _f32(value_from_first_cell) if with_value else None
    nu = _f32(value_residual_lora) if with_value else None
    outs = {n: np.empty(shape, dtype=np.float64) for n in
            ("weight_decay", "replacement_key", "removal_key_normalized", "replacement")}
    value = np.empty(shape, dtype=np.float64) if with_value else None
    null = ctypes.c_void_p(0)
    lib().oracle_weight_prepare_f64(
        _p(k), _p(lr), _p(d), _p(xi), _p(al), _p(vp) if with_value else null, _p(vf) if with_value else null,
        _p(nu) if with_value else null, _p(outs["weight_decay"]), _p(outs["replacement_key"]),
        _p(outs["removal_key_normalized"]), _p(outs["replacement"]), _p(value) if with_value else null,
        ctypes.c_int64(rows), ctypes.c_int64(H), ctypes.c_int64(N))
    outs["value"] = value
    return outs


def gated_readout(wkv7_output, receptance, replacement_key, value, gate, gamma, beta, bonus, num_heads,
                  epsilon=64e-5):
    """``GatedReadout::forward`` between the gate LoRA and the output projection; float64."""
    y = _f32(wkv7_output)
    shape = y.shape
    C = int(np.prod(shape[2:]))
    H = int(num_heads)
    N = C // H
    rows = shape[0] * shape[1] * H
    r, k, v, g = _f32(receptance), _f32(replacement_key), _f32(value), _f32(gate)
    ga, be, rho = _f32(gamma).reshape(C), _f32(beta).reshape(C), _f32(bonus).reshape(C)
    out = np.empty(shape, dtype=np.float64)
    lib().oracle_gated_readout_f64(_p(y), _p(r), _p(k), _p(v), _p(g), _p(ga), _p(be), _p(rho),
                                   ctypes.c_double(epsilon), _p(out), ctypes.c_int64(rows),
                                   ctypes.c_int64(H), ctypes.c_int64(N))
    return out


def channel_mixer(x, key_scale, key_weight, value_weight):
    """``channel_mixer_reference``; ``x`` ``[B,T,C]``, ``key_weight`` ``[F,C]``, ``value_weight`` ``[C,F]``; float64."""
    x = _f32(x)
    B, T, C = x.shape
    kw, vw = _f32(key_weight), _f32(value_weight)
    F = kw.shape[0]
    out = np.empty((B, T, C), dtype=np.float64)
    lib().oracle_channel_mixer_f64(_p(x), _p(_f32(key_scale).reshape(C)), _p(kw), _p(vw), _p(out),
                                   ctypes.c_int64(B), ctypes.c_int64(T), ctypes.c_int64(C), ctypes.c_int64(F))
    return out


def token_shift_diff(x, state, ids):
    """Returns ``(diff, next_state)``; ``state`` is not modified."""
    x = _f32(x)
    B, T, C = x.shape
    st = np.array(state, dtype=np.float32, copy=True, order="C")
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    diff = np.empty((B, T, C), dtype=np.float32)
    lib().oracle_token_shift_diff_f32(_p(x), _p(st), _p(ids), _p(diff),
                                      ctypes.c_int64(B), ctypes.c_int64(T), ctypes.c_int64(C))
    return diff, st


def lm_head_ce(x, W, target):
    """Returns ``(lse, loss)`` per row, float64."""
    x, W = _f32(x), _f32(W)
    R, C = x.shape
    V = W.shape[0]
    target = np.ascontiguousarray(target, dtype=np.int64)
    lse = np.empty(R, dtype=np.float64)
    loss = np.empty(R, dtype=np.float64)
    lib().oracle_lm_head_ce_f64(_p(x), _p(W), _p(target), _p(lse), _p(loss),
                                ctypes.c_int64(R), ctypes.c_int64(C), ctypes.c_int64(V))
    return lse, loss
