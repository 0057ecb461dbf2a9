"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the
header declares, and rejects bad inputs with the reference's error kinds before
touching CUDA.  Mirrors the reference's panic tests (wkv7/mod.rs:329-336,
mix6/mod.rs:248-257, token_shift_diff/mod.rs:330-347)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pkg):
    header = open(os.path.join(ROOT, "include", "rwkv7_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = set(re.findall(r"\b(rwkv7_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 18
    L = pkg.lib()
    for n in sorted(names):
        assert hasattr(L, n), f"librwkv7_b200.so does not export {n}"
    assert L.rwkv7_abi_version() == 1
    assert L.rwkv7_status_string(2) == b"ShapeMismatch"


def test_tensor_struct_layout(pkg):
    # data(8) dtype device ndim reserved (4x4) shape[5] stride[5] (2x40)
    assert ctypes.sizeof(pkg.Tensor) == 8 + 16 + 40 + 40


def _seq(pkg, shape, dtype=torch.float32, chunk_len=16):
    t = [torch.zeros(shape, dtype=dtype) for _ in range(6)]
    return pkg.Wkv7PretrainForwardInputs(*t, chunk_len=chunk_len)


def test_wkv7_panics_on_wrong_context_len(pkg):
    """wkv7/mod.rs:329-336: T = 15 is rejected by the reference contract."""
    with pytest.raises(pkg.KernelInputsError, match="multiple of chunk_len"):
        pkg.wkv7_pretrain_custom(_seq(pkg, (1, 15, 1, 4)))
    with pytest.raises(pkg.KernelInputsError, match="chunk_len=16"):
        pkg.wkv7_pretrain_custom(_seq(pkg, (1, 16, 1, 4), chunk_len=32))


def test_wkv7_contract_errors(pkg):
    E = pkg.KernelInputsError
    seq = _seq(pkg, (2, 16, 2, 8))
    seq.value = torch.zeros(2, 16, 2, 4)
    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(seq)
    assert e.value.kind == "ShapeMismatch" and "value" in str(e.value)
    assert "expected=[2, 16, 2, 8], actual=[2, 16, 2, 4]" in str(e.value)

    seq = _seq(pkg, (2, 16, 2, 8))
    seq.replacement = torch.zeros(3, 16, 2, 8)
    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(seq)
    assert e.value.kind == "AxisMismatch"
    assert "receptance[0]=2 != replacement[0]=3" in str(e.value)

    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(_seq(pkg, (2, 0, 2, 8)), reference_contract=False)
    assert e.value.kind == "EmptyAxis" and "receptance[1]" in str(e.value)
    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(_seq(pkg, (2, 16, 2, 0)))
    assert e.value.kind == "EmptyAxis" and "receptance[3]" in str(e.value)

    seq = _seq(pkg, (2, 16, 2, 8))
    seq.weight_decay = torch.zeros(2, 16, 2, 8, dtype=torch.bfloat16)
    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(seq)
    assert e.value.kind == "DTypeMismatch" and "weight_decay=BF16" in str(e.value)

    seq = _seq(pkg, (2, 16, 2, 8))
    seq.receptance = torch.zeros(2, 16, 8, 2).transpose(2, 3)
    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(seq)
    assert e.value.kind == "NotContiguous" and "receptance" in str(e.value)

    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(_seq(pkg, (1, 16, 1, 4), chunk_len=0), reference_contract=False)
    assert e.value.kind == "BadChunk"

    # initial_state must be [B,H,N,N] (check_initial_state, wkv7/io.rs:243-258)
    with pytest.raises(E) as e:
        pkg.wkv7_statepass_custom(torch.zeros(2, 2, 8, 4), _seq(pkg, (2, 16, 2, 8)))
    assert e.value.kind == "ShapeMismatch" and "initial_state" in str(e.value)
    with pytest.raises(E) as e:
        pkg.wkv7_statetune_custom(torch.zeros(2, 2, 8, 8, dtype=torch.bfloat16), _seq(pkg, (2, 16, 2, 8)))
    assert e.value.kind == "DTypeMismatch"

    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(_seq(pkg, (1, 16, 1, 8), dtype=torch.float16))
    assert e.value.kind == "Unsupported"


def test_wkv7_device_mismatch_is_reported(pkg):
    seq = _seq(pkg, (1, 16, 1, 4))
    six = [pkg.describe(t, device=0) for t in seq.six()]
    six[3].device = 1
    y = pkg.describe(torch.zeros(1, 16, 1, 4), device=0)
    st = pkg.lib().rwkv7_fused_wkv7_pretrain(*[ctypes.byref(d) for d in six], ctypes.c_int64(16),
                                             ctypes.byref(y), None, ctypes.c_size_t(0), None)
    assert st == 4
    assert b"DeviceMismatch" in pkg.lib().rwkv7_last_error_message()


def test_null_descriptor(pkg):
    seq = _seq(pkg, (1, 16, 1, 4))
    six = [pkg.describe(t, device=0) for t in seq.six()]
    y = pkg.describe(torch.zeros(1, 16, 1, 4), device=0)
    args = [ctypes.byref(d) for d in six]
    args[2] = None
    st = pkg.lib().rwkv7_fused_wkv7_pretrain(*args, ctypes.c_int64(16), ctypes.byref(y), None,
                                             ctypes.c_size_t(0), None)
    assert st == 9 and b"replacement_key" in pkg.lib().rwkv7_last_error_message()


def test_mix6_panics_on_wrong_scale_shape(pkg):
    """mix6/mod.rs:248-257: gate_scale [1,1,7] against C = 8."""
    x = torch.zeros(2, 4, 8)
    mus = [torch.zeros(1, 1, 8) for _ in range(5)] + [torch.zeros(1, 1, 7)]
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.mix6_custom(x, *mus)
    assert e.value.kind == "ShapeMismatch" and "gate_scale" in str(e.value)
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.mix6_custom(torch.zeros(2, 4, 0), *[torch.zeros(1, 1, 0) for _ in range(6)])
    assert e.value.kind == "EmptyAxis"


def test_addcmul_contract_errors(pkg):
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.addcmul_custom(torch.zeros(2, 8, 32), torch.zeros(2, 8, 16), torch.zeros(1, 1, 32))
    assert e.value.kind == "ShapeMismatch" and "diff" in str(e.value)
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.addcmul_custom(torch.zeros(2, 8, 32), torch.zeros(2, 8, 32), torch.zeros(32))
    assert e.value.kind == "ShapeMismatch" and "scale" in str(e.value)
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.addcmul5_custom(torch.zeros(2, 8, 32), torch.zeros(2, 8, 32),
                            *[torch.zeros(1, 1, 32) for _ in range(4)], torch.zeros(1, 1, 31))
    assert e.value.kind == "ShapeMismatch" and "learning_rate_scale" in str(e.value)


def test_token_shift_diff_shape_mismatch_panics(pkg):
    """token_shift_diff/mod.rs:330-347: state [3,7] against C = 8."""
    with pytest.raises(pkg.KernelInputsError, match="ShapeMismatch") as e:
        pkg.token_shift_diff_custom(torch.zeros(2, 4, 8), torch.zeros(3, 7), torch.tensor([0, 1], dtype=torch.int32))
    assert "embedded_token_shift" in str(e.value)
    with pytest.raises(pkg.KernelInputsError, match="ShapeMismatch") as e:
        pkg.token_shift_diff_custom(torch.zeros(2, 4, 8), torch.zeros(3, 8), torch.tensor([0], dtype=torch.int32))
    assert "batch_ids" in str(e.value)


def test_token_shift_diff_empty_context_is_noop(pkg):
    """T == 0 returns without any CUDA call (token_shift_diff/mod.rs:88-97)."""
    state = torch.rand(4, 8)
    out = pkg.token_shift_diff_custom(torch.zeros(2, 0, 8), state, torch.tensor([3, 1], dtype=torch.int32))
    assert out.token_shifted_diff.shape == (2, 0, 8)
    assert torch.equal(out.next_token_shift, state)


def test_lm_head_contract_errors(pkg):
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    w = torch.zeros(16, 32, dtype=torch.bfloat16)
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.lm_head_ce_partial(x, w, torch.zeros(4, dtype=torch.int64))
    assert e.value.kind == "AxisMismatch"
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.lm_head_ce_partial(x.float(), torch.zeros(16, 64), torch.zeros(4, dtype=torch.int64))
    assert e.value.kind == "Unsupported"


def test_no_cpu_fallback(pkg):
    """Valid inputs without a CUDA device must fail loudly, not compute on the host."""
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.wkv7_pretrain_custom(_seq(pkg, (1, 16, 1, 4)))
    assert e.value.kind in ("CudaError", "BadArgument")


def test_wkv7_path_switch(pkg):
    assert pkg.get_wkv7_path() == pkg.WKV7_AUTO
    pkg.set_wkv7_path(pkg.WKV7_SEQUENTIAL)
    assert pkg.get_wkv7_path() == pkg.WKV7_SEQUENTIAL
    pkg.set_wkv7_path(pkg.WKV7_AUTO)
    with pytest.raises(pkg.KernelInputsError):
        pkg.set_wkv7_path(9)


def test_unaligned_views_are_refused_on_the_host(pkg):
    """A contiguous view that starts at an odd element of its storage is not 16-byte aligned.  Every
    kernel (forward, both backward paths, the streaming kernels) uses 16-byte vector accesses or TMA, so
    such a tensor is refused by the host-side contract check instead of faulting on the device."""
    E = pkg.KernelInputsError
    shape = (1, 64, 2, 64)
    base = torch.zeros(1 * 64 * 2 * 64 + 1, dtype=torch.bfloat16)
    view = base[1:].view(shape)
    assert view.is_contiguous() and view.data_ptr() % 16 != 0
    seq = _seq(pkg, shape, dtype=torch.bfloat16)
    seq.receptance = view
    with pytest.raises(E) as e:
        pkg.wkv7_pretrain_custom(seq)
    assert e.value.kind == "Unsupported" and "16-byte aligned" in str(e.value) and "receptance" in str(e.value)
    # the backward entry points share the check
    good = _seq(pkg, shape, dtype=torch.bfloat16)
    saved = pkg.Wkv7SavedForward(output=None, next_state=None, snapshots=torch.zeros(1, 2, 4, 64, 64),
                                 state_replacement=torch.zeros(shape, dtype=torch.bfloat16))
    for parallel in (True, False):
        with pytest.raises(E) as e:
            pkg.wkv7_backward(good, saved, view, None, parallel=parallel)
        assert e.value.kind == "Unsupported" and "16-byte aligned" in str(e.value)
    with pytest.raises(E) as e:
        pkg.addcmul_custom(view.view(1, 64, 128), torch.zeros(1, 64, 128, dtype=torch.bfloat16),
                           torch.zeros(1, 1, 128, dtype=torch.bfloat16))
    assert e.value.kind == "Unsupported" and "16-byte aligned" in str(e.value)


def test_host_statepass_contract(pkg):
    """``rwkv7_wkv7_statepass_host``: the device-resident statepass's contract applied to host descriptors, plus
    its own arguments (slices dividing the batch, device staging of the reported size); all checked on the host."""
    L = pkg.lib()
    L.rwkv7_wkv7_host_staging_bytes.restype = ctypes.c_size_t
    L.rwkv7_wkv7_host_staging_bytes.argtypes = [ctypes.c_int64] * 4 + [ctypes.c_int32] * 3
    B, T, H, N = 4, 64, 2, 64
    need = L.rwkv7_wkv7_host_staging_bytes(B, T, H, N, pkg.BF16, 2, 2)
    seq_bytes, state_bytes = 2 * T * H * N * 2, 2 * H * N * N * 4
    assert need >= 2 * (7 * seq_bytes + 2 * state_bytes)
    assert L.rwkv7_wkv7_host_staging_bytes(B, T, H, N, pkg.BF16, 3, 2) == 0      # 3 slices do not divide B = 4
    six = [torch.zeros(B, T, H, N, dtype=torch.bfloat16) for _ in range(6)]
    y = torch.zeros(B, T, H, N, dtype=torch.bfloat16)
    s = torch.zeros(B, H, N, N)
    desc = [pkg.describe(t, device=-1) for t in six]
    arr = (ctypes.POINTER(pkg.Tensor) * 6)(*[ctypes.pointer(d) for d in desc])
    yd, sd = pkg.describe(y, device=-1), pkg.describe(s, device=-1)
    streams = (ctypes.c_void_p * 1)(None)

    def call(slices, staging_bytes, six_arr=arr):
        return L.rwkv7_wkv7_statepass_host(None, six_arr, ctypes.c_int64(16), ctypes.byref(yd), ctypes.byref(sd),
                                           ctypes.c_int32(0), ctypes.c_int32(slices), ctypes.c_void_p(256),
                                           ctypes.c_size_t(staging_bytes), streams, ctypes.c_int32(1),
                                           ctypes.c_void_p(None), ctypes.c_int32(0))

    assert L.rwkv7_status_string(call(3, 1 << 30)) == b"ShapeMismatch"
    assert L.rwkv7_status_string(call(2, 1024)) == b"WorkspaceTooSmall"
    bad = [pkg.describe(t, device=-1) for t in six]
    bad[3] = pkg.describe(torch.zeros(B, T, H, 32, dtype=torch.bfloat16), device=-1)
    bad_arr = (ctypes.POINTER(pkg.Tensor) * 6)(*[ctypes.pointer(d) for d in bad])
    assert L.rwkv7_status_string(call(2, 1 << 30, bad_arr)) == b"ShapeMismatch"
    assert b"value" in L.rwkv7_last_error_message()
    on_device = [pkg.describe(t, device=0) for t in six]
    dev_arr = (ctypes.POINTER(pkg.Tensor) * 6)(*[ctypes.pointer(d) for d in on_device])
    assert L.rwkv7_status_string(call(2, 1 << 30, dev_arr)) == b"DeviceMismatch"
