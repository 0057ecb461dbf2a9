"""GPU parity of mix6, addcmul, addcmul5 and token_shift_diff against the CPU
oracle, through the C ABI, on the reference's own test shapes plus bf16, odd
channel counts and benchmark-sized rows.  fp32: 1e-6 relative (the kernels fuse
the multiply-add; the reference's tolerances are 1e-4 abs for mix6 and Burn's
default elsewhere).  bf16: fp32 arithmetic rounded once, within one bf16 spacing."""
import numpy as np
import pytest
import torch

import parity

pytestmark = pytest.mark.gpu


def _check(x, ref, dtype):
    x = x.float().cpu().numpy().astype(np.float64)
    if dtype == torch.bfloat16:
        assert (np.abs(x - ref) <= parity.BF16_ULP * np.abs(ref) + 1e-30).all()
    else:
        np.testing.assert_allclose(x, ref, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 8, 32), (1, 3, 17), (3, 1, 64), (2, 40, 768), (1, 33, 2056)])
def test_mix6(pkg, oracle, workloads, cuda, shape, dtype):
    """mix6/mod.rs:193-204 shapes [2,8,32] and [1,3,17] (odd C) and larger ones."""
    x, mus = workloads.mix_inputs(*shape, seed=1, dtype=dtype)
    ref = oracle.mix6(x.float().numpy(), [m.float().numpy() for m in mus])
    out = pkg.mix6_custom(x.to(cuda), *[m.to(cuda) for m in mus])
    stacked = pkg.mix6_custom(x.to(cuda), *[m.to(cuda) for m in mus], stacked=True)
    torch.cuda.synchronize()
    for i, name in enumerate(pkg.MIX6_BRANCHES):
        _check(out[name], ref[i], dtype)
        assert torch.equal(stacked[i], out[name])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 8, 32), (1, 5, 17), (2, 40, 768)])
def test_addcmul_and_addcmul5(pkg, oracle, workloads, cuda, shape, dtype):
    """addcmul/mod.rs:194-269: [2,8,32] with scale [1,1,32]."""
    base, mus = workloads.mix_inputs(*shape, seed=2, dtype=dtype, nscale=5)
    diff, _ = workloads.mix_inputs(*shape, seed=3, dtype=dtype, nscale=1)
    ref = oracle.addcmul(base.float().numpy(), diff.float().numpy(), [m.float().numpy() for m in mus])
    b, d, m = base.to(cuda), diff.to(cuda), [t.to(cuda) for t in mus]
    one = pkg.addcmul_custom(b, d, m[0])
    five = pkg.addcmul5_custom(b, d, *m)
    inplace = b.clone()
    ret = pkg.addcmul_custom(inplace, d, m[0], inplace=True)
    torch.cuda.synchronize()
    _check(one, ref[0], dtype)
    assert ret.data_ptr() == inplace.data_ptr() and torch.equal(inplace, one)
    for i, name in enumerate(pkg.MIX6_BRANCHES[:5]):
        _check(five[name], ref[i], dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ids_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("B,T,C,S,ids", [(1, 1, 8, 1, [0]), (1, 4, 8, 3, [2]), (3, 5, 16, 8, [6, 1, 4]),
                                         (2, 0, 8, 4, [3, 1]), (4, 50, 776, 9, [8, 0, 3, 5]),
                                         (2, 16, 17, 4, [1, 2])])
def test_token_shift_diff(pkg, oracle, cuda, B, T, C, S, ids, ids_dtype, dtype):
    """token_shift_diff/mod.rs:222-227 cases (T == 0 included) plus larger ones."""
    g = torch.Generator().manual_seed(5)
    x = torch.rand((B, T, C), generator=g).to(dtype)
    state = torch.rand((S, C), generator=g).to(dtype)
    idt = torch.tensor(ids, dtype=ids_dtype)
    d_ref, s_ref = oracle.token_shift_diff(x.float().numpy(), state.float().numpy(), idt.numpy())
    out = pkg.token_shift_diff_custom(x.to(cuda), state.to(cuda), idt.to(cuda))
    torch.cuda.synchronize()
    assert tuple(out.token_shifted_diff.shape) == (B, T, C)
    if T:
        _check(out.token_shifted_diff, d_ref.astype(np.float64), dtype)
    # the carried rows are copies: bit-exact
    assert torch.equal(out.next_token_shift.float().cpu(), torch.from_numpy(s_ref))
    assert pkg.read_device_status(0) == 0


def test_token_shift_diff_bad_id_is_reported_not_faulted(pkg, cuda):
    x = torch.rand(2, 4, 8, device=cuda)
    state = torch.rand(3, 8, device=cuda)
    before = state.clone()
    out = pkg.token_shift_diff_custom(x, state, torch.tensor([1, 7], dtype=torch.int32, device=cuda))
    torch.cuda.synchronize()
    assert pkg.read_device_status(0) == 13  # BadIndex
    assert pkg.read_device_status(0) == 0   # cleared by the read
    assert torch.equal(out.next_token_shift[0], before[0]) and torch.equal(out.next_token_shift[2], before[2])
    assert torch.equal(out.next_token_shift[1], x[0, 3])
