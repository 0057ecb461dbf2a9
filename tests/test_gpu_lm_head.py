"""GPU parity of the fused LM-head cross entropy against the fp64 CPU oracle,
through the C ABI.  The operator has no reference implementation (parity
unpinned); the oracle itself is checked against torch's cross_entropy on CPU.
Tolerance: bf16 products are exact in fp32, so only accumulation order and the
exp2 approximation differ: 2e-4 absolute on lse / loss (values are O(10))."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(pkg, oracle, workloads, cuda, R, C, V, shards=1, ignore=True):
    x, w, tg = workloads.lm_head_inputs(R, C, V, seed=R + V)
    x = x * 4  # spread the logits so that the max/sum-exp bookkeeping is exercised
    if ignore:
        tg[::7] = -1
    lse_ref, loss_ref = oracle.lm_head_ce(x.float().numpy(), w.float().numpy(), tg.numpy())
    xg, wg, tgg = x.to(cuda), w.to(cuda), tg.to(cuda)
    if shards == 1:
        lse, loss = pkg.lm_head_ce(xg, wg, tgg)
    else:
        bounds = np.linspace(0, V, shards + 1).astype(int)
        parts = [pkg.lm_head_ce_partial(xg, wg[lo:hi].contiguous(), tgg, int(lo))
                 for lo, hi in zip(bounds[:-1], bounds[1:])]
        lse, loss = pkg.lm_head_ce_finalize(torch.stack(parts), tgg)
    torch.cuda.synchronize()
    assert pkg.read_device_status(0) == 0
    np.testing.assert_allclose(lse.cpu().numpy(), lse_ref, rtol=0, atol=2e-4)
    np.testing.assert_allclose(loss.cpu().numpy(), loss_ref, rtol=0, atol=2e-4)


@pytest.mark.parametrize("R,C,V", [(128, 64, 256), (300, 128, 1000), (77, 192, 513), (1024, 512, 4096)])
def test_lm_head_ce(pkg, oracle, workloads, cuda, R, C, V):
    _check(pkg, oracle, workloads, cuda, R, C, V)


def test_lm_head_ce_vocab_shards(pkg, oracle, workloads, cuda):
    """Vocabulary-sharded partials (as on 2 and 3 GPUs) combined by the finalize step."""
    _check(pkg, oracle, workloads, cuda, 200, 128, 1536, shards=2)
    _check(pkg, oracle, workloads, cuda, 200, 128, 1000, shards=3)


def test_lm_head_ce_int32_targets_and_many_rows(pkg, oracle, workloads, cuda):
    R, C, V = 40000, 64, 512   # more row blocks than 2 x SMs: no vocabulary split
    x, w, tg = workloads.lm_head_inputs(R, C, V, seed=3)
    lse_ref, loss_ref = oracle.lm_head_ce(x.float().numpy(), w.float().numpy(), tg.numpy())
    lse, loss = pkg.lm_head_ce(x.to(cuda), w.to(cuda), tg.to(torch.int32).to(cuda))
    torch.cuda.synchronize()
    np.testing.assert_allclose(lse.cpu().numpy(), lse_ref, rtol=0, atol=2e-4)
    np.testing.assert_allclose(loss.cpu().numpy(), loss_ref, rtol=0, atol=2e-4)


def test_lm_head_ce_at_the_benchmark_vocabulary(pkg, oracle, workloads, cuda):
    """A 256-row slice of configuration 2's LM head at its real width and vocabulary
    (C = 2048, V = 65 536, weights N(0, 0.02), hidden rows N(0, 1)) against the fp64 oracle."""
    R, C, V = 256, 2048, 65536
    x, w, tg = workloads.lm_head_inputs(R, C, V, seed=11)
    tg[::9] = -1
    lse_ref, loss_ref = oracle.lm_head_ce(x.float().numpy(), w.float().numpy(), tg.numpy())
    lse, loss = pkg.lm_head_ce(x.to(cuda), w.to(cuda), tg.to(cuda))
    torch.cuda.synchronize()
    assert pkg.read_device_status(0) == 0
    np.testing.assert_allclose(lse.cpu().numpy(), lse_ref, rtol=0, atol=2e-4)
    np.testing.assert_allclose(loss.cpu().numpy(), loss_ref, rtol=0, atol=2e-4)


def test_lm_head_ce_partial_at_the_long_context_shard_shape(pkg, workloads, cuda):
    """One vocabulary shard of configuration 4 (C = 4096, 8192 of 65 536 columns, the fourth of eight
    shards, so vocab_offset = 24 576): the per-row triple (max, sum of exp, target logit) against an fp64
    computation of the shard's logits.  Targets fall inside the shard, on either side of it, and on the
    ignore index; the target logit is zero for every row whose target lies outside."""
    R, C, Vs, off = 256, 4096, 8192, 3 * 8192
    x, w, _ = workloads.lm_head_inputs(R, C, Vs, seed=12)
    g = torch.Generator().manual_seed(99)
    tg = torch.randint(0, 65536, (R,), generator=g, dtype=torch.int64)
    tg[0::4] = off + torch.randint(0, Vs, (R // 4,), generator=g)     # inside the shard
    tg[1] = off - 1; tg[2] = off + Vs; tg[3] = -1; tg[4] = off; tg[8] = off + Vs - 1
    z = x.double().numpy() @ w.double().numpy().T
    m_ref = z.max(axis=1)
    s_ref = np.exp(z - m_ref[:, None]).sum(axis=1)
    tn = tg.numpy()
    inside = (tn >= off) & (tn < off + Vs)
    zt_ref = np.where(inside, z[np.arange(R), np.clip(tn - off, 0, Vs - 1)], 0.0)
    part = pkg.lm_head_ce_partial(x.to(cuda), w.to(cuda), tg.to(cuda), off)
    torch.cuda.synchronize()
    assert pkg.read_device_status(0) == 0
    p = part.cpu().numpy().astype(np.float64)
    # the kernel may report any reference maximum as long as (max, sum) describe the same sum of exponentials
    np.testing.assert_allclose(p[:, 0] + np.log(p[:, 1]), m_ref + np.log(s_ref), rtol=0, atol=2e-4)
    assert np.all(p[:, 0] <= m_ref + 1e-3)
    np.testing.assert_allclose(p[:, 2], zt_ref, rtol=0, atol=2e-4)
    assert np.all(p[~inside, 2] == 0.0)
