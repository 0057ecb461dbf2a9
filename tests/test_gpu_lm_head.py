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
