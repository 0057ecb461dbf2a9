"""world_size-2 gloo tests (CPU) of the multi-GPU host logic: shard geometry and
the vocabulary-sharded LM-head combine over an all-gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _partials_cpu(x, w, targets, lo):
    z = x.double() @ w.double().T
    m = z.max(dim=1).values
    s = torch.exp(z - m[:, None]).sum(dim=1)
    local = targets - lo
    own = (local >= 0) & (local < w.shape[0])
    zt = torch.where(own, z.gather(1, local.clamp(0, w.shape[0] - 1)[:, None])[:, 0], torch.zeros_like(m))
    return torch.stack([m, s, zt], dim=1)


def _worker(rank, world, port, root, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import sys
    sys.path.insert(0, root)
    import __graft_entry__ as entry
    entry.load_package()
    from rwkv_rs_stable_b200 import dist as rdist, workloads
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        R, C, V = 64, 32, 101                       # V not divisible by the world size
        x, w, tg = workloads.lm_head_inputs(R, C, V, seed=4)
        tg[::5] = -1
        lo, hi = rdist.vocab_shard(V, rank, world)
        parts = _partials_cpu(x, w[lo:hi], tg, lo)
        allp = rdist.gather_partials(parts)
        assert allp.shape == (world, R, 3)
        lse, loss = rdist.combine_partials_reference(allp, tg)
        z = x.double() @ w.double().T
        ref_lse = torch.logsumexp(z, dim=1)
        ref_loss = torch.nn.functional.cross_entropy(z, tg.clamp_min(0), reduction="none")
        ref_loss[tg < 0] = 0
        ok = torch.allclose(lse, ref_lse, rtol=1e-10, atol=1e-10) and torch.allclose(loss, ref_loss, rtol=1e-10, atol=1e-10)
        result[rank] = 1 if ok else 0
    finally:
        dist.destroy_process_group()


def _gather_worker(rank, world, port, root, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import sys
    sys.path.insert(0, root)
    import __graft_entry__ as entry
    entry.load_package()
    from rwkv_rs_stable_b200 import dist as rdist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ok = True
        for B, H in ((4, 3), (1, 6), (3, 4)):       # batch split, head split, head split with B > 1
            full = torch.arange(B * 5 * H * 2, dtype=torch.float32).reshape(B, 5, H, 2)
            bs, hs = rdist.shard_ranges(B, H, world)[rank]
            got = rdist.gather_outputs(full[bs, :, hs].contiguous(), B, H)
            ok = ok and torch.equal(got, full)
        result[rank] = 1 if ok else 0
    finally:
        dist.destroy_process_group()


def test_output_gather_two_ranks():
    """C1: every rank ends with the full [B,T,H,N] output, for batch and for head splits."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ctx = mp.get_context("spawn")
    result = ctx.Array("i", [0, 0])
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, root, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert list(result) == [1, 1]


def test_vocab_sharded_combine_two_ranks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ctx = mp.get_context("spawn")
    result = ctx.Array("i", [0, 0])
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, root, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert list(result) == [1, 1]


@pytest.mark.parametrize("B,H,world", [(8, 12, 1), (8, 12, 2), (8, 12, 4), (8, 12, 8), (16, 32, 8), (4, 64, 8),
                                       (1024, 40, 8), (2, 12, 4), (3, 12, 4)])
def test_shard_ranges_cover_every_chain_once(pkg, B, H, world):
    from rwkv_rs_stable_b200 import dist as rdist
    cover = np.zeros((B, H), dtype=int)
    sizes = set()
    for bs, hs in rdist.shard_ranges(B, H, world):
        cover[bs, hs] += 1
        sizes.add(cover[bs, hs].size)
    assert (cover == 1).all() and len(sizes) == 1


def test_shard_ranges_rejects_ragged_split(pkg):
    from rwkv_rs_stable_b200 import dist as rdist
    with pytest.raises(ValueError):
        rdist.shard_ranges(3, 5, 4)


def test_vocab_shard_partition(pkg):
    from rwkv_rs_stable_b200 import dist as rdist
    for V, world in ((65536, 8), (101, 2), (7, 8)):
        edges = [rdist.vocab_shard(V, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == V
        assert all(a[1] == b[0] for a, b in zip(edges[:-1], edges[1:]))
