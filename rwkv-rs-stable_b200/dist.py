"""Multi-GPU plumbing for the WKV7 hot path (one process per GPU, torch.distributed).

WKV7 itself needs no exchange: (b,h) chains are independent, so every rank runs
the kernels on its own batch x head shard.  The only collective on this path is
the vocabulary-sharded LM-head combine: each rank holds per-row partial triples
``(max, sum-exp, target logit)`` over its vocabulary shard (12 bytes per row),
the triples are all-gathered and combined on every rank.  NCCL has no custom
reduction operator, hence all-gather + combine rather than all-reduce.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_ranges(B: int, H: int, world: int) -> list[tuple[slice, slice]]:
    """Contiguous batch x head shards, one per rank: whole-batch splits when the
    batch divides evenly over the ranks, else whole-head splits, else a split of
    the flattened (b,h) index into near-equal runs of heads inside one batch row."""
    if B % world == 0:
        n = B // world
        return [(slice(r * n, (r + 1) * n), slice(0, H)) for r in range(world)]
    if H % world == 0:
        n = H // world
        return [(slice(0, B), slice(r * n, (r + 1) * n)) for r in range(world)]
    if world % B == 0 and H % (world // B) == 0:
        per_b = world // B
        n = H // per_b
        return [(slice(r // per_b, r // per_b + 1), slice((r % per_b) * n, (r % per_b + 1) * n))
                for r in range(world)]
    raise ValueError(f"cannot split B={B}, H={H} into {world} rectangular batch x head shards")


def gather_outputs(y_local: torch.Tensor, B: int, H: int, group=None) -> torch.Tensor:
    """All-gathers the per-rank y shards (``[B_loc, T, H_loc, N]``, cut as :func:`shard_ranges`
    cuts them) into the full ``[B, T, H, N]`` tensor on every rank.  Only for consumers that
    need the whole tensor; the WKV7 path itself never calls it.  A batch split is one
    all-gather into place; a head split gathers ``[world, B_loc, T, H_loc, N]`` and moves the
    head blocks into their slots with one strided copy (whole-head shards) or one per rank."""
    world = dist.get_world_size(group)
    ranges = shard_ranges(B, H, world)
    T, N = y_local.shape[1], y_local.shape[3]
    gathered = torch.empty((world,) + tuple(y_local.shape), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(gathered.view(-1, *y_local.shape[1:]), y_local.contiguous(), group=group)
    if ranges[0][1] == slice(0, H):      # whole-batch shards: the gather already is [B, T, H, N]
        return gathered.view(B, T, H, N)
    full = torch.empty((B, T, H, N), dtype=y_local.dtype, device=y_local.device)
    if ranges[0][0] == slice(0, B):      # whole-head shards: one strided copy [world,B,T,H_loc,N] -> [B,T,world,H_loc,N]
        full.view(B, T, world, H // world, N).copy_(gathered.permute(1, 2, 0, 3, 4))
        return full
    for r, (bs, hs) in enumerate(ranges):
        full[bs, :, hs] = gathered[r]
    return full


def vocab_shard(V: int, rank: int, world: int) -> tuple[int, int]:
    """``[lo, hi)`` rows of the LM-head weight owned by ``rank`` (near-equal, contiguous)."""
    base, rem = divmod(V, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def gather_partials(partials: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers the ``[R,3]`` partial triples of every rank into ``[world,R,3]``."""
    world = dist.get_world_size(group)
    R = partials.shape[0]
    out = torch.empty((world * R,) + tuple(partials.shape[1:]), dtype=partials.dtype, device=partials.device)
    dist.all_gather_into_tensor(out, partials.contiguous(), group=group)   # concatenated along rows
    return out.view((world, R) + tuple(partials.shape[1:]))


def combine_partials_reference(partials_all: torch.Tensor, targets: torch.Tensor):
    """The combine in plain torch: ``M = max_g m_g``, ``lse = M + log sum_g s_g exp(m_g - M)``,
    ``loss = lse - sum_g zt_g`` (0 for ignored rows).  The GPU path runs the same
    arithmetic in ``rwkv7_lm_head_ce_finalize``; this version documents it and
    serves the CPU (gloo) tests."""
    m, s, zt = partials_all[..., 0], partials_all[..., 1], partials_all[..., 2]
    M = m.max(dim=0).values
    lse = M + torch.log((s * torch.exp(m - M)).sum(dim=0))
    loss = torch.where(targets >= 0, lse - zt.sum(dim=0), torch.zeros_like(lse))
    return lse, loss


def lm_head_ce_sharded(pkg, x: torch.Tensor, weight_shard: torch.Tensor, targets: torch.Tensor,
                       vocab_offset: int, group=None):
    """Vocabulary-sharded fused LM-head cross entropy: local partials on this
    rank's shard, all-gather of the triples, combine.  Returns per-row ``(lse, loss)``."""
    partials = pkg.lm_head_ce_partial(x, weight_shard, targets, vocab_offset)
    return pkg.lm_head_ce_finalize(gather_partials(partials, group), targets)
