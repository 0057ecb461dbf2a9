"""Second, independent restatement of the reference's tensor-op definitions in
torch fp64, written operation by operation after the reference's Burn code so
that it shares no code with ``oracle/rwkv7_oracle.c``.  Used only to cross-check
the C oracle.
"""
import torch


def wkv7_reference_with_state(r, w, k, v, a, b, state):
    """crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:179-242."""
    r, w, k, v, a, b = (t.double() for t in (r, w, k, v, a, b))
    B, T, H, N = r.shape
    state = torch.zeros(B, H, N, N, dtype=torch.float64) if state is None else state.double().clone()
    outputs = []
    for t in range(T):
        receptance = r[:, t]                      # [B,H,N]
        decay = (-(w[:, t].exp())).exp()
        replacement_key = k[:, t]
        value = v[:, t]
        removal = a[:, t]
        replacement = b[:, t]
        state_replacement = (state * removal.unsqueeze(2)).sum(dim=3)          # [B,H,N]
        state = (state * decay.unsqueeze(2)
                 + state_replacement.unsqueeze(3) * replacement.unsqueeze(2)
                 + value.unsqueeze(3) * replacement_key.unsqueeze(2))
        outputs.append((state * receptance.unsqueeze(2)).sum(dim=3).reshape(B, 1, H, N))
    return torch.cat(outputs, dim=1), state


def mix6_reference(x, mus):
    """crates/rwkv-nn/src/kernels/train/time_mixer/mix6/mod.rs:111-156."""
    x = x.double()
    B, T, C = x.shape
    if T == 0:
        return [x.clone() for _ in range(6)]
    zero = torch.zeros(B, 1, C, dtype=torch.float64)
    shifted = zero if T == 1 else torch.cat([zero, x[:, : T - 1]], dim=1)
    diff = shifted - x
    return [x + diff * m.double() for m in mus]


def addcmul_reference(base, diff, scale):
    """crates/rwkv-nn/src/kernels/template/addcmul/mod.rs:122-124."""
    return base.double() + diff.double() * scale.double()


def token_shift_diff_reference(x, state, ids):
    """crates/rwkv-nn/src/kernels/template/token_shift_diff/mod.rs:114-155,170-200."""
    B, T, C = x.shape
    if T == 0:
        return x.clone(), state.clone()
    active = state.index_select(0, ids)
    shifted = active.unsqueeze(1) if T == 1 else torch.cat([active.unsqueeze(1), x[:, : T - 1]], dim=1)
    diff = shifted - x
    last = x[:, T - 1]
    selected = torch.zeros(state.shape[0], dtype=state.dtype).index_add(0, ids, torch.ones(B, dtype=state.dtype))
    nxt = (state * (1 - selected).unsqueeze(1)).index_add(0, ids, last)
    return diff, nxt
