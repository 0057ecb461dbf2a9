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


def weight_prepare_reference(key_precursor, learning_rate_lora, weight_decay_lora, key_removal, key_replacement,
                             num_heads, value_precursor=None, value_from_first_cell=None,
                             value_residual_lora=None):
    """``WeightPrepare::forward`` after the projections (``weight_prepare.rs:252-287``), with torch
    tensor ops in the order the reference applies them."""
    B, T, C = key_precursor.shape
    learning_rate = torch.sigmoid(learning_rate_lora)
    alpha_modulated = key_replacement * (learning_rate - 1.0) + 1.0
    replacement_key = key_precursor * alpha_modulated
    weight_decay = -torch.nn.functional.softplus(-weight_decay_lora, beta=1.0, threshold=1e9) - 0.5
    removal_key = (key_precursor * key_removal).reshape(B, T, num_heads, C // num_heads)
    norm = removal_key.abs().pow(2.0).sum(-1, keepdim=True).pow(0.5).clamp_min(1e-12)
    removal_key_normalized = -(removal_key / norm).reshape(B, T, C)
    replacement = -removal_key_normalized * learning_rate
    value = None
    if value_precursor is not None:
        nu = torch.sigmoid(value_residual_lora)
        value = value_precursor + (value_from_first_cell - value_precursor) * nu
    return dict(weight_decay=weight_decay, replacement_key=replacement_key,
                removal_key_normalized=removal_key_normalized, replacement=replacement, value=value)


def gated_readout_reference(wkv7_output, receptance, replacement_key, value, gate, gamma, beta, bonus,
                            num_heads, epsilon=64e-5):
    """``GatedReadout::forward`` (``gated_readout.rs:123-141``) with torch's own GroupNorm."""
    B, T, C = wkv7_output.shape
    N = C // num_heads
    norm = torch.nn.functional.group_norm(wkv7_output.reshape(B * T, C), num_heads, gamma.reshape(C),
                                          beta.reshape(C), epsilon).reshape(B, T, C)
    r4, k4, v4 = (t.reshape(B, T, num_heads, N) for t in (receptance, replacement_key, value))
    bonus4 = (r4 * k4 * bonus.reshape(1, 1, num_heads, N)).sum(3, keepdim=True) * v4
    return (norm + bonus4.reshape(B, T, C)) * gate


def channel_mixer_reference(x, key_scale, key_weight, value_weight):
    """``channel_mixer_reference`` (``kernels/train/channel_mixer/mod.rs:96-128``), op for op."""
    B, T, C = x.shape
    shifted = torch.cat([torch.zeros(B, 1, C, dtype=x.dtype), x[:, :T - 1]], 1) if T > 0 else x
    key_input = x + (shifted - x) * key_scale.reshape(1, 1, C)
    activated = torch.relu(key_input.reshape(B * T, C) @ key_weight.T).pow(2.0)
    return (activated @ value_weight.T).reshape(B, T, C)
