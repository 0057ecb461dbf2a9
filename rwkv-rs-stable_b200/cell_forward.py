"""The prefill forward of a stack of RWKV-7 cells as the call sequence a drop-in user gets.

Measurement harness for the whole-model prefill configuration (random-init weights,
uniform-random token ids, fused LM-head cross entropy on the shifted targets): every
operator of the hot path runs through this library's C ABI, and everything around
it is the plain library call the reference makes there as well — the dense
projections and the LoRA products are matmuls (``torch`` → cuBLAS), layer norms and
residual additions are ``torch`` ops.

Call order followed (paths inside the rwkv-rs repository):

* ``CausalCell::forward`` — ``crates/rwkv-nn/src/cells/causal.rs:213-248``: layer norm,
  time mixer, residual, layer norm, channel mixer, residual;
* ``TimeMixer::forward`` — ``crates/rwkv-nn/src/modules/time_mixer/mod.rs:157-215``:
  mix6, ``WeightPrepare::forward``, WKV7 (pretrain: zero initial state), ``GatedReadout::forward``;
* ``WeightPrepare::forward`` — ``modules/time_mixer/weight_prepare.rs:231-298``: three dense
  projections, the learning-rate / weight-decay / value-residual LoRAs
  (``layers/lora.rs:105-124``), then the tail that ``rwkv7_fused_weight_prepare`` computes;
* ``GatedReadout::forward`` — ``modules/time_mixer/gated_readout.rs:109-145``: gate LoRA
  (sigmoid inside), the body that ``rwkv7_fused_gated_readout`` computes, output projection;
* ``ChannelMixer::forward`` through ``rwkv7_fused_channel_mixer``.

Nothing here is on the product's hot path itself and nothing here is a CPU fallback:
without the CUDA library the operator calls raise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

# LoRA ranks of the 1.5B-class RWKV-7 models (decay, in-context learning rate, value residual, gate).
LORA_RANKS = {"weight_decay": 96, "learning_rate": 96, "value_residual": 64, "gate": 256}


@dataclass
class CellWeights:
    ln1: tuple
    ln2: tuple
    mix6_scales: list            # six [1,1,C]: receptance, weight_decay, key, value, learning_rate, gate
    w_receptance: torch.Tensor   # [C,C] (out, in)
    w_key: torch.Tensor
    w_value: torch.Tensor
    w_output: torch.Tensor
    lora_weight_decay: tuple     # (w_a [C,r], w_b [r,C], bias [C])
    lora_learning_rate: tuple
    lora_value_residual: Optional[tuple]
    lora_gate: tuple             # (w_a, w_b, None)
    key_removal: torch.Tensor    # [1,1,C]
    key_replacement: torch.Tensor
    group_norm: tuple            # gamma [C], beta [C]
    receptance_key_bonus: torch.Tensor   # [H,N]
    cm_key_scale: torch.Tensor   # [C]
    cm_key_weight: torch.Tensor  # [F,C]
    cm_value_weight: torch.Tensor  # [C,F]


def decay_speed_bias(num_cells: int, C: int, head_size: int, cell_id: int) -> torch.Tensor:
    """The reference's initial bias of the weight-decay LoRA (``calculate_decay_speed``,
    ``functions/init_weights.rs:54-75``, applied in ``layers/lora.rs:73-84``): per channel
    ``-6 + 6 (n/(C-1))^(1 + layer_ratio^0.3) + 0.5 + 2.5 z|z|`` with ``z`` running from -1 to 1 inside every head.
    It spreads the per-token decay ``exp(-exp(-softplus(-bias) - 0.5))`` from 0.998 (first channels) to the
    strongest value the model allows, 0.55 (last channels of the later heads)."""
    layer_ratio = cell_id / (num_cells - 1) if num_cells > 1 else 0.0
    n = torch.arange(C, dtype=torch.float64)
    base = -6.0 + 6.0 * (n / max(C - 1, 1)) ** (1.0 + layer_ratio ** 0.3)
    half = (head_size - 1.0) / 2.0
    z = ((n % head_size) - half) / max(half, 1.0)
    return (base + 0.5 + 2.5 * z * z.abs()).to(torch.float32)


def random_cell(cell_id: int, C: int, H: int, Fdim: int, *, device, seed: int = 0, std: float = 0.02,
                num_cells: int = 1) -> CellWeights:
    """bf16 weights ``N(0, std)``; norm scales 1, biases 0; the two key parameters at their
    initial values 0.71 / 1.02 (``weight_prepare.rs:200-201``); the weight-decay LoRA's bias at the
    reference's initial decay speeds (:func:`decay_speed_bias`)."""
    g = torch.Generator(device=device)
    g.manual_seed(7 * 1000003 + 131 * seed + cell_id)
    bf = torch.bfloat16

    def mat(*shape, s=std):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * s).to(bf)

    def lora(rank, bias=True):
        return (mat(C, rank), mat(rank, C), torch.zeros(C, device=device, dtype=bf) if bias else None)

    ones = torch.ones(C, device=device, dtype=bf)
    zeros = torch.zeros(C, device=device, dtype=bf)
    N = C // H
    return CellWeights(
        ln1=(ones.clone(), zeros.clone()), ln2=(ones.clone(), zeros.clone()),
        mix6_scales=[torch.rand((1, 1, C), generator=g, device=device, dtype=torch.float32).to(bf) for _ in range(6)],
        w_receptance=mat(C, C), w_key=mat(C, C), w_value=mat(C, C), w_output=mat(C, C),
        lora_weight_decay=lora(LORA_RANKS["weight_decay"])[:2] + (decay_speed_bias(num_cells, C, N, cell_id).to(device).to(bf),),
        lora_learning_rate=lora(LORA_RANKS["learning_rate"]),
        lora_value_residual=lora(LORA_RANKS["value_residual"]) if cell_id > 0 else None,
        lora_gate=lora(LORA_RANKS["gate"], bias=False),
        key_removal=torch.full((1, 1, C), 0.71, device=device, dtype=bf),
        key_replacement=torch.full((1, 1, C), 1.02, device=device, dtype=bf),
        group_norm=(ones.clone(), zeros.clone()),
        receptance_key_bonus=mat(H, N),
        cm_key_scale=torch.rand((C,), generator=g, device=device, dtype=torch.float32).to(bf),
        cm_key_weight=mat(Fdim, C), cm_value_weight=mat(C, Fdim))


def _lora(x: torch.Tensor, w, act=None) -> torch.Tensor:
    h = x @ w[0]
    if act is not None:
        h = act(h)
    if w[2] is None:
        return h @ w[1]
    # bias + h w_b in one library call (the bias enters the product's epilogue)
    return torch.addmm(w[2], h.reshape(-1, h.shape[-1]), w[1]).view(*h.shape[:-1], w[1].shape[1])


def cell_forward(pkg, w: CellWeights, x: torch.Tensor, value_from_first_cell: Optional[torch.Tensor],
                 cell_id: int, H: int, cm_workspace: Optional[torch.Tensor] = None):
    """One cell on ``x [B,T,C]`` bf16.  Returns ``(x_out, value_from_first_cell)``."""
    B, T, C = x.shape
    N = C // H
    xn = F.layer_norm(x, (C,), w.ln1[0], w.ln1[1])
    m = pkg.mix6_custom(xn, *w.mix6_scales)
    del xn
    receptance = m["receptance_input"] @ w.w_receptance.t()
    key_precursor = m["key_input"] @ w.w_key.t()
    value_precursor = m["value_input"] @ w.w_value.t()
    lr = _lora(m["learning_rate_input"], w.lora_learning_rate)
    wd = _lora(m["weight_decay_input"], w.lora_weight_decay, torch.tanh)
    if cell_id == 0:
        value_from_first_cell = value_precursor
        wp = pkg.weight_prepare_epilogue(key_precursor, lr, wd, w.key_removal, w.key_replacement, H)
        value = value_precursor
    else:
        nu = _lora(m["value_input"], w.lora_value_residual)
        wp = pkg.weight_prepare_epilogue(key_precursor, lr, wd, w.key_removal, w.key_replacement, H,
                                         value_precursor=value_precursor,
                                         value_from_first_cell=value_from_first_cell, value_residual_lora=nu)
        value = wp.value
        del nu
    gate = _lora(m["gate_input"], w.lora_gate, torch.sigmoid)
    del m, lr, wd, key_precursor
    shape = (B, T, H, N)
    seq = pkg.Wkv7PretrainForwardInputs(receptance.view(shape), wp.weight_decay.view(shape),
                                        wp.replacement_key.view(shape), value.view(shape),
                                        wp.removal_key_normalized.view(shape), wp.replacement.view(shape))
    y = pkg.wkv7_pretrain_custom(seq)
    out = pkg.gated_readout_epilogue(y.view(B, T, C), receptance, wp.replacement_key, value, gate,
                                     w.group_norm[0], w.group_norm[1], w.receptance_key_bonus, H)
    del y, gate, wp, seq, receptance
    x = torch.addmm(x.view(-1, C), out.view(-1, C), w.w_output.t()).view(B, T, C)   # residual inside the projection
    del out
    xn = F.layer_norm(x, (C,), w.ln2[0], w.ln2[1])
    x = x + pkg.channel_mixer_custom(xn, w.cm_key_scale, w.cm_key_weight, w.cm_value_weight, workspace=cm_workspace)
    return x, value_from_first_cell


def prefill_forward(pkg, cells, embedding: torch.Tensor, head: torch.Tensor, final_ln, ids: torch.Tensor, H: int,
                    cm_workspace: Optional[torch.Tensor] = None):
    """Embedding, every cell, final layer norm and the fused LM-head cross entropy on the
    targets ``ids`` shifted left by one (the last position of each sequence is given its own
    id as target, so that every row has one).  Returns the mean loss (a 0-d tensor)."""
    B, T = ids.shape
    x = embedding[ids]
    v_first = None
    for i, w in enumerate(cells):
        x, v_first = cell_forward(pkg, w, x, v_first, i, H, cm_workspace)
    x = F.layer_norm(x, (x.shape[-1],), final_ln[0], final_ln[1])
    targets = torch.cat([ids[:, 1:], ids[:, -1:]], dim=1).reshape(-1)
    _, loss = pkg.lm_head_ce(x.view(B * T, -1), head, targets)
    return loss.mean()
