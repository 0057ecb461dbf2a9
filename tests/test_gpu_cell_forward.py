"""The callers either side of the hot path: one stack of RWKV-7 cells run through the library
(`cell_forward.prefill_forward`) against a restatement that takes every hot-path operator from
the CPU oracle and everything else (layer norms, projections, LoRAs, residuals) from fp64 torch.

Both sides store bf16 between operators (the restatement rounds at the same points), so what
remains is the rounding inside the operators: the cell output must agree to 3e-2 of its largest
magnitude with cosine >= 0.9995, the mean loss to 2e-3."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _bf(x):   # numpy/torch fp64 -> rounded to bf16, back as fp64 torch
    t = torch.as_tensor(np.asarray(x), dtype=torch.float64) if not torch.is_tensor(x) else x
    return t.to(torch.bfloat16).double()


def _d(t):
    return None if t is None else t.detach().cpu().double()


def _lora(x, w, act=None):
    h = _bf(x @ _d(w[0]))
    if act is not None:
        h = _bf(act(h))
    y = h @ _d(w[1])
    return _bf(y if w[2] is None else y + _d(w[2]))   # the bias is added inside the product


def _cell_restated(oracle, w, x, v_first, cell_id, H):
    B, T, C = x.shape
    N = C // H
    xn = _bf(F.layer_norm(x, (C,), _d(w.ln1[0]), _d(w.ln1[1])))
    m = _bf(oracle.mix6(xn.numpy(), [_d(s).numpy() for s in w.mix6_scales]))   # [6,B,T,C]
    xr, xw, xk, xv, xa, xg = (m[i] for i in range(6))
    receptance = _bf(xr @ _d(w.w_receptance).t())
    key_precursor = _bf(xk @ _d(w.w_key).t())
    value_precursor = _bf(xv @ _d(w.w_value).t())
    lr = _lora(xa, w.lora_learning_rate)
    wd = _lora(xw, w.lora_weight_decay, torch.tanh)
    args = [t.numpy() for t in (key_precursor, lr, wd, _d(w.key_removal), _d(w.key_replacement))]
    if cell_id == 0:
        v_first = value_precursor
        wp = oracle.weight_prepare(*args, H)
        value = value_precursor
    else:
        nu = _lora(xv, w.lora_value_residual)
        wp = oracle.weight_prepare(*args, H, value_precursor.numpy(), v_first.numpy(), nu.numpy())
        value = _bf(wp["value"])
    wp = {k: _bf(v) for k, v in wp.items() if v is not None}
    gate = _lora(xg, w.lora_gate, torch.sigmoid)
    s4 = (B, T, H, N)
    y, _ = oracle.wkv7(*[t.reshape(s4).numpy() for t in (receptance, wp["weight_decay"], wp["replacement_key"], value,
                                                          wp["removal_key_normalized"], wp["replacement"])],
                       None, precision="f64", want_state=True)
    y = _bf(y).reshape(B, T, C)
    out = _bf(oracle.gated_readout(*[t.numpy() for t in (y, receptance, wp["replacement_key"], value, gate,
                                                         _d(w.group_norm[0]), _d(w.group_norm[1]),
                                                         _d(w.receptance_key_bonus))], H))
    x = _bf(x + out @ _d(w.w_output).t())   # the residual is added inside the projection
    xn = _bf(F.layer_norm(x, (C,), _d(w.ln2[0]), _d(w.ln2[1])))
    cm = _bf(oracle.channel_mixer(xn.numpy(), _d(w.cm_key_scale).numpy(), _d(w.cm_key_weight).numpy(),
                                  _d(w.cm_value_weight).numpy()))
    return _bf(x + cm), v_first


def test_two_cells_and_lm_head_against_restatement(pkg, oracle, cuda):
    from rwkv_rs_stable_b200 import cell_forward as cf
    B, T, C, H, Fd, V = 2, 64, 128, 2, 256, 512
    # weights large enough that every branch matters at this small width
    cells = [cf.random_cell(i, C, H, Fd, device=cuda, seed=3, std=0.08) for i in range(2)]
    g = torch.Generator(device=cuda)
    g.manual_seed(5)
    emb = torch.randn((V, C), generator=g, device=cuda).to(torch.bfloat16)
    head = (torch.randn((V, C), generator=g, device=cuda) * 0.08).to(torch.bfloat16)
    ids = torch.randint(0, V, (B, T), generator=g, device=cuda)
    ones, zeros = torch.ones(C, device=cuda, dtype=torch.bfloat16), torch.zeros(C, device=cuda, dtype=torch.bfloat16)

    x = emb[ids]
    v_first = None
    for i, w in enumerate(cells):
        x, v_first = cf.cell_forward(pkg, w, x, v_first, i, H)
    loss = cf.prefill_forward(pkg, cells, emb, head, (ones, zeros), ids, H)
    torch.cuda.synchronize()
    assert pkg.read_device_status(0) == 0

    xr = _d(emb)[ids.cpu()]
    vr = None
    for i, w in enumerate(cells):
        xr, vr = _cell_restated(oracle, w, xr, vr, i, H)
    got = x.double().cpu()
    err = float((got - xr).abs().max() / xr.abs().max())
    cos = float((got * xr).sum() / (got.norm() * xr.norm()))
    assert err <= 3e-2 and cos >= 0.9995, (err, cos)

    xf = _bf(F.layer_norm(xr, (C,), _d(ones), _d(zeros))).reshape(B * T, C)
    targets = torch.cat([ids[:, 1:], ids[:, -1:]], dim=1).reshape(-1).cpu().numpy()
    _, loss_ref = oracle.lm_head_ce(xf.numpy(), _d(head).numpy(), targets)
    assert abs(float(loss.item()) - float(loss_ref.mean())) <= 2e-3 * float(loss_ref.mean())
