"""CPU tests of the oracle: against the committed golden fixtures, against an
independent torch fp64 restatement of the reference's tensor-op code, and against
closed-form known answers.  (The reference has no golden vectors of its own.)"""
import os

import numpy as np
import pytest
import torch

import torch_restatement as tr

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


@pytest.mark.parametrize("name", ["wkv7_cfg0.npz", "wkv7_ref_test_shape.npz", "wkv7_bf16_t40.npz"])
def test_oracle_reproduces_golden(oracle, name):
    g = _load(name)
    y, s = oracle.wkv7(g["r"], g["w"], g["k"], g["v"], g["a"], g["b"], g.get("s0"))
    np.testing.assert_allclose(y, g["y"], rtol=0, atol=2e-6 * np.abs(g["y"]).max())
    np.testing.assert_allclose(s, g["s_out"], rtol=0, atol=2e-6 * np.abs(g["s_out"]).max())


@pytest.mark.parametrize("shape,with_state", [((2, 16, 2, 8), True), ((1, 16, 1, 4), False),
                                              ((1, 24, 2, 8), False), ((2, 5, 3, 16), True)])
def test_oracle_matches_torch_restatement(oracle, workloads, shape, with_state):
    B, T, H, N = shape
    six = workloads.uniform_inputs(shape, seed=5)
    s0 = workloads.uniform_inputs((B, H, N, N), seed=6, n=1)[0] if with_state else None
    y_t, s_t = tr.wkv7_reference_with_state(*six, s0)
    y, s = oracle.wkv7(*[t.numpy() for t in six], None if s0 is None else s0.numpy())
    np.testing.assert_allclose(y, y_t.numpy(), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(s, s_t.numpy(), rtol=1e-12, atol=1e-12)
    # the f32 variant follows the reference kernel's accumulation order; the
    # reference's own tolerance between its two paths is abs 1e-2 (wkv7/mod.rs:400-408)
    y32, s32 = oracle.wkv7(*[t.numpy() for t in six], None if s0 is None else s0.numpy(), precision="f32")
    assert np.abs(y32 - y).max() <= 1e-4 * max(1.0, np.abs(y).max())
    assert np.abs(s32 - s).max() <= 1e-4 * max(1.0, np.abs(s).max())


def test_oracle_benchmark_distribution(oracle, workloads):
    inp = workloads.wkv7_inputs(1, 32, 2, 64, seed=9, state="normal")
    y_t, s_t = tr.wkv7_reference_with_state(inp["r"], inp["w"], inp["k"], inp["v"], inp["a"], inp["b"], inp["s0"])
    f = {k: v.numpy() for k, v in inp.items()}
    y, s = oracle.wkv7(f["r"], f["w"], f["k"], f["v"], f["a"], f["b"], f["s0"])
    np.testing.assert_allclose(y, y_t.numpy(), rtol=1e-11, atol=1e-11)
    np.testing.assert_allclose(s, s_t.numpy(), rtol=1e-11, atol=1e-11)


def test_oracle_known_answer_no_removal(oracle):
    """With a = b = 0 the recurrence is S_t = S_{t-1} diag(d) + v k^T, so
    S_T[i][j] = sum_t v_t[i] k_t[j] d_j^(T-1-t) for a constant decay."""
    rng = np.random.default_rng(3)
    B, T, H, N = 1, 7, 1, 4
    r, k, v = (rng.standard_normal((B, T, H, N)).astype(np.float32) for _ in range(3))
    wj = rng.uniform(-3, -0.5, size=N).astype(np.float32)
    w = np.broadcast_to(wj, (B, T, H, N)).copy()
    z = np.zeros((B, T, H, N), np.float32)
    y, s = oracle.wkv7(r, w, k, v, z, z, None)
    d = np.exp(-np.exp(wj.astype(np.float64)))
    S = np.zeros((N, N))
    for t in range(T):
        S += np.outer(v[0, t, 0].astype(np.float64), k[0, t, 0].astype(np.float64)) * d[None, :] ** (T - 1 - t)
    np.testing.assert_allclose(s[0, 0], S, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(y[0, T - 1, 0], S @ r[0, T - 1, 0].astype(np.float64), rtol=1e-12, atol=1e-12)


def test_oracle_known_answer_scalar_head(oracle):
    """N = 1: s_t = s_{t-1} (d_t + a_t b_t) + v_t k_t and y_t = s_t r_t."""
    rng = np.random.default_rng(4)
    T = 9
    x = [rng.uniform(0, 1, size=(1, T, 1, 1)).astype(np.float32) for _ in range(6)]
    s0 = np.array([[[[0.3]]]], np.float32)
    y, s = oracle.wkv7(*x, s0)
    r, w, k, v, a, b = (t.astype(np.float64).ravel() for t in x)
    st = 0.3 if False else float(np.float32(0.3))
    for t in range(T):
        st = st * (np.exp(-np.exp(w[t])) + a[t] * b[t]) + v[t] * k[t]
        assert abs(y.ravel()[t] - st * r[t]) < 1e-12
    assert abs(s.ravel()[0] - st) < 1e-12


def test_oracle_state_carry(oracle, workloads):
    """statepass(T1) then statepass(T2) equals statepass(T1 + T2)."""
    inp = workloads.wkv7_inputs(1, 48, 2, 16, seed=2)
    f = [inp[n].numpy() for n in "rwkvab"]
    y, s = oracle.wkv7(*f, None)
    y1, s1 = oracle.wkv7(*[t[:, :20] for t in f], None)
    y2, s2 = oracle.wkv7(*[t[:, 20:] for t in f], s1)
    np.testing.assert_allclose(np.concatenate([y1, y2], 1), y, rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(s2, s, rtol=1e-13, atol=1e-13)


@pytest.mark.parametrize("shape", [(2, 8, 32), (1, 3, 17), (2, 1, 8)])
def test_oracle_mix6(oracle, workloads, shape):
    x, mus = workloads.mix_inputs(*shape, seed=1)
    ref = tr.mix6_reference(x, mus)
    out = oracle.mix6(x.numpy(), [m.numpy() for m in mus])
    for i in range(6):
        np.testing.assert_allclose(out[i], ref[i].numpy(), rtol=1e-14, atol=1e-14)


@pytest.mark.parametrize("n", [1, 5])
def test_oracle_addcmul(oracle, workloads, n):
    base, mus = workloads.mix_inputs(2, 8, 32, seed=2, nscale=n)
    diff, _ = workloads.mix_inputs(2, 8, 32, seed=3, nscale=1)
    out = oracle.addcmul(base.numpy(), diff.numpy(), [m.numpy() for m in mus])
    for i in range(n):
        np.testing.assert_allclose(out[i], tr.addcmul_reference(base, diff, mus[i]).numpy(), rtol=1e-14, atol=0)


@pytest.mark.parametrize("B,T,C,S,ids", [(1, 1, 8, 1, [0]), (1, 4, 8, 3, [2]), (3, 5, 16, 8, [6, 1, 4]),
                                         (2, 0, 8, 4, [3, 1])])
def test_oracle_token_shift_diff(oracle, B, T, C, S, ids):
    """The reference's own cases (token_shift_diff/mod.rs:222-227), T == 0 included."""
    g = torch.Generator().manual_seed(5)
    x = torch.rand((B, T, C), generator=g)
    state = torch.rand((S, C), generator=g)
    idt = torch.tensor(ids, dtype=torch.int64)
    d_ref, s_ref = tr.token_shift_diff_reference(x, state, idt)
    d, s = oracle.token_shift_diff(x.numpy(), state.numpy(), idt.numpy())
    assert d.shape == tuple(d_ref.shape)
    if T:
        np.testing.assert_array_equal(d, d_ref.numpy())
    np.testing.assert_array_equal(s, s_ref.numpy())


def test_oracle_lm_head_ce(oracle, workloads):
    x, w, tg = workloads.lm_head_inputs(12, 64, 96, seed=0)
    tg[3] = -1  # ignored row
    lse, loss = oracle.lm_head_ce(x.float().numpy(), w.float().numpy(), tg.numpy())
    z = x.double() @ w.double().T
    np.testing.assert_allclose(lse, torch.logsumexp(z, dim=1).numpy(), rtol=1e-12)
    ce = torch.nn.functional.cross_entropy(z, tg.clamp_min(0), reduction="none")
    ce[3] = 0
    np.testing.assert_allclose(loss, ce.numpy(), rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("shape", [(2, 5, 3, 64), (1, 4, 2, 20), (3, 2, 1, 7)])
def test_time_mixer_epilogues_match_torch_restatement(oracle, workloads, shape):
    """The C restatements of the WeightPrepare tail and of GatedReadout against independent
    torch fp64 versions written with the reference's tensor ops (torch's own softplus,
    GroupNorm and clamp_min)."""
    import torch_restatement as tr
    B, T, H, N = shape
    inp = workloads.time_mixer_epilogue_inputs(B, T, H, N, seed=4)
    d = {k: v.double() for k, v in inp.items()}
    ref = tr.weight_prepare_reference(d["key_precursor"], d["learning_rate_lora"], d["weight_decay_lora"],
                                      d["key_removal"], d["key_replacement"], H, d["value_precursor"],
                                      d["value_from_first_cell"], d["value_residual_lora"])
    got = oracle.weight_prepare(inp["key_precursor"].numpy(), inp["learning_rate_lora"].numpy(),
                                inp["weight_decay_lora"].numpy(), inp["key_removal"].numpy(),
                                inp["key_replacement"].numpy(), H, inp["value_precursor"].numpy(),
                                inp["value_from_first_cell"].numpy(), inp["value_residual_lora"].numpy())
    for name, r in ref.items():
        np.testing.assert_allclose(got[name], r.numpy(), rtol=1e-12, atol=1e-12, err_msg=name)
    first = oracle.weight_prepare(inp["key_precursor"].numpy(), inp["learning_rate_lora"].numpy(),
                                  inp["weight_decay_lora"].numpy(), inp["key_removal"].numpy(),
                                  inp["key_replacement"].numpy(), H)
    assert first["value"] is None and np.array_equal(first["replacement"], got["replacement"])
    # known answers: unit norm per head, b = -a * lr, decay precursor below -0.5
    a = got["removal_key_normalized"].reshape(B, T, H, N)
    np.testing.assert_allclose((a * a).sum(-1), 1.0, rtol=1e-12)
    assert (got["weight_decay"] < -0.5).all()

    ref = tr.gated_readout_reference(d["wkv7_output"], d["receptance"], d["replacement_key"], d["value"],
                                     d["gate"], d["group_norm_gamma"], d["group_norm_beta"],
                                     d["receptance_key_bonus"], H)
    got = oracle.gated_readout(*[inp[n].numpy() for n in ("wkv7_output", "receptance", "replacement_key", "value",
                                                          "gate", "group_norm_gamma", "group_norm_beta",
                                                          "receptance_key_bonus")], H)
    np.testing.assert_allclose(got, ref.numpy(), rtol=1e-11, atol=1e-11)


def test_weight_prepare_zero_key_uses_the_epsilon(oracle):
    """normalize.rs:38-40 clamps the norm at 1e-12: an all-zero head gives zeros, not NaN."""
    z = np.zeros((1, 1, 8), dtype=np.float32)
    one = np.ones((1, 1, 8), dtype=np.float32)
    got = oracle.weight_prepare(z, z, z, one, one, 2)
    assert np.array_equal(got["removal_key_normalized"], np.zeros_like(z, dtype=np.float64))
    np.testing.assert_allclose(got["weight_decay"], -np.log(2.0) - 0.5)


@pytest.mark.parametrize("shape", [(2, 5, 16, 40), (1, 1, 8, 8), (3, 4, 24, 64)])
def test_channel_mixer_matches_torch_restatement(oracle, workloads, shape):
    """channel_mixer/mod.rs:204-232 compares the custom path with channel_mixer_reference; here
    the C restatement against the same tensor ops in torch fp64."""
    import torch_restatement as tr
    x, ks, kw, vw = workloads.channel_mixer_inputs(*shape, seed=2, dtype=torch.float32)
    ref = tr.channel_mixer_reference(x.double(), ks.double(), kw.double(), vw.double())
    got = oracle.channel_mixer(x.numpy(), ks.numpy(), kw.numpy(), vw.numpy())
    np.testing.assert_allclose(got, ref.numpy(), rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("shape,with_state", [((1, 16, 1, 4), False), ((2, 32, 2, 8), True), ((1, 48, 1, 16), True)])
def test_wkv7_backward_matches_torch_autograd(oracle, workloads, shape, with_state):
    """wkv7/mod.rs:294-328 differentiates sum(y) through the tensor-op reference with Burn's autodiff;
    here the C reverse pass against torch autograd through the fp64 torch restatement, with a random
    output gradient and a gradient on the final state as well."""
    inp = workloads.wkv7_inputs(*shape, seed=21, state="normal" if with_state else None)
    B, T, H, N = shape
    g = torch.Generator().manual_seed(5)
    dy = torch.randn(B, T, H, N, generator=g, dtype=torch.float64)
    ds = torch.randn(B, H, N, N, generator=g, dtype=torch.float64)
    leaves = {n: inp[n].double().requires_grad_(True) for n in "rwkvab"}
    s0 = inp["s0"].double().requires_grad_(True) if with_state else torch.zeros(B, H, N, N, dtype=torch.float64)
    y, s_out = tr.wkv7_reference_with_state(*[leaves[n] for n in "rwkvab"], s0)
    ((y * dy).sum() + (s_out * ds).sum()).backward()
    f = {n: inp[n].numpy() for n in "rwkvab"}
    got = oracle.wkv7_backward(*[f[n] for n in "rwkvab"], dy.numpy(), s0=inp["s0"].numpy() if with_state else None,
                               ds_out=ds.numpy())
    for n in "rwkvab":
        np.testing.assert_allclose(got[n], leaves[n].grad.numpy(), rtol=1e-9, atol=1e-9, err_msg=n)
    if with_state:
        np.testing.assert_allclose(got["s0"], s0.grad.numpy(), rtol=1e-9, atol=1e-9)


def test_wkv7_train_forward_saves(oracle, workloads):
    """snapshots hold the state after tokens 15, 31, ...; state_replacement is S_{t-1} a_t."""
    inp = workloads.wkv7_inputs(2, 32, 2, 8, seed=22, state="normal")
    f = {n: inp[n].numpy() for n in inp}
    y, s_out, snaps, sa = oracle.wkv7_train(*[f[n] for n in "rwkvab"], s0=f["s0"], chunk_len=16)
    y_ref, s_ref = oracle.wkv7(*[f[n] for n in "rwkvab"], f["s0"], precision="f64")
    np.testing.assert_allclose(y, y_ref, rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(snaps[:, :, 1], s_ref, rtol=1e-13, atol=1e-13)
    _, s_half = oracle.wkv7(*[f[n][:, :16] for n in "rwkvab"], f["s0"], precision="f64")
    np.testing.assert_allclose(snaps[:, :, 0], s_half, rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(sa[:, 0], np.einsum("bhij,bhj->bhi", f["s0"].astype(np.float64),
                                                   f["a"][:, 0].astype(np.float64)), rtol=1e-13, atol=1e-13)


def test_oracle_reproduces_golden_of_the_other_operators(oracle):
    """The committed fixtures of mix6 / addcmul5 / token_shift_diff, the two time-mixer epilogues,
    the channel mixer and the training path: drift of the oracle shows up here, on CPU."""
    g = _load("mix_ops.npz")
    mus = [m for m in g["mus"]]
    np.testing.assert_allclose(oracle.mix6(g["x"], mus), g["mix6"], rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(oracle.addcmul(g["x"], g["diff"], mus[:5]), g["addcmul5"], rtol=1e-13, atol=1e-13)
    tsd, st = oracle.token_shift_diff(g["x"], g["state"], g["ids"])
    assert np.array_equal(tsd, g["tsd"]) and np.array_equal(st, g["tsd_state"])
    g = _load("time_mixer_epilogues.npz")
    e = {k[3:]: v for k, v in g.items() if k.startswith("in_")}
    wp = oracle.weight_prepare(e["key_precursor"], e["learning_rate_lora"], e["weight_decay_lora"], e["key_removal"],
                               e["key_replacement"], 2, e["value_precursor"], e["value_from_first_cell"],
                               e["value_residual_lora"])
    for k, v in wp.items():
        np.testing.assert_allclose(v, g["wp_" + k], rtol=1e-13, atol=1e-13, err_msg=k)
    gr = oracle.gated_readout(e["wkv7_output"], e["receptance"], e["replacement_key"], e["value"], e["gate"],
                              e["group_norm_gamma"], e["group_norm_beta"], e["receptance_key_bonus"], 2)
    np.testing.assert_allclose(gr, g["gated_readout"], rtol=1e-13, atol=1e-13)
    g = _load("channel_mixer.npz")
    np.testing.assert_allclose(oracle.channel_mixer(g["x"], g["key_scale"], g["key_weight"], g["value_weight"]),
                               g["out"], rtol=1e-13, atol=1e-13)
    for name in ("wkv7_train_ref_shape.npz", "wkv7_train_n64.npz"):
        g = _load(name)
        y, s_out, snaps, sa = oracle.wkv7_train(*[g[n] for n in "rwkvab"], s0=g["s0"], chunk_len=16)
        for got, key in ((y, "y"), (s_out, "s_out"), (snaps, "snapshots"), (sa, "state_replacement")):
            np.testing.assert_allclose(got, g[key], rtol=1e-12, atol=1e-12, err_msg=key)
        grads = oracle.wkv7_backward(*[g[n] for n in "rwkvab"], g["dy"], s0=g["s0"], ds_out=g["ds"])
        for k, v in grads.items():
            np.testing.assert_allclose(v, g["d" + k], rtol=1e-11, atol=1e-11, err_msg="d" + k)
