"""The CUDA kernels against the committed golden fixtures of the operators other than the WKV7
forward (whose fixtures are checked in test_gpu_wkv7.py): nothing here needs the oracle at run time."""
import os

import numpy as np
import pytest
import torch

import parity

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def _t(a, cuda, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).to(cuda)


def test_mix_ops_golden(pkg, cuda):
    g = _load("mix_ops.npz")
    x, diff = _t(g["x"], cuda), _t(g["diff"], cuda)
    mus = [_t(m, cuda) for m in g["mus"]]
    out = pkg.mix6_custom(x, *mus)
    for i, name in enumerate(pkg.MIX6_BRANCHES):
        np.testing.assert_allclose(out[name].cpu().numpy(), g["mix6"][i], rtol=1e-6, atol=1e-6)
    five = pkg.addcmul5_custom(x, diff, *mus[:5])
    for i, name in enumerate(pkg.MIX6_BRANCHES[:5]):
        np.testing.assert_allclose(five[name].cpu().numpy(), g["addcmul5"][i], rtol=1e-6, atol=1e-6)
    state = _t(g["state"], cuda)
    res = pkg.token_shift_diff_custom(x, state, torch.from_numpy(g["ids"]).to(cuda), inplace_state=True)
    torch.cuda.synchronize()
    assert np.array_equal(res.token_shifted_diff.cpu().numpy(), g["tsd"])
    assert np.array_equal(state.cpu().numpy(), g["tsd_state"])


def test_time_mixer_epilogues_golden(pkg, cuda):
    g = _load("time_mixer_epilogues.npz")
    e = {k[3:]: _t(v, cuda) for k, v in g.items() if k.startswith("in_")}
    out = pkg.weight_prepare_epilogue(e["key_precursor"], e["learning_rate_lora"], e["weight_decay_lora"],
                                      e["key_removal"], e["key_replacement"], 2,
                                      value_precursor=e["value_precursor"],
                                      value_from_first_cell=e["value_from_first_cell"],
                                      value_residual_lora=e["value_residual_lora"])
    for name in ("weight_decay", "replacement_key", "removal_key_normalized", "replacement", "value"):
        parity.assert_close_f32(getattr(out, name).cpu().numpy(), g["wp_" + name], 2e-5, name)
    gr = pkg.gated_readout_epilogue(e["wkv7_output"], e["receptance"], e["replacement_key"], e["value"], e["gate"],
                                    e["group_norm_gamma"], e["group_norm_beta"], e["receptance_key_bonus"], 2)
    parity.assert_close_f32(gr.cpu().numpy(), g["gated_readout"], 2e-5, "gated_readout")


def test_channel_mixer_golden(pkg, cuda):
    g = _load("channel_mixer.npz")       # the fixture's inputs are bf16-representable
    out = pkg.channel_mixer_custom(*[_t(g[k], cuda, torch.bfloat16) for k in ("x", "key_scale", "key_weight", "value_weight")])
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    assert np.abs(got - g["out"]).max() <= 2e-2 * np.abs(g["out"]).max()


@pytest.mark.parametrize("name", ["wkv7_train_ref_shape.npz", "wkv7_train_n64.npz"])
def test_training_golden(pkg, cuda, name):
    g = _load(name)
    six = [_t(g[n], cuda) for n in "rwkvab"]
    s0 = _t(g["s0"], cuda)
    inputs = pkg.Wkv7PretrainForwardInputs(*six)
    saved = pkg.wkv7_forward_saved(inputs, s0, want_state=True)
    grads, ds0 = pkg.wkv7_backward(inputs, saved, _t(g["dy"], cuda), _t(g["ds"], cuda), initial_state=s0)
    torch.cuda.synchronize()
    parity.assert_close_f32(saved.output.cpu().numpy(), g["y"], 2e-5, "y")
    parity.assert_close_f32(saved.snapshots.cpu().numpy(), g["snapshots"], 2e-5, "snapshots")
    parity.assert_close_f32(saved.state_replacement.cpu().numpy(), g["state_replacement"], 2e-5, "state_replacement")
    for n, got in zip("rwkvab", grads):
        parity.assert_close_f32(got.cpu().numpy(), g["d" + n], 2e-4, "d" + n)
    parity.assert_close_f32(ds0.cpu().numpy(), g["ds0"], 2e-4, "ds0")
