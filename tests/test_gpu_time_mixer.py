"""GPU parity of the two time-mixer epilogues (the tail of WeightPrepare::forward and
the body of GatedReadout::forward) against the fp64 CPU oracle, through the C ABI.

Tolerance: the kernels compute in fp32 and round once, so fp32 outputs must agree to
2e-5 of the tensor's largest magnitude (fast `exp`, `rsqrt`) and bf16 outputs to one bf16
spacing of the value plus the same fp32 term."""
import numpy as np
import pytest
import torch

import parity

pytestmark = pytest.mark.gpu

WP_IN = ("key_precursor", "learning_rate_lora", "weight_decay_lora", "key_removal", "key_replacement")
WP_VAL = ("value_precursor", "value_from_first_cell", "value_residual_lora")
GR_IN = ("wkv7_output", "receptance", "replacement_key", "value", "gate", "group_norm_gamma", "group_norm_beta",
         "receptance_key_bonus")


def _close(x, ref, dtype, what):
    x = x.float().cpu().numpy().astype(np.float64)
    tol = 2e-5 * max(np.abs(ref).max(), 1e-30)
    if dtype == torch.bfloat16:
        tol = tol + parity.BF16_ULP * np.abs(ref)
    bad = np.abs(x - ref) > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} elements off, worst {np.abs(x - ref).max():.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 8, 2, 64), (1, 3, 5, 64), (2, 7, 3, 20), (1, 5, 2, 7), (2, 512, 12, 64)])
def test_weight_prepare(pkg, oracle, workloads, cuda, shape, dtype):
    """Head size 64 takes the vector path (also with a row count that does not fill the last
    warp), other head sizes the generic one; with and without the value-residual inputs."""
    B, T, H, N = shape
    inp = workloads.time_mixer_epilogue_inputs(B, T, H, N, seed=5, dtype=dtype)
    f = {k: v.float().numpy() for k, v in inp.items()}
    g = {k: v.to(cuda) for k, v in inp.items()}
    ref = oracle.weight_prepare(*[f[n] for n in WP_IN], H, *[f[n] for n in WP_VAL])
    out = pkg.weight_prepare_epilogue(*[g[n] for n in WP_IN], H, value_precursor=g["value_precursor"],
                                      value_from_first_cell=g["value_from_first_cell"],
                                      value_residual_lora=g["value_residual_lora"])
    first = pkg.weight_prepare_epilogue(*[g[n] for n in WP_IN], H)
    torch.cuda.synchronize()
    for name in ("weight_decay", "replacement_key", "removal_key_normalized", "replacement", "value"):
        _close(getattr(out, name), ref[name], dtype, name)
    assert first.value is None
    for name in ("weight_decay", "replacement_key", "removal_key_normalized", "replacement"):
        assert torch.equal(getattr(first, name), getattr(out, name))


def test_weight_prepare_feeds_wkv7(pkg, workloads, cuda):
    """[B,T,C] outputs are the [B,T,H,N] inputs of the recurrence: the decay precursor stays below
    -0.5 and the removal key has unit norm, which is what keeps the chunked kernel in range."""
    B, T, H, N = 2, 128, 3, 64
    g = {k: v.to(cuda) for k, v in workloads.time_mixer_epilogue_inputs(B, T, H, N, seed=6,
                                                                       dtype=torch.bfloat16).items()}
    out = pkg.weight_prepare_epilogue(*[g[n] for n in WP_IN], H)
    seq = pkg.Wkv7PretrainForwardInputs(*[t.reshape(B, T, H, N) for t in (
        g["receptance"], out.weight_decay, out.replacement_key, g["value"], out.removal_key_normalized,
        out.replacement)])
    y = pkg.wkv7_pretrain_custom(seq)
    torch.cuda.synchronize()
    assert float(out.weight_decay.float().max()) <= -0.5
    assert torch.isfinite(y.float()).all()
    assert pkg.read_device_status(0) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 8, 2, 64), (1, 3, 5, 64), (2, 7, 3, 20), (1, 5, 2, 7), (2, 512, 12, 64)])
def test_gated_readout(pkg, oracle, workloads, cuda, shape, dtype):
    B, T, H, N = shape
    inp = workloads.time_mixer_epilogue_inputs(B, T, H, N, seed=7, dtype=dtype)
    ref = oracle.gated_readout(*[inp[n].float().numpy() for n in GR_IN], H)
    g = {k: v.to(cuda) for k, v in inp.items()}
    out = pkg.gated_readout_epilogue(*[g[n] for n in GR_IN], H)
    # the same memory described as [B,T,H,N], as the recurrence hands it over
    four = pkg.gated_readout_epilogue(g["wkv7_output"].reshape(B, T, H, N), g["receptance"].reshape(B, T, H, N),
                                      g["replacement_key"].reshape(B, T, H, N), g["value"].reshape(B, T, H, N),
                                      g["gate"], g["group_norm_gamma"], g["group_norm_beta"],
                                      g["receptance_key_bonus"], H)
    torch.cuda.synchronize()
    _close(out, ref, dtype, "output")
    assert four.shape == (B, T, H, N) and torch.equal(four.reshape(B, T, H * N), out)


def test_epilogue_contracts(pkg, workloads, cuda):
    g = {k: v.to(cuda) for k, v in workloads.time_mixer_epilogue_inputs(1, 4, 2, 64, seed=8).items()}
    wp = [g[n] for n in WP_IN]
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.weight_prepare_epilogue(*wp, 3)                       # 3 heads do not divide 128 channels
    assert e.value.kind == "BadArgument"
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.weight_prepare_epilogue(wp[0], wp[1][:, :2].contiguous(), *wp[2:], 2)
    assert e.value.kind == "ShapeMismatch"
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.weight_prepare_epilogue(wp[0], wp[1].to(torch.bfloat16), *wp[2:], 2)
    assert e.value.kind == "DTypeMismatch"
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.weight_prepare_epilogue(*wp, 2, value_precursor=g["value_precursor"])   # value inputs: all or none
    assert e.value.kind == "NullPointer"
    gr = [g[n] for n in GR_IN]
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.gated_readout_epilogue(*gr[:5], gr[5][:64].contiguous(), *gr[6:], 2)
    assert e.value.kind == "ShapeMismatch"
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.gated_readout_epilogue(gr[0].transpose(0, 1), *gr[1:], 2)
    assert e.value.kind in ("NotContiguous", "ShapeMismatch")
    empty = torch.empty(0, 4, 128, device=cuda)
    out = pkg.gated_readout_epilogue(empty, empty, empty, empty, empty, *gr[5:], 2)
    assert out.numel() == 0


@pytest.mark.parametrize("shape", [(2, 8, 64, 256), (1, 130, 72, 264), (3, 33, 128, 520), (1, 1, 8, 8),
                                   (2, 300, 768, 3072)])
def test_channel_mixer(pkg, oracle, workloads, cuda, shape):
    """Token-shift mix, key projection with relu^2 in the epilogue, value projection, against the fp64
    oracle on the same bf16 inputs.  The tensor-core path rounds key_input and the hidden activation
    to bf16 once each (the reference with F = bf16 rounds after every op), so the tolerance is the
    bf16 rounding of those two operands through the contractions: 2e-2 of the output's largest
    magnitude, plus one bf16 spacing for the output's own storage.  Shapes cover edge tiles in every
    dimension (rows, C and F not multiples of the 128 x 256 x 64 tile)."""
    B, T, C, F = shape
    x, ks, kw, vw = workloads.channel_mixer_inputs(B, T, C, F, seed=3)
    ref = oracle.channel_mixer(x.float().numpy(), ks.float().numpy(), kw.float().numpy(), vw.float().numpy())
    out = pkg.channel_mixer_custom(x.to(cuda), ks.to(cuda), kw.to(cuda), vw.to(cuda))
    torch.cuda.synchronize()
    assert pkg.read_device_status(0) == 0
    got = out.float().cpu().numpy().astype(np.float64)
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() <= 2e-2 * scale, np.abs(got - ref).max() / scale
    assert parity.stats(got, ref)["cosine"] >= 0.9999
    # a finer check against a restatement that rounds where the kernel rounds
    ki = torch.cat([torch.zeros(B, 1, C), x.float()[:, :-1]], 1)
    ki = (x.float() + (ki - x.float()) * ks.float()).to(torch.bfloat16).double().reshape(B * T, C)
    hid = (torch.relu(ki @ kw.double().T) ** 2).to(torch.bfloat16).double()
    fine = (hid @ vw.double().T).reshape(B, T, C).numpy()
    tol = 2e-3 * np.abs(fine).max() + 2 * parity.BF16_ULP * np.abs(fine)
    assert (np.abs(got - fine) <= tol).all(), float((np.abs(got - fine) - tol).max())


def test_channel_mixer_contracts(pkg, workloads, cuda):
    x, ks, kw, vw = (t.to(cuda) for t in workloads.channel_mixer_inputs(1, 4, 64, 128, seed=4))
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.channel_mixer_custom(x, ks[:32].contiguous(), kw, vw)
    assert e.value.kind == "ShapeMismatch"
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.channel_mixer_custom(x, ks, kw, vw.T.contiguous())
    assert e.value.kind in ("AxisMismatch", "ShapeMismatch")
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.channel_mixer_custom(x.float(), ks.float(), kw.float(), vw.float())
    assert e.value.kind == "Unsupported"
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.channel_mixer_custom(x, ks, kw, vw, workspace=torch.empty(256, dtype=torch.uint8, device=cuda))
    assert e.value.kind == "WorkspaceTooSmall"
    empty = pkg.channel_mixer_custom(x[:, :0].contiguous(), ks, kw, vw)
    assert empty.shape == (1, 0, 64)
