"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no dataset is involved anywhere on this path).

WKV7 sequence inputs follow the ranges the reference's ``WeightPrepare`` produces
(``crates/rwkv-nn/src/modules/time_mixer/weight_prepare.rs:252-287``):
``r, k, v ~ N(0,1)``; ``w ~ U(-6,-0.5)`` (the op applies ``exp(-exp(w))``);
``kk`` = L2-normalised ``N(0,1)`` per head; ``a = -kk``; ``b = kk * sigmoid(N(0,1))``.
Values are generated in fp32 and rounded ONCE to the requested dtype, so the
oracle and the kernels consume identical numbers.
"""
from __future__ import annotations

import torch

SEED_BASE = 0x5257_4B56  # "RWKV"

# (B, T, H, N) of the benchmark configurations that are a single WKV7 call.
WKV7_CONFIGS = {
    "cfg0_cpu_f32": dict(B=1, T=64, H=4, N=64, dtype=torch.float32),
    "cfg1_prefill_bf16": dict(B=8, T=4096, H=12, N=64, dtype=torch.bfloat16),
    "cfg2_layer_bf16": dict(B=16, T=8192, H=32, N=64, dtype=torch.bfloat16),
    "cfg3_decode_layer_bf16": dict(B=1024, T=1, H=40, N=64, dtype=torch.bfloat16),
    "cfg4_layer_bf16": dict(B=4, T=65536, H=64, N=64, dtype=torch.bfloat16),
}


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(SEED_BASE * 1000 + seed)
    return g


def wkv7_inputs(B: int, T: int, H: int, N: int, *, seed: int = 0, dtype=torch.float32,
                device="cpu", state: str | None = None):
    """Returns ``dict(r, w, k, v, a, b[, s0])``; ``state`` is None (zero state,
    not materialised), ``"zeros"`` or ``"normal"`` (``N(0, 0.1)`` fp32)."""
    g = _gen(device, seed)
    shape = (B, T, H, N)

    def normal():
        return torch.randn(shape, generator=g, device=device, dtype=torch.float32)

    r, k, v = normal(), normal(), normal()
    w = torch.rand(shape, generator=g, device=device, dtype=torch.float32) * 5.5 - 6.0
    kk = normal()
    kk = kk / kk.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    a = -kk
    b = kk * torch.sigmoid(normal())
    out = {n: t.to(dtype).contiguous() for n, t in dict(r=r, w=w, k=k, v=v, a=a, b=b).items()}
    if state == "zeros":
        out["s0"] = torch.zeros((B, H, N, N), device=device, dtype=torch.float32)
    elif state == "normal":
        out["s0"] = torch.randn((B, H, N, N), generator=g, device=device, dtype=torch.float32) * 0.1
    return out


def uniform_inputs(shape, *, seed: int = 0, dtype=torch.float32, device="cpu", n: int = 6):
    """``n`` tensors of U[0,1): the distribution of the reference's own unit tests
    (``Tensor::random(.., Distribution::Default)``, ``wkv7/mod.rs:386-398``)."""
    g = _gen(device, 7919 + seed)
    return [torch.rand(shape, generator=g, device=device, dtype=torch.float32).to(dtype) for _ in range(n)]


def mix_inputs(B: int, T: int, C: int, *, seed: int = 0, dtype=torch.float32, device="cpu", nscale: int = 6):
    """``x ~ N(0,1)`` of shape ``[B,T,C]`` and ``nscale`` scales ``U[0,1)`` of shape ``[1,1,C]``."""
    g = _gen(device, 104729 + seed)
    x = torch.randn((B, T, C), generator=g, device=device, dtype=torch.float32).to(dtype)
    mus = [torch.rand((1, 1, C), generator=g, device=device, dtype=torch.float32).to(dtype)
           for _ in range(nscale)]
    return x, mus


def lm_head_inputs(R: int, C: int, V: int, *, seed: int = 0, device="cpu"):
    """Hidden rows ``N(0,1)`` bf16, weights ``N(0,0.02)`` bf16, uniform targets in ``[0,V)``."""
    g = _gen(device, 1299709 + seed)
    x = torch.randn((R, C), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn((V, C), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    tg = torch.randint(0, V, (R,), generator=g, device=device, dtype=torch.int64)
    return x, w, tg


def time_mixer_epilogue_inputs(B: int, T: int, H: int, N: int, *, seed: int = 0, dtype=torch.float32,
                               device="cpu"):
    """Inputs of the two time-mixer epilogues at model-like scales: projections and LoRA
    outputs ``N(0,1)``, ``key_removal`` / ``key_replacement`` around their initial values 0.71 /
    1.02 (``weight_prepare.rs:200-201``), GroupNorm gamma around 1, beta and the
    receptance-key bonus small, gate in (0,1)."""
    g = _gen(device, 15485863 + seed)
    C = H * N

    def big(scale=1.0):
        return (torch.randn((B, T, C), generator=g, device=device, dtype=torch.float32) * scale).to(dtype)

    def chan(mean, spread):
        return (mean + spread * torch.randn((1, 1, C), generator=g, device=device, dtype=torch.float32)).to(dtype)

    out = {name: big() for name in ("key_precursor", "learning_rate_lora", "weight_decay_lora",
                                    "value_precursor", "value_from_first_cell", "value_residual_lora",
                                    "wkv7_output", "receptance", "replacement_key", "value")}
    out["gate"] = torch.sigmoid(big().float()).to(dtype)
    out["key_removal"] = chan(0.71, 0.1)
    out["key_replacement"] = chan(1.02, 0.1)
    out["group_norm_gamma"] = chan(1.0, 0.2).reshape(C)
    out["group_norm_beta"] = chan(0.0, 0.1).reshape(C)
    out["receptance_key_bonus"] = chan(0.0, 0.1).reshape(H, N)
    return out


def channel_mixer_inputs(B: int, T: int, C: int, F: int, *, seed: int = 0, dtype=torch.bfloat16, device="cpu"):
    """``x ~ N(0,1)``, ``key_scale ~ U[0,1)``, weights ``N(0, 1/sqrt(fan_in))`` so that the hidden
    activation and the output stay O(1)."""
    g = _gen(device, 32452843 + seed)
    x = torch.randn((B, T, C), generator=g, device=device, dtype=torch.float32).to(dtype)
    key_scale = torch.rand((C,), generator=g, device=device, dtype=torch.float32).to(dtype)
    key_weight = (torch.randn((F, C), generator=g, device=device, dtype=torch.float32) / C ** 0.5).to(dtype)
    value_weight = (torch.randn((C, F), generator=g, device=device, dtype=torch.float32) / F ** 0.5).to(dtype)
    return x, key_scale, key_weight, value_weight
