"""Generates the committed golden fixtures in this directory.

The reference holds no golden vectors for these operators, so the fixtures are
produced by the fp64 CPU oracle (``oracle/rwkv7_oracle.c``) on seeded inputs:
they pin the oracle and the kernels against silent drift, not against reference
outputs.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    oracle = entry.load_oracle()
    oracle.build()
    entry.load_package()
    from rwkv_rs_stable_b200 import workloads

    # Benchmark configuration 0: B=1, T=64, H=4, N=64, fp32, S0 = 0.
    inp = workloads.wkv7_inputs(1, 64, 4, 64, seed=0, dtype=torch.float32)
    f = {k: v.numpy() for k, v in inp.items()}
    y, s = oracle.wkv7(f["r"], f["w"], f["k"], f["v"], f["a"], f["b"], None)
    np.savez_compressed(os.path.join(HERE, "wkv7_cfg0.npz"), y=y.astype(np.float32),
                        s_out=s.astype(np.float32), **{k: v for k, v in f.items()})

    # The reference's own test shape (wkv7/mod.rs:266-292): [2,16,2,8], U[0,1), S0 U[0,1).
    six = workloads.uniform_inputs((2, 16, 2, 8), seed=1)
    s0 = workloads.uniform_inputs((2, 2, 8, 8), seed=2, n=1)[0]
    n = [t.numpy() for t in six]
    y, s = oracle.wkv7(*n, s0.numpy())
    np.savez_compressed(os.path.join(HERE, "wkv7_ref_test_shape.npz"), r=n[0], w=n[1], k=n[2], v=n[3],
                        a=n[4], b=n[5], s0=s0.numpy(), y=y, s_out=s)

    # bf16 inputs, N=64, T not a multiple of 16, non-zero state.
    inp = workloads.wkv7_inputs(2, 40, 2, 64, seed=3, dtype=torch.bfloat16, state="normal")
    f = {k: v.float().numpy() for k, v in inp.items()}
    y, s = oracle.wkv7(f["r"], f["w"], f["k"], f["v"], f["a"], f["b"], f["s0"])
    np.savez_compressed(os.path.join(HERE, "wkv7_bf16_t40.npz"), y=y.astype(np.float32),
                        s_out=s.astype(np.float32), **f)
    # Mixing kernels, the two time-mixer epilogues and the channel mixer at small shapes.
    x, mus = workloads.mix_inputs(2, 8, 32, seed=4)
    diff, _ = workloads.mix_inputs(2, 8, 32, seed=5, nscale=1)
    state = workloads.mix_inputs(1, 4, 32, seed=6, nscale=1)[0][0]          # [4, 32] carried tokens
    ids = np.array([2, 0], dtype=np.int64)
    tsd, tsd_state = oracle.token_shift_diff(x.numpy(), state.numpy(), ids)
    np.savez_compressed(
        os.path.join(HERE, "mix_ops.npz"), x=x.numpy(), diff=diff.numpy(), mus=np.stack([m.numpy() for m in mus]),
        mix6=oracle.mix6(x.numpy(), [m.numpy() for m in mus]),
        addcmul5=oracle.addcmul(x.numpy(), diff.numpy(), [m.numpy() for m in mus[:5]]),
        state=state.numpy(), ids=ids, tsd=tsd, tsd_state=tsd_state)

    ep = workloads.time_mixer_epilogue_inputs(2, 4, 2, 64, seed=7)
    e = {k: v.numpy() for k, v in ep.items()}
    wp = oracle.weight_prepare(e["key_precursor"], e["learning_rate_lora"], e["weight_decay_lora"], e["key_removal"],
                               e["key_replacement"], 2, e["value_precursor"], e["value_from_first_cell"],
                               e["value_residual_lora"])
    gr = oracle.gated_readout(e["wkv7_output"], e["receptance"], e["replacement_key"], e["value"], e["gate"],
                              e["group_norm_gamma"], e["group_norm_beta"], e["receptance_key_bonus"], 2)
    np.savez_compressed(os.path.join(HERE, "time_mixer_epilogues.npz"), gated_readout=gr,
                        **{"in_" + k: v for k, v in e.items()}, **{"wp_" + k: v for k, v in wp.items()})

    cx, cks, ckw, cvw = workloads.channel_mixer_inputs(2, 6, 32, 64, seed=8)
    c = [t.float().numpy() for t in (cx, cks, ckw, cvw)]
    np.savez_compressed(os.path.join(HERE, "channel_mixer.npz"), x=c[0], key_scale=c[1], key_weight=c[2],
                        value_weight=c[3], out=oracle.channel_mixer(*c))

    # Training: saved tensors and gradients at the reference's backward test shape and at N = 64.
    for name, shape in (("wkv7_train_ref_shape", (1, 16, 1, 4)), ("wkv7_train_n64", (1, 32, 1, 64))):
        inp = workloads.wkv7_inputs(*shape, seed=9, state="normal")
        f = {k: v.numpy() for k, v in inp.items()}
        g = torch.Generator().manual_seed(10)
        dy = torch.randn(shape, generator=g).numpy()
        ds = torch.randn(f["s0"].shape, generator=g).numpy()
        y, s_out, snaps, sa = oracle.wkv7_train(*[f[n] for n in "rwkvab"], s0=f["s0"], chunk_len=16)
        grads = oracle.wkv7_backward(*[f[n] for n in "rwkvab"], dy, s0=f["s0"], ds_out=ds)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), dy=dy, ds=ds, y=y, s_out=s_out, snapshots=snaps,
                            state_replacement=sa, **f, **{"d" + k: v for k, v in grads.items()})
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
