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
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
