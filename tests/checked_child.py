"""Child process of test_gpu_checked_build.py: runs small WKV7 parity cases on the index-checked build of the
library (RWKV7_B200_LIB points at it) with every output and the workspace placed between canary pads, then
verifies the results against the fp64 oracle, the canaries, and that no device-side index check fired."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
import parity  # noqa: E402

PAD = 4096
CANARY = 0xA5


def padded(nbytes, dev):
    """A uint8 buffer [PAD | payload | PAD] filled with the canary byte; returns (whole, payload view)."""
    n = (nbytes + 255) // 256 * 256
    whole = torch.full((PAD + n + PAD,), CANARY, dtype=torch.uint8, device=dev)
    return whole, whole[PAD:PAD + nbytes]


def intact(whole, nbytes):
    n = (nbytes + 255) // 256 * 256
    return bool((whole[:PAD] == CANARY).all() and (whole[PAD + nbytes:PAD + n + PAD] == CANARY).all())


def main():
    pkg = entry.load_package()
    oracle = entry.load_oracle()
    from rwkv_rs_stable_b200 import workloads
    assert pkg.lib().rwkv7_build_features() == 3, "not the checked build"
    dev = torch.device("cuda:0")
    bf, f32 = torch.bfloat16, torch.float32
    cases = [(pkg.WKV7_SPLIT, (2, 192, 3, 64), bf), (pkg.WKV7_SPLIT, (1, 100, 2, 64), bf), (pkg.WKV7_SPLIT, (1, 130, 150, 64), bf),
             (pkg.WKV7_SPLIT, (2, 192, 3, 64), f32), (pkg.WKV7_SPLIT, (1, 100, 2, 64), f32),
             (pkg.WKV7_CHUNKED, (2, 128, 2, 64), bf), (pkg.WKV7_SEQUENTIAL, (2, 37, 3, 64), bf), (pkg.WKV7_SEQUENTIAL, (3, 1, 5, 64), bf)]
    for path, shape, dtype in cases:
        B, T, H, N = shape
        esize = 2 if dtype == bf else 4
        inp = workloads.wkv7_inputs(*shape, seed=91, dtype=dtype, state="normal")
        f = {k: v.float().numpy() for k, v in inp.items()}
        y_ref, s_ref = oracle.wkv7(f["r"], f["w"], f["k"], f["v"], f["a"], f["b"], f["s0"])
        gpu = {k: v.to(dev) for k, v in inp.items()}
        seq = pkg.Wkv7PretrainForwardInputs(*[gpu[n] for n in "rwkvab"])
        pkg.set_wkv7_path(path)
        ws_bytes = int(pkg.lib().rwkv7_wkv7_workspace_bytes(B, T, H, N, pkg.BF16 if dtype == bf else pkg.F32))
        y_whole, y_buf = padded(B * T * H * N * esize, dev)
        s_whole, s_buf = padded(B * H * N * N * 4, dev)
        w_whole, w_buf = padded(max(ws_bytes, 256), dev)
        y = y_buf.view(dtype).view(B, T, H, N)
        s = s_buf.view(torch.float32).view(B, H, N, N)
        out = pkg.wkv7_statepass_custom(gpu["s0"], seq, reference_contract=False, next_state=s, output=y,
                                        workspace=w_buf if ws_bytes else None)
        torch.cuda.synchronize()
        pkg.set_wkv7_path(pkg.WKV7_AUTO)
        status = pkg.read_device_status(0)
        assert status == 0, f"device status {status} for {shape}"
        assert intact(y_whole, B * T * H * N * esize) and intact(s_whole, B * H * N * N * 4), f"canary around an output overwritten, {shape}"
        assert intact(w_whole, max(ws_bytes, 256)), f"canary around the workspace overwritten, {shape}"
        (parity.assert_close_bf16_store if dtype == bf else parity.assert_close_f32)(out.output.float().cpu().numpy(), y_ref, 1e-3, f"y {shape}")
        parity.assert_close_f32(out.next_state.cpu().numpy(), s_ref, 1e-3, f"state {shape}")
    # streaming kernels on the same build
    x, mus = workloads.mix_inputs(2, 8, 32, seed=5, dtype=torch.bfloat16, device=dev)
    outs = pkg.mix6_custom(x, *mus)
    torch.cuda.synchronize()
    assert all(torch.isfinite(o.float()).all() for o in outs.values()) and pkg.read_device_status(0) == 0
    print("CHECKED_BUILD_OK")


if __name__ == "__main__":
    main()
