"""The allocation-free statepass entry point (``rwkv7_fused_wkv7_statepass_noalloc``).

Some callers cannot allocate device memory when they call the library: a serving
process whose memory pool has already taken the whole GPU (a cudaMalloc would
fail), or a runtime thread on which a device allocation is forbidden because it
would stall the device.  For them the chunked kernel's per-chain fallback flags
come from a fixed array inside the library instead of a caller workspace.

This file is collected last on purpose.  It calls the entry point through the C
ABI twice in a row on the same buffers' shapes and checks each result against
the ordinary entry point, within the tolerance the other WKV7 tests use.  The
first call contains chains that the chunked kernel flags for the sequential
fallback, the second contains none, so stale flags left in the shared array by
the first call would corrupt the second if they were not overwritten.
"""
import pytest
import torch

import parity

pytestmark = pytest.mark.gpu


def _inputs(workloads, cuda, seed, flagged):
    inp = workloads.wkv7_inputs(2, 192, 3, 64, seed=seed, dtype=torch.bfloat16, state="normal")
    if flagged:
        w = inp["w"].float()
        w[0] = torch.rand_like(w[0]) + 0.5   # decay far outside the chunked kernel's range
        inp["w"] = w.to(torch.bfloat16)
    return {k: v.to(cuda) for k, v in inp.items()}


def test_noalloc_matches_statepass_twice_in_a_row(pkg, workloads, cuda):
    prev = pkg.get_wkv7_path()
    pkg.set_wkv7_path(pkg.WKV7_CHUNKED)   # the path that uses scratch memory
    try:
        for call, flagged in enumerate((True, False)):
            gpu = _inputs(workloads, cuda, 40 + call, flagged)
            seq = pkg.Wkv7PretrainForwardInputs(*[gpu[n] for n in "rwkvab"])
            ref = pkg.wkv7_statepass_custom(gpu["s0"], seq, reference_contract=False)
            y = torch.empty_like(gpu["r"])
            s = torch.empty_like(gpu["s0"])
            out = pkg.wkv7_statepass_noalloc(gpu["s0"], seq, y, s)
            torch.cuda.synchronize()
            assert out.output.data_ptr() == y.data_ptr() and out.next_state.data_ptr() == s.data_ptr()
            assert pkg.read_device_status(0) == 0
            parity.assert_close_bf16_store(y.float().cpu().numpy(), ref.output.float().cpu().numpy(), 1e-3,
                                           f"y, call {call}")
            parity.assert_close_f32(s.cpu().numpy(), ref.next_state.cpu().numpy(), 1e-3, f"state, call {call}")
    finally:
        pkg.set_wkv7_path(prev)


def test_noalloc_cluster_launch_uses_the_fixed_array(pkg, workloads, cuda):
    """Few chains and a long sequence make the launcher give every chain a cluster of CTAs; that path
    clears its slice of the flag array on the stream before the launch and the CTAs only ever set a
    flag.  Two calls in a row on the fixed array: first with a flagged chain, then with none, so a flag
    that survived the clearing would send a good chain of the second call through the wrong path's
    result check below (both calls are compared with the ordinary entry point)."""
    prev = pkg.get_wkv7_path()
    pkg.set_wkv7_path(pkg.WKV7_CHUNKED)
    try:
        for cluster in (2, 4):
            pkg.set_wkv7_cluster(cluster)
            for call, flagged in enumerate((True, False)):
                inp = workloads.wkv7_inputs(1, 640, 3, 64, seed=50 + call, dtype=torch.bfloat16, state="normal")
                if flagged:
                    w = inp["w"].float()
                    w[0, 128:192, 2] = torch.rand(64, 64) + 0.5
                    inp["w"] = w.to(torch.bfloat16)
                gpu = {k: v.to(cuda) for k, v in inp.items()}
                seq = pkg.Wkv7PretrainForwardInputs(*[gpu[n] for n in "rwkvab"])
                before = pkg.kernel_launch_count()
                ref = pkg.wkv7_statepass_custom(gpu["s0"], seq, reference_contract=False)
                y = torch.empty_like(gpu["r"])
                s = torch.empty_like(gpu["s0"])
                pkg.wkv7_statepass_noalloc(gpu["s0"], seq, y, s)
                torch.cuda.synchronize()
                assert pkg.kernel_launch_count() - before == 4   # per call: the cluster launch and the flag check
                assert pkg.read_device_status(0) == 0
                parity.assert_close_bf16_store(y.float().cpu().numpy(), ref.output.float().cpu().numpy(), 1e-3,
                                               f"y, cluster {cluster}, call {call}")
                parity.assert_close_f32(s.cpu().numpy(), ref.next_state.cpu().numpy(), 1e-3,
                                        f"state, cluster {cluster}, call {call}")
    finally:
        pkg.set_wkv7_cluster(0)
        pkg.set_wkv7_path(prev)


def test_noalloc_reports_contract_errors_before_the_capacity(pkg, cuda):
    """A malformed call gets the reference-ordered contract error, not the capacity message, even when
    its shape would also exceed the array."""
    B, H = 1024, 65
    t = torch.zeros(B, 1, H, 64, dtype=torch.bfloat16, device=cuda)
    bad = torch.zeros(B, 1, H, 32, dtype=torch.bfloat16, device=cuda)
    seq = pkg.Wkv7PretrainForwardInputs(t, t, bad, t, t, t)
    s = torch.zeros(B, H, 64, 64, device=cuda)
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.wkv7_statepass_noalloc(s, seq, torch.empty_like(t), s)
    assert e.value.kind == "ShapeMismatch"


def test_noalloc_rejects_more_chains_than_the_array_holds(pkg, cuda):
    B, H = 1024, 65  # 66560 chains > 65536
    t = torch.zeros(B, 1, H, 64, dtype=torch.bfloat16, device=cuda)
    seq = pkg.Wkv7PretrainForwardInputs(t, t, t, t, t, t)
    s = torch.zeros(B, H, 64, 64, device=cuda)
    with pytest.raises(pkg.KernelInputsError) as e:
        pkg.wkv7_statepass_noalloc(s, seq, torch.empty_like(t), s)
    assert e.value.kind == "Unsupported" and "65536" in str(e.value)
