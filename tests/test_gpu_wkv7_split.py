"""GPU parity of the two-kernel WKV7 prefill (per-chunk operators on the tensor cores in fp16, then one
scan per chain) against the fp64 CPU oracle, through the C ABI.

Tolerances are those of the other WKV7 tests: final state max|d|/max|ref| <= 1e-3, y the same plus one
bf16 spacing of the value (its storage rounding).  Chains that the fp16 operands cannot resolve are
flagged and recomputed by the tf32 chunked kernel, and from there by the sequential scan; the tests
below drive each tier and the hand-over between them.
"""
import numpy as np
import pytest
import torch

import parity

pytestmark = pytest.mark.gpu


def _oracle(oracle, inp):
    f = {k: v.float().numpy() for k, v in inp.items()}
    return oracle.wkv7(f["r"], f["w"], f["k"], f["v"], f["a"], f["b"], f.get("s0"))


def _statepass(pkg, cuda, inp, path, *, alias=False, workspace=None):
    gpu = {k: v.to(cuda) for k, v in inp.items()}
    seq = pkg.Wkv7PretrainForwardInputs(*[gpu[n] for n in "rwkvab"])
    prev = pkg.get_wkv7_path()
    pkg.set_wkv7_path(path)
    try:
        out = pkg.wkv7_statepass_custom(gpu["s0"], seq, reference_contract=False,
                                        next_state=gpu["s0"] if alias else None, workspace=workspace)
        torch.cuda.synchronize()
    finally:
        pkg.set_wkv7_path(prev)
    assert pkg.read_device_status(0) == 0
    return out.output.float().cpu().numpy(), out.next_state.cpu().numpy()


@pytest.mark.parametrize("shape,state", [
    ((1, 64, 1, 64), "normal"), ((2, 128, 3, 64), "normal"), ((1, 100, 2, 64), "normal"),   # T = 100: partial last chunk
    ((2, 65, 2, 64), None), ((1, 37, 2, 64), "normal"),                                     # one token / 37 tokens in the last chunk
    ((1, 1024, 4, 64), "normal"), ((1, 256, 300, 64), None),                                # 300 chains: two scan CTAs per SM
])
def test_split_against_oracle(pkg, oracle, workloads, cuda, shape, state):
    inp = workloads.wkv7_inputs(*shape, seed=71, dtype=torch.bfloat16, state=state)
    y_ref, s_ref = _oracle(oracle, inp)
    if state is None:
        inp["s0"] = torch.zeros(shape[0], shape[2], 64, 64)
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT)
    print("split parity", shape, parity.headline(y, y_ref), parity.headline(s, s_ref))
    parity.assert_close_bf16_store(y, y_ref, 1e-3, "y")
    parity.assert_close_f32(s, s_ref, 1e-3, "state")


def test_split_pretrain_and_statetune_modes(pkg, oracle, workloads, cuda):
    inp = workloads.wkv7_inputs(2, 192, 2, 64, seed=72, dtype=torch.bfloat16)
    y_ref0, _ = _oracle(oracle, inp)
    gpu = {k: v.to(cuda) for k, v in inp.items()}
    seq = pkg.Wkv7PretrainForwardInputs(*[gpu[n] for n in "rwkvab"])
    pkg.set_wkv7_path(pkg.WKV7_SPLIT)
    try:
        y0 = pkg.wkv7_pretrain_custom(seq, reference_contract=False)
        inp["s0"] = workloads.wkv7_inputs(2, 192, 2, 64, seed=73, dtype=torch.bfloat16, state="normal")["s0"]
        y_ref1, _ = _oracle(oracle, inp)
        y1 = pkg.wkv7_statetune_custom(inp["s0"].to(cuda), seq, reference_contract=False)
        torch.cuda.synchronize()
    finally:
        pkg.set_wkv7_path(pkg.WKV7_AUTO)
    parity.assert_close_bf16_store(y0.float().cpu().numpy(), y_ref0, 1e-3, "pretrain y")
    parity.assert_close_bf16_store(y1.float().cpu().numpy(), y_ref1, 1e-3, "statetune y")


def test_split_long_context(pkg, oracle, workloads, cuda):
    """One chain over T = 65 536 (1024 chunks): drift of the fp16 operators against the fp64 oracle."""
    inp = workloads.wkv7_inputs(1, 65536, 1, 64, seed=65, dtype=torch.bfloat16)
    y_ref, s_ref = _oracle(oracle, inp)
    inp["s0"] = torch.zeros(1, 1, 64, 64)
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT)
    print(f"split long context: y {parity.headline(y, y_ref):.3e} state {parity.headline(s, s_ref):.3e}")
    parity.assert_close_bf16_store(y, y_ref, 1e-3, "y")
    parity.assert_close_f32(s, s_ref, 1e-3, "state")


@pytest.mark.parametrize("alias", [False, True])
def test_split_hands_strong_decay_to_the_tf32_kernel(pkg, oracle, workloads, cuda, alias):
    """w = -0.5 throughout (log-decay 38.8 per chunk, the strongest the model's range allows) in one chain:
    beyond what fp16 operands resolve, so the chain is flagged and the tf32 chunked kernel computes it.  Its
    result must be bitwise what the tf32 kernel gives when asked directly, the other chains must come from
    the two-kernel path, and an aliased state must still hold the initial state when the second tier runs."""
    inp = workloads.wkv7_inputs(2, 320, 2, 64, seed=74, dtype=torch.bfloat16, state="normal")
    w = inp["w"].clone()
    w[1, :, 0] = -0.5
    inp["w"] = w
    y_ref, s_ref = _oracle(oracle, inp)
    try:
        pkg.set_wkv7_cluster(1)
        y_tf32, s_tf32 = _statepass(pkg, cuda, inp, pkg.WKV7_CHUNKED)
    finally:
        pkg.set_wkv7_cluster(0)
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, alias=alias)
    parity.assert_close_bf16_store(y, y_ref, 1e-3, "y")
    parity.assert_close_f32(s, s_ref, 1e-3, "state")
    assert np.array_equal(s[1, 0], s_tf32[1, 0]) and np.array_equal(y[1, :, 0], y_tf32[1, :, 0])
    assert not np.array_equal(s[0, 0], s_tf32[0, 0])   # (a different rounding path: equal only by accident)


@pytest.mark.parametrize("alias", [False, True])
def test_split_falls_through_to_the_sequential_scan(pkg, oracle, workloads, cuda, alias):
    """Decay inputs in [0.5, 1.5] (the reference's own test distribution lies there) leave the range of both
    tensor-core kernels: the chain ends in the sequential scan, again from the untouched initial state."""
    inp = workloads.wkv7_inputs(2, 256, 2, 64, seed=75, dtype=torch.bfloat16, state="normal")
    w = inp["w"].float()
    w[0, 64:128, 1] = torch.rand(64, 64) + 0.5   # one chunk in the middle of one chain
    inp["w"] = w.to(torch.bfloat16)
    y_ref, s_ref = _oracle(oracle, inp)
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, alias=alias)
    parity.assert_close_bf16_store(y, y_ref, 1e-3, "y")
    parity.assert_close_f32(s, s_ref, 1e-3, "state")


def test_split_flags_non_finite_operators(pkg, oracle, workloads, cuda):
    """Keys of magnitude 1e4 overflow the fp16 operator although the decay is in range: the scan sees
    non-finite values, flags the chain and the tf32 kernel (fp32 exponent range) computes it."""
    inp = workloads.wkv7_inputs(1, 256, 3, 64, seed=76, dtype=torch.bfloat16, state="normal")
    k = inp["k"].float()
    k[:, :, 2] *= 1.0e4
    inp["k"] = k.to(torch.bfloat16)
    y_ref, s_ref = _oracle(oracle, inp)
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, alias=True)
    assert np.isfinite(y).all() and np.isfinite(s).all()
    for h in range(3):   # per chain: the scales differ by 1e4
        parity.assert_close_bf16_store(y[:, :, h], y_ref[:, :, h], 1e-3, f"y, head {h}")
        parity.assert_close_f32(s[:, h], s_ref[:, h], 1e-3, f"state, head {h}")


@pytest.mark.parametrize("alias", [False, True])
def test_split_in_segments_is_bitwise_the_single_pass(pkg, workloads, cuda, alias):
    """With the smallest workspace the call is cut into one-chunk segments (the state travels through the
    workspace in fp32): same arithmetic, bitwise the same result as with room for every operator."""
    B, T, H = 2, 640, 3
    inp = workloads.wkv7_inputs(B, T, H, 64, seed=77, dtype=torch.bfloat16, state="normal")
    pkg.set_wkv7_path(pkg.WKV7_SPLIT)
    try:
        full = int(pkg.lib().rwkv7_wkv7_workspace_bytes(B, T, H, 64, pkg.BF16))
    finally:
        pkg.set_wkv7_path(pkg.WKV7_AUTO)
    chains = B * H
    least = 256 + 4096 + chains * 64 * 64 * 4 + chains * (512 + 32768)   # flags, work counters, carried state, one chunk of operators
    assert least < full
    y1, s1 = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT)
    for nbytes in (least, least + 3 * chains * (512 + 32768) + 100):   # segments of 1 and of 4 chunks
        ws = torch.empty(nbytes, dtype=torch.uint8, device=cuda)
        y2, s2 = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, alias=alias, workspace=ws)
        assert np.array_equal(y1, y2) and np.array_equal(s1, s2)
    with pytest.raises(pkg.KernelInputsError) as e:
        _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, workspace=torch.empty(least - 1024, dtype=torch.uint8, device=cuda))
    assert e.value.kind == "WorkspaceTooSmall"


def test_automatic_choice(pkg, workloads, cuda):
    """bf16, N = 64, T >= 512 with a workspace of the reported size: the two-kernel path (operators, scan,
    and the two flagged-chain kernels that exit at once: four launches).  A workspace that only holds the
    flags or a short sequence keep the earlier kernels."""
    inp = workloads.wkv7_inputs(2, 512, 2, 64, seed=78, dtype=torch.bfloat16, device=cuda, state="normal")
    seq = pkg.Wkv7PretrainForwardInputs(*[inp[n] for n in "rwkvab"])
    before = pkg.kernel_launch_count()
    a = pkg.wkv7_statepass_custom(inp["s0"], seq, reference_contract=False)
    assert pkg.kernel_launch_count() - before == 4
    pkg.set_wkv7_path(pkg.WKV7_SPLIT)
    try:
        b = pkg.wkv7_statepass_custom(inp["s0"], seq, reference_contract=False)
    finally:
        pkg.set_wkv7_path(pkg.WKV7_AUTO)
    torch.cuda.synchronize()
    assert torch.equal(a.output, b.output) and torch.equal(a.next_state, b.next_state)
    before = pkg.kernel_launch_count()
    small = torch.empty(4 * 4, dtype=torch.uint8, device=cuda)   # flags only
    c = pkg.wkv7_statepass_custom(inp["s0"], seq, reference_contract=False, workspace=small)
    torch.cuda.synchronize()
    assert pkg.kernel_launch_count() - before == 2   # the tf32 chunked kernel and its flagged-chain check
    assert (c.next_state - a.next_state).abs().max() <= 1e-3 * a.next_state.abs().max()
    short = workloads.wkv7_inputs(2, 256, 2, 64, seed=79, dtype=torch.bfloat16, device=cuda, state="normal")
    before = pkg.kernel_launch_count()
    pkg.wkv7_statepass_custom(short["s0"], pkg.Wkv7PretrainForwardInputs(*[short[n] for n in "rwkvab"]), reference_contract=False)
    torch.cuda.synchronize()
    assert pkg.kernel_launch_count() - before == 2


def test_split_shard_equals_single(pkg, workloads, cuda):
    """(b,h) chains are independent and each chain's arithmetic does not depend on how many chains a call
    holds: a batch x head shard computed alone is bitwise the slice of the full result."""
    inp = workloads.wkv7_inputs(4, 384, 6, 64, seed=80, dtype=torch.bfloat16, device=cuda, state="normal")
    full = pkg.wkv7_statepass_custom(inp["s0"], pkg.Wkv7PretrainForwardInputs(*[inp[n] for n in "rwkvab"]),
                                     reference_contract=False)
    for bs, hs in ((slice(0, 2), slice(0, 6)), (slice(0, 4), slice(3, 6)), (slice(3, 4), slice(1, 2))):
        part = {n: inp[n][bs, :, hs].contiguous() for n in "rwkvab"}
        s0 = inp["s0"][bs, hs].contiguous()
        out = pkg.wkv7_statepass_custom(s0, pkg.Wkv7PretrainForwardInputs(*[part[n] for n in "rwkvab"]),
                                        reference_contract=False)
        torch.cuda.synchronize()
        assert torch.equal(out.output, full.output[bs, :, hs]) and torch.equal(out.next_state, full.next_state[bs, hs])


@pytest.mark.parametrize("alias", [False, True])
def test_split_overlapped_scan_is_bitwise_the_serial_one(pkg, oracle, workloads, cuda, alias):
    """Few chains and a long sequence: the call is cut into segments, and the scan of a segment runs beside the
    operator kernel of the next one, each on its own partition of the SMs.  Same kernels on the same data: the
    result must be bitwise that of the single-stream schedule, and both must match the oracle."""
    B, T, H = 1, 16384, 3
    inp = workloads.wkv7_inputs(B, T, H, 64, seed=81, dtype=torch.bfloat16, state="normal")
    y_ref, s_ref = _oracle(oracle, inp)
    before = pkg.kernel_launch_count()
    y1, s1 = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, alias=alias)
    # 256 chunks in four segments, then the two flagged-chain kernels (one segment where the driver offers no SM partitions:
    # with so few chains the schedule beside operator CTAs does not pay)
    assert pkg.kernel_launch_count() - before in (2 * 4 + 2, 2 + 2)
    try:
        pkg.set_wkv7_overlap(False)
        before = pkg.kernel_launch_count()
        y2, s2 = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, alias=alias)
        assert pkg.kernel_launch_count() - before == 2 + 2      # one segment
    finally:
        pkg.set_wkv7_overlap(True)
    assert np.array_equal(y1, y2) and np.array_equal(s1, s2)
    parity.assert_close_bf16_store(y1, y_ref, 1e-3, "y")
    parity.assert_close_f32(s1, s_ref, 1e-3, "state")
    # back-to-back calls on the same buffers reuse the second stream and its events
    gpu = {k: v.to(cuda) for k, v in inp.items()}
    seq = pkg.Wkv7PretrainForwardInputs(*[gpu[n] for n in "rwkvab"])
    outs = [pkg.wkv7_statepass_custom(gpu["s0"], seq, reference_contract=False) for _ in range(4)]
    torch.cuda.synchronize()
    for o in outs:
        assert np.array_equal(o.next_state.cpu().numpy(), s1)


@pytest.mark.parametrize("shape,state", [
    ((2, 128, 3, 64), "normal"), ((1, 100, 2, 64), "normal"), ((2, 65, 2, 64), None),   # partial last chunks
    ((1, 1024, 4, 64), "normal"), ((1, 256, 200, 64), None),                             # 200 chains: more than SMs
])
def test_split_fp32_tensors_against_oracle(pkg, oracle, workloads, cuda, shape, state):
    """fp32 sequence tensors (the dtype of every test of the reference, wkv7/mod.rs:386-398) take the same two
    kernels: fp32 tiles in, fp16 operands on the tensor cores, fp32 y out.  The oracle sees the unrounded
    fp32 inputs; y and the final state within 1e-3 of the largest reference value."""
    inp = workloads.wkv7_inputs(*shape, seed=91, dtype=torch.float32, state=state)
    y_ref, s_ref = _oracle(oracle, inp)
    if state is None:
        inp["s0"] = torch.zeros(shape[0], shape[2], 64, 64)
    before = pkg.kernel_launch_count()
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT)
    assert pkg.kernel_launch_count() - before == 3      # operators, scan, flagged chains by the sequential scan (none)
    print("split fp32 parity", shape, parity.headline(y, y_ref), parity.headline(s, s_ref))
    parity.assert_close_f32(y, y_ref, 1e-3, "y")
    parity.assert_close_f32(s, s_ref, 1e-3, "state")


@pytest.mark.parametrize("alias", [False, True])
def test_split_fp32_flagged_chains_take_the_sequential_scan(pkg, oracle, workloads, cuda, alias):
    """fp32 tensors, one chain with the strongest decay and one with keys that overflow fp16: both are flagged
    and recomputed by the sequential scan from the untouched initial state; the others come from the tensor cores."""
    inp = workloads.wkv7_inputs(2, 320, 3, 64, seed=92, dtype=torch.float32, state="normal")
    inp["w"][1, :, 0] = -0.5
    inp["k"][0, :, 2] *= 1.0e4
    y_ref, s_ref = _oracle(oracle, inp)
    y_seq, s_seq = _statepass(pkg, cuda, inp, pkg.WKV7_SEQUENTIAL)
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_SPLIT, alias=alias)
    assert np.isfinite(y).all() and np.isfinite(s).all()
    for b in range(2):
        for h in range(3):
            parity.assert_close_f32(y[b, :, h], y_ref[b, :, h], 1e-3, f"y, chain {b},{h}")
            parity.assert_close_f32(s[b, h], s_ref[b, h], 1e-3, f"state, chain {b},{h}")
    for b, h in ((1, 0), (0, 2)):
        assert np.array_equal(s[b, h], s_seq[b, h]) and np.array_equal(y[b, :, h], y_seq[b, :, h])
    assert not np.array_equal(s[0, 0], s_seq[0, 0])


def test_split_fp32_automatic_choice_and_long_context(pkg, oracle, workloads, cuda):
    """Under the automatic choice fp32 tensors of T >= 512 take the two-kernel path too (a pair of launches per
    segment of chunks, then the flagged-chain scan), and one chain over T = 16 384 stays within the tolerance."""
    inp = workloads.wkv7_inputs(1, 16384, 1, 64, seed=93, dtype=torch.float32)
    y_ref, s_ref = _oracle(oracle, inp)
    inp["s0"] = torch.zeros(1, 1, 64, 64)
    before = pkg.kernel_launch_count()
    y, s = _statepass(pkg, cuda, inp, pkg.WKV7_AUTO)
    launches = pkg.kernel_launch_count() - before
    assert launches >= 3 and launches % 2 == 1
    print(f"split fp32 long context: y {parity.headline(y, y_ref):.3e} state {parity.headline(s, s_ref):.3e}")
    parity.assert_close_f32(y, y_ref, 1e-3, "y")
    parity.assert_close_f32(s, s_ref, 1e-3, "state")


def test_split_overlap_schedules_agree_bitwise(pkg, workloads, cuda):
    """24 chains x 256 chunks: in sequence on the caller's stream (0), scans on their own SM partition beside the next
    segment's operator kernel (1, the default), and the schedule without partitions, scan CTAs beside operator CTAs
    (2): the same kernels' arithmetic on the same data, so y and the final state must agree bit for bit."""
    inp = workloads.wkv7_inputs(1, 16384, 24, 64, seed=95, dtype=torch.bfloat16, device=cuda, state="normal")
    seq = pkg.Wkv7PretrainForwardInputs(*[inp[n] for n in "rwkvab"])
    outs = {}
    try:
        for mode in (0, 1, 2):
            pkg.set_wkv7_overlap(mode)
            before = pkg.kernel_launch_count()
            o = pkg.wkv7_statepass_custom(inp["s0"], seq, reference_contract=False)
            torch.cuda.synchronize()
            outs[mode] = (o.output.clone(), o.next_state.clone(), pkg.kernel_launch_count() - before)
            assert pkg.read_device_status(0) == 0
    finally:
        pkg.set_wkv7_overlap(1)
    assert outs[0][2] == 2 + 2 and outs[2][2] == 2 * 4 + 2 and outs[1][2] in (2 * 4 + 2, 2 + 2)
    for mode in (1, 2):
        assert torch.equal(outs[mode][0], outs[0][0]) and torch.equal(outs[mode][1], outs[0][1])
