"""Benchmark of the WKV7 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one WKV7 statepass over one batch of seeded synthetic input through
the C ABI.  At N = 1 the workload is benchmark configuration 1 (chunked prefill,
B=8, T=4096, H=12, N=64, bf16 inputs, fp32 state).  With N > 1 (one rank per
GPU, launched by torch.distributed.run) every rank runs the same per-GPU
workload on its own batch x head shard; WKV7 needs no collective, so scaling is
weak and `value` is the aggregate over ranks divided by the slowest rank's time.

One JSON line is printed by rank 0.  `value` is tokens/s with inputs resident in
HBM; `e2e` is the same metric with pinned host buffers copied in and results
copied out inside the timed region; `roofline` relates the dominant kernel to
the measured HBM peak; `cpu_baseline` times the CPU oracle on a bounded sample;
`decode` reports the batched single-token state sweep of configuration 3.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

CFG1 = dict(B=8, T=4096, H=12, N=64)
DECODE = dict(B=1024, T=1, H=40, N=64)  # one layer-step of configuration 3
METRIC = "wkv7_prefill_tokens_per_s"
UNIT = "tokens/s"
# Algorithmic traffic of one prefill launch: six bf16 inputs and one bf16 output
# per token-head element (14 B x N) plus the fp32 final state per (b,h).
BYTES_PER_TOKEN_HEAD = 64 * 14
STATE_BYTES = 64 * 64 * 4
# Decode: state read + write (fp32) plus seven bf16 vectors per (b,h) per step.
DECODE_BYTES_PER_BH = 2 * STATE_BYTES + 7 * 64 * 2


def bench_config(B, T, H, N, path="auto"):
    """The `config` object of the JSON line (shared by both arms)."""
    return {"workload": f"cfg1 WKV7 chunked prefill B={B} T={T} H={H} N={N} per GPU, S0=0, bf16 in/out, fp32 state, "
                        "64-token chunks: per-chunk operators (fp16 tensor-core tiles) + one scan per chain",
            "B": B, "T": T, "H": H, "N": N, "path": path,
            "l2": "inputs (302 MB per step) exceed the 126 MB L2; no flush needed",
            "sharding": "batch x head shard per rank, no collective on the data path"}


# DRAM bytes of one prefill step from an ncu capture of this very workload (configuration 1, B=8): the
# operator kernel reads 251.7 MB (the five inputs it needs, once) and writes 160 MB (the per-chunk operators;
# part of them is still in L2 when it ends), the scan reads 256.4 MB (operators and v) and writes 34 MB of y.
# Traffic is proportional to the number of chains.  A constant taken from that capture, not measured in the run.
NCU_TRAFFIC_BYTES_CFG1 = 702.6e6   # dram__bytes_read.sum + dram__bytes_write.sum over both kernels, B=8
NCU_TRAFFIC_SOURCE = ("ncu capture of wkv7_chunk_operator_kernel + wkv7_state_scan_kernel on configuration 1 "
                      "(constant, scaled by B/8); about twice the algorithmic bytes because the per-chunk "
                      "operators (32.5 KB per 64 tokens of a chain) pass through memory between the two kernels")


def sustained_tflops():
    """Dense bf16 throughput of a seconds-long cuBLAS loop under the power cap (measured on this pool)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        return 1400.0   # earlier measurement on this pool


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the GPU works."""

    HW_SLOWDOWN = 0x8
    SW_THERMAL = 0x20
    HW_THERMAL = 0x40
    SW_POWER_CAP = 0x4

    def __init__(self, index: int):
        self.samples = []
        self.reasons = set()
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:  # NVML missing: report nulls, never fail the bench
            self.nv = None

    def sample(self):
        if self.nv is None:
            return
        try:
            self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
            r = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            for bit, name in ((self.HW_SLOWDOWN, "hw_slowdown"), (self.SW_THERMAL, "sw_thermal_slowdown"),
                              (self.HW_THERMAL, "hw_thermal_slowdown"), (self.SW_POWER_CAP, "sw_power_cap")):
                if r & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def start(self):
        def loop():
            while not self._stop.is_set():
                self.sample()
                time.sleep(0.005)
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.sm_max,
                "reasons": sorted(self.reasons), "samples": len(s)}


def cpu_baseline(oracle, workloads, torch, budget_s: float = 12.0):
    """Times the fp32 CPU oracle (the restatement of the reference's CPU path) on a
    bounded sample of configuration 1: all T = 4096 tokens of as many (b,h) chains
    as fit the time budget, one chain per host thread at a time."""
    threads = oracle.use_all_cores()
    probe = workloads.wkv7_inputs(1, 256, threads, 64, seed=1, dtype=torch.bfloat16)
    f = [probe[n].float().numpy() for n in "rwkvab"]
    oracle.wkv7(*f, None, precision="f32")
    t0 = time.perf_counter()
    oracle.wkv7(*f, None, precision="f32")
    per_round = (time.perf_counter() - t0) * (CFG1["T"] / 256)  # one chain per thread, full T
    rounds = max(1, min(int(budget_s / max(per_round, 1e-3)), (CFG1["B"] * CFG1["H"]) // threads))
    chains = rounds * threads
    inp = workloads.wkv7_inputs(1, CFG1["T"], chains, 64, seed=1, dtype=torch.bfloat16)
    f = [inp[n].float().numpy() for n in "rwkvab"]
    # The sample usually is the whole workload (a fraction of a second on a many-core host):
    # repeat it for about ten seconds of CPU work and keep the mean.
    reps = 0
    t0 = time.perf_counter()
    while True:
        oracle.wkv7(*f, None, precision="f32")
        reps += 1
        dt_all = time.perf_counter() - t0
        if dt_all > budget_s or (reps >= 5 and dt_all >= 10.0):
            break
    dt = dt_all / reps
    token_heads_per_s = chains * CFG1["T"] / dt
    return {"value": token_heads_per_s / CFG1["H"], "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{chains} of {CFG1['B'] * CFG1['H']} (b,h) chains x T={CFG1['T']} "
                      f"(fp32 oracle, OpenMP), mean of {reps} runs of {dt:.2f} s; tokens/s = token-heads/s / H"}


def run_reference(args):
    """The reference's CPU path cannot be built here (Rust on un-vendored Burn /
    CubeCL), so this arm times the CPU oracle port with every host thread."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    oracle = entry.load_oracle()
    oracle.build()
    entry.load_package()
    from rwkv_rs_stable_b200 import workloads
    threads = oracle.use_all_cores()
    # One step = the whole configuration-1 workload: all T tokens of all B*H chains, OpenMP over the chains.
    chains = CFG1["B"] * CFG1["H"]
    inp = workloads.wkv7_inputs(1, CFG1["T"], chains, 64, seed=1, dtype=torch.bfloat16)
    f = [inp[n].float().numpy() for n in "rwkvab"]
    for _ in range(args.warmup):
        oracle.wkv7(*f, None, precision="f32")
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.wkv7(*f, None, precision="f32")
    dt = (time.perf_counter() - t0) / steps
    value = chains * CFG1["T"] / dt / CFG1["H"]
    sample = (f"all {chains} (b,h) chains x T={CFG1['T']} per step (fp32 oracle port, OpenMP over chains), "
              f"{steps} steps after {args.warmup} warm-up steps")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(**CFG1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "sequential", "chunked"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-streaming", action="store_true")
    ap.add_argument("--no-channel-mixer", action="store_true")
    ap.add_argument("--no-train", action="store_true")
    ap.add_argument("--no-prefill-other", action="store_true")
    ap.add_argument("--no-lm-head", action="store_true")
    ap.add_argument("--no-forward", action="store_true")
    ap.add_argument("--no-cfg4", action="store_true")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: B=4 instead of 8 (151 MB of inputs, still larger than L2)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    from rwkv_rs_stable_b200 import workloads
    pkg.set_wkv7_path({"auto": pkg.WKV7_AUTO, "sequential": pkg.WKV7_SEQUENTIAL, "chunked": pkg.WKV7_CHUNKED}[args.path])

    cfg = dict(CFG1)
    if args.small:
        cfg["B"] = 4
    B, T, H, N = cfg["B"], cfg["T"], cfg["H"], cfg["N"]
    # each rank owns its own batch x head shard: a different seed, the same shape
    host = workloads.wkv7_inputs(B, T, H, N, seed=100 + rank, dtype=torch.bfloat16, device=dev)
    six = [host[n] for n in "rwkvab"]
    s0 = torch.zeros(B, H, N, N, device=dev)
    y = torch.empty_like(six[0])
    s_out = torch.empty_like(s0)
    seq = pkg.Wkv7PretrainForwardInputs(*six)
    ws_bytes = int(pkg.lib().rwkv7_wkv7_workspace_bytes(B, T, H, N, pkg.BF16))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev) if ws_bytes else None

    step = pkg.Wkv7StatepassCall(s0, seq, y, s_out, ws)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()

    sampler = ClockSampler(local_rank)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    launches0 = pkg.kernel_launch_count()
    sampler.start()
    sync_all()
    for i in range(args.steps):
        starts[i].record()
        step()
        ends[i].record()
    sync_all()
    clocks = sampler.stop()
    launches = pkg.kernel_launch_count() - launches0
    total_ms = starts[0].elapsed_time(ends[-1])
    kernel_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends)) / args.steps
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    tokens_per_step = B * T * world
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---- end to end: pinned host buffers in, y and S_T out, every step ----------
    # The library's host-buffer entry cuts the batch into slices on a few streams, so the
    # copy of one slice overlaps the kernel and the copy-back of the ones before it.
    pinned = [t_.cpu().pin_memory() for t_ in six]
    y_host = torch.empty(y.shape, dtype=y.dtype).pin_memory()
    s_host = torch.empty(s_out.shape, dtype=s_out.dtype).pin_memory()
    e2e_step = pkg.Wkv7HostStatepass(pinned, None, y_host, s_host, device=dev)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(e2e_steps):
        e2e_step(join=(i + 1 == e2e_steps))   # passes are issued back to back; the last one joins
    e1.record()
    sync_all()
    te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = tokens_per_step / (float(te.item()) / e2e_steps * 1e-3)
    h2d, d2h = e2e_step.bytes_per_call()
    # A batch slice has few enough chains for the cluster-of-4 variant of the kernel, which applies the
    # triangular inverse as one precomputed operand (a different, equally accurate rounding path: both
    # are 2-3e-4 from the fp64 oracle and 1.1-1.6e-4 from each other), hence a tolerance, not equality.
    y_dev, s_dev = y.float().cpu(), s_out.cpu()
    if not ((y_host.float() - y_dev).abs().max() <= 1e-3 * y_dev.abs().max() + 2 ** -8 * y_dev.abs().max()
            and (s_host - s_dev).abs().max() <= 5e-4 * s_dev.abs().max()):
        raise SystemExit("end-to-end result differs from the device-resident call")

    # ---- bare host-to-device copies of one step's inputs (what bounds `e2e`) ---------------
    # Every rank copies its six pinned input tensors to the device, nothing else, all ranks at once:
    # the ceiling of the end-to-end figure above, whose steps move the same bytes plus y and S_T back.
    host_copy = None
    if True:
        hc_steps = 5
        for d_, h_ in zip(six, pinned):
            d_.copy_(h_, non_blocking=True)
        sync_all()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record()
        for _ in range(hc_steps):
            for d_, h_ in zip(six, pinned):
                d_.copy_(h_, non_blocking=True)
        h1.record()
        sync_all()
        th = torch.tensor([h0.elapsed_time(h1) / hc_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(th, op=dist.ReduceOp.MAX)
        copy_gbs = h2d / (float(th.item()) * 1e-3) / 1e9
        e2e_gbs = h2d / (float(te.item()) / e2e_steps * 1e-3) / 1e9
        host_copy = {"what": f"{hc_steps} x six pinned input tensors ({h2d} B) host to device per rank, all {world} "
                             "ranks at once, no kernels; slowest rank",
                     "h2d_gb_per_s_per_rank": copy_gbs, "h2d_gb_per_s_all_ranks": copy_gbs * world,
                     "e2e_h2d_gb_per_s_per_rank": e2e_gbs,
                     "e2e_over_copy_ceiling": e2e_gbs / copy_gbs,
                     "e2e_bound": "host copies" if e2e_gbs >= 0.8 * copy_gbs else "pipeline"}

    # ---- the same prefill kernel at the other configurations' per-GPU shapes --------------
    # (Runs before the tensor-core legs: right after the LM-head leg the SM clock is still held down by the
    # power cap for some tens of milliseconds, which a latency-bound kernel feels one to one.)
    prefill_other = None
    if not args.no_prefill_other and rank == 0 and not args.small:
        peak_gbs, _ = measured_peaks()
        prefill_other = {}
        for name, (Bo, To, Ho, odt) in (("cfg2_layer_1gpu", (16, 8192, 32, torch.bfloat16)),
                                        ("cfg4_layer_shard_of_8", (4, 65536, 8, torch.bfloat16)),
                                        ("single_sequence_cfg2_model", (1, 8192, 32, torch.bfloat16)),
                                        ("cfg1_fp32_tensors", (CFG1["B"], CFG1["T"], CFG1["H"], torch.float32))):
            oin = workloads.wkv7_inputs(Bo, To, Ho, 64, seed=11, dtype=odt, device=dev)
            oseq = pkg.Wkv7PretrainForwardInputs(*[oin[n] for n in "rwkvab"])
            os0 = torch.zeros(Bo, Ho, 64, 64, device=dev)
            oy, oso = torch.empty_like(oin["r"]), torch.empty_like(os0)
            esize = oin["r"].element_size()
            ows_bytes = int(pkg.lib().rwkv7_wkv7_workspace_bytes(Bo, To, Ho, 64, pkg.BF16 if esize == 2 else pkg.F32))
            ows = torch.empty(max(ows_bytes, 1), dtype=torch.uint8, device=dev)
            ocall = pkg.Wkv7StatepassCall(os0, oseq, oy, oso, ows)
            for _ in range(2):
                ocall()
            torch.cuda.synchronize()
            o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            o0.record()
            for _ in range(3):
                ocall()
            o1.record()
            torch.cuda.synchronize()
            oms = o0.elapsed_time(o1) / 3
            obytes = Bo * To * Ho * 64 * 7 * esize + Bo * Ho * STATE_BYTES
            prefill_other[name] = {"shape": f"B={Bo} T={To} H={Ho} N=64 {'bf16' if esize == 2 else 'fp32'} ({Bo * Ho} chains)",
                                   "ms": oms, "tokens_per_s": Bo * To / (oms * 1e-3), "gb_per_s": obytes / (oms * 1e-3) / 1e9,
                                   "frac_of_hbm_peak": obytes / (oms * 1e-3) / 1e9 / peak_gbs,
                                   "algorithmic_bytes": obytes}
            del oin, oseq, os0, oy, oso, ows, ocall

    # ---- configuration 4 as a configuration: heads sharded over the ranks -----------------
    # 7B shape (H = 64 heads of 64, C = 4096), B = 4 sequences of T = 65 536 tokens.  One layer's WKV7
    # call on this rank's heads (modules/time_mixer/mod.rs:187-198 makes one call per layer over
    # [B,T,H,N]), the all-gather of the head-split y into [B,T,H,N] on every rank (C1), and the
    # vocabulary-sharded LM head with the log-sum-exp combine over NCCL (C2) on a bounded number of rows.
    # (The WKV7 call and the gather run here, before the tensor-core legs: after those the SM clock stays held down
    # by the power cap for some tens of milliseconds, which a latency-bound kernel feels one to one.)
    cfg4 = None
    cfg4_run = world > 1 and 64 % world == 0 and not args.small and not args.no_cfg4
    if cfg4_run:
        from rwkv_rs_stable_b200 import dist as rdist4
        torch.cuda.empty_cache()
        B4, T4, H4 = 4, 65536, 64
        bs, hs = rdist4.shard_ranges(B4, H4, world)[rank]
        Bl4, Hl4 = bs.stop - bs.start, hs.stop - hs.start
        in4 = workloads.wkv7_inputs(Bl4, T4, Hl4, 64, seed=400 + rank, dtype=torch.bfloat16, device=dev)
        seq4 = pkg.Wkv7PretrainForwardInputs(*[in4[n] for n in "rwkvab"])
        s04 = torch.zeros(Bl4, Hl4, 64, 64, device=dev)
        y4, so4 = torch.empty_like(in4["r"]), torch.empty_like(s04)
        ws4_bytes = int(pkg.lib().rwkv7_wkv7_workspace_bytes(Bl4, T4, Hl4, 64, pkg.BF16))
        ws4 = torch.empty(max(ws4_bytes, 1), dtype=torch.uint8, device=dev)
        call4 = pkg.Wkv7StatepassCall(s04, seq4, y4, so4, ws4)

        def timed_all(fn, reps):
            fn()
            sync_all()
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_.record()
            for _ in range(reps):
                r_ = fn()
            b_.record()
            sync_all()
            t_ = torch.tensor([a_.elapsed_time(b_) / reps], device=dev, dtype=torch.float64)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            return float(t_.item()), r_

        wkv4_ms, _ = timed_all(call4, 3)
        gather_ms, full4 = timed_all(lambda: rdist4.gather_outputs(y4, B4, H4), 2)
        gather_ok = bool(torch.equal(full4[bs, :, hs], y4))
        # every rank's slot must hold that rank's tensor: compare a checksum of each slot with its owner's
        sums = torch.stack([full4[b_, :, h_].float().sum() for b_, h_ in rdist4.shard_ranges(B4, H4, world)])
        own = torch.zeros(world, device=dev)
        own[rank] = y4.float().sum()
        dist.all_reduce(own)
        gather_ok = gather_ok and bool(torch.equal(sums, own))
        okt = torch.tensor([1.0 if gather_ok else 0.0], device=dev)
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        gather_ok = bool(okt.item() == 1.0)
        y_bytes = B4 * T4 * H4 * 64 * 2
        del full4, in4, seq4, y4, call4, s04, so4, ws4
        torch.cuda.empty_cache()
        if not gather_ok:
            raise SystemExit("cfg4 leg: the gathered y differs from the rank-local shards")

    # ---- training forward (with saved tensors) and backward at configuration 1 ------------
    train = None
    if not args.no_train and rank == 0:
        peak_gbs, _ = measured_peaks()
        tin = pkg.Wkv7PretrainForwardInputs(*six)
        saved = pkg.wkv7_forward_saved(tin, None, want_state=True)
        dy = torch.randn_like(six[0])

        def timed(fn, reps=3):
            fn()
            torch.cuda.synchronize()
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_.record()
            for _ in range(reps):
                fn()
            b_.record()
            torch.cuda.synchronize()
            return a_.elapsed_time(b_) / reps

        seq_bytes = B * T * H * N * 2
        snap_bytes = B * H * (T // 16) * N * N * 4
        fwd_ms = timed(lambda: pkg.wkv7_forward_saved(tin, None, want_state=True))
        bws = torch.empty(pkg.wkv7_backward_workspace_bytes(B, T, H, N), dtype=torch.uint8, device=dev)
        bwd_ms = timed(lambda: pkg.wkv7_backward(tin, saved, dy, None, workspace=bws))
        bwd_seq_ms = timed(lambda: pkg.wkv7_backward(tin, saved, dy, None, parallel=False), reps=2)
        fwd_bytes = 8 * seq_bytes + snap_bytes + B * H * STATE_BYTES             # 6 in, y and sa out, snapshots, S_T
        bwd_bytes = 14 * seq_bytes + snap_bytes + B * H * STATE_BYTES            # 6 in, sa, dy, 6 grads, snapshots, dS0
        train = {"workload": f"B={B} T={T} H={H} N={N} bf16, chunk_len 16",
                 "forward_saved_ms": fwd_ms, "forward_saved_gb_per_s": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                 "forward_saved_frac_of_hbm_peak": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak_gbs,
                 "backward_ms": bwd_ms, "backward_token_by_token_ms": bwd_seq_ms, "backward_gb_per_s": bwd_bytes / (bwd_ms * 1e-3) / 1e9,
                 "backward_frac_of_hbm_peak": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak_gbs,
                 "forward_algorithmic_bytes": fwd_bytes, "backward_algorithmic_bytes": bwd_bytes}
        del saved, dy, bws

    # ---- token-shift mixing kernels at the configuration-2 layer shape (HBM-bound) --------
    streaming = None
    if not args.no_streaming and rank == 0:
        peak_gbs, _ = measured_peaks()
        Bs, Ts, Cs = (4, 4096, 2048) if args.small else (16, 8192, 2048)
        x, mus = workloads.mix_inputs(Bs, Ts, Cs, seed=5, dtype=torch.bfloat16, device=dev)
        diff = torch.randn_like(x)
        state = torch.zeros(Bs + 1, Cs, dtype=torch.bfloat16, device=dev)
        ids = torch.arange(Bs, dtype=torch.int32, device=dev)
        elems = Bs * Ts * Cs

        def timeit(fn, nbytes, reps=10):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            ms = None
            for _ in range(3):   # best of three rounds: the first kernels after another leg have measured up to 25 % slow
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(reps):
                    fn()
                b.record()
                torch.cuda.synchronize()
                t = a.elapsed_time(b) / reps
                ms = t if ms is None else min(ms, t)
            gbs = nbytes / (ms * 1e-3) / 1e9
            return {"ms": ms, "gb_per_s": gbs, "frac_of_hbm_peak": gbs / peak_gbs, "algorithmic_bytes": nbytes}

        # outputs are allocated inside the wrappers (caching allocator, no cudaMalloc after warm-up)
        streaming = {
            "shape": f"B={Bs} T={Ts} C={Cs} bf16 (configuration 2 layer shape)",
            "mix6": timeit(lambda: pkg.mix6_custom(x, *mus), 7 * 2 * elems),
            "addcmul": timeit(lambda: pkg.addcmul_custom(x, diff, mus[0]), 3 * 2 * elems),
            "addcmul5": timeit(lambda: pkg.addcmul5_custom(x, diff, *mus[:5]), 7 * 2 * elems),
            "token_shift_diff": timeit(lambda: pkg.token_shift_diff_custom(x, state, ids, inplace_state=True),
                                       2 * 2 * elems),
        }
        del x, diff, mus
        # the two time-mixer epilogues at the same layer shape (H = C / 64 heads)
        Hs = Cs // 64
        ep = workloads.time_mixer_epilogue_inputs(Bs, Ts, Hs, 64, seed=6, dtype=torch.bfloat16, device=dev)
        wp = [ep[n] for n in ("key_precursor", "learning_rate_lora", "weight_decay_lora", "key_removal",
                              "key_replacement")]
        gr = [ep[n] for n in ("wkv7_output", "receptance", "replacement_key", "value", "gate",
                              "group_norm_gamma", "group_norm_beta", "receptance_key_bonus")]
        streaming["weight_prepare"] = timeit(
            lambda: pkg.weight_prepare_epilogue(*wp, Hs, value_precursor=ep["value_precursor"],
                                                value_from_first_cell=ep["value_from_first_cell"],
                                                value_residual_lora=ep["value_residual_lora"]),
            11 * 2 * elems)
        streaming["gated_readout"] = timeit(lambda: pkg.gated_readout_epilogue(*gr, Hs), 6 * 2 * elems)
        del ep, wp, gr

    # ---- decode: configuration 3 (32 layers, B=1024 sequences, H=40), state in place ----
    # (After the streaming leg: a second of saturated HBM traffic and 21.5 GB of fresh allocations
    # cost the streaming kernels that followed it up to 10 %.)
    # One decode step = one single-token statepass per layer, every layer on its own fp32 state
    # (21.5 GB in all, far beyond L2).  With N GPUs the batch is split over the ranks (strong
    # scaling, no exchange: sequences are independent).  Timed twice: launch by launch, and as
    # one CUDA graph per step replayed (the launches of a shard of 1/8 are ~26 us each).
    decode = None
    if not args.no_decode and DECODE["B"] % world == 0:
        dec_L = 4 if args.small else 32
        dec_B = (256 if args.small else DECODE["B"]) // world
        dcalls, dkeep = [], []
        for layer in range(dec_L):
            d = workloads.wkv7_inputs(dec_B, 1, DECODE["H"], 64, seed=100 * rank + layer, dtype=torch.bfloat16,
                                      device=dev, state="normal")
            dseq = pkg.Wkv7PretrainForwardInputs(*[d[n] for n in "rwkvab"])
            dy = torch.empty_like(d["r"])
            dcalls.append(pkg.Wkv7StatepassCall(d["s0"], dseq, dy, d["s0"]))
            dkeep.append((d, dseq, dy))

        def decode_step():
            for c in dcalls:
                c()

        def time_steps(fn, n):
            for _ in range(3):
                fn()
            sync_all()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(n):
                fn()
            t1.record()
            sync_all()
            t = torch.tensor([t0.elapsed_time(t1) / n], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        n_dec = 8 if args.small else 64
        dms = time_steps(decode_step, n_dec)
        gms, graph_note = None, None
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                decode_step()   # warm-up on the capturing stream
                with torch.cuda.graph(graph, stream=side):
                    decode_step()
            torch.cuda.current_stream(dev).wait_stream(side)
            gms = time_steps(graph.replay, n_dec)
            del graph
        except Exception as exc:   # the eager figure stands on its own
            graph_note = f"graph capture failed: {type(exc).__name__}"
            torch.cuda.synchronize()
        if pkg.read_device_status(local_rank) != 0:
            raise SystemExit("decode leg: device status word reports an error")
        dbytes = dec_B * world * DECODE["H"] * DECODE_BYTES_PER_BH * dec_L
        best = min(dms, gms) if gms is not None else dms
        decode = {"workload": f"cfg3 decode step: {dec_L} layers x B={dec_B * world} H=40 N=64, one token per sequence, "
                              "fp32 state updated in place (every layer its own state, far larger than L2)",
                  "sharding": "none" if world == 1 else f"batch over {world} GPUs ({dec_B} sequences each), no exchange",
                  "scaling": "strong", "steps_timed": n_dec,
                  "ms_per_step": best, "ms_per_step_launch_by_launch": dms, "ms_per_step_cuda_graph": gms,
                  "ms_per_layer_step": best / dec_L,
                  "state_gb_per_s": dbytes / (best * 1e-3) / 1e9,
                  "tokens_per_s": dec_B * world / (best * 1e-3),
                  "algorithmic_bytes": dbytes}
        if graph_note:
            decode["note"] = graph_note
        del dcalls, dkeep
        torch.cuda.empty_cache()

    # ---- whole prefill forward of the configuration-2 model (secondary figure) ------------
    # 24 cells of C = 2048 (32 heads), vocabulary 65 536, B = 16 sequences of T = 8192 random token
    # ids, random-init bf16 weights, fused LM-head cross entropy on the shifted targets.  Every
    # hot-path operator goes through the C ABI; the dense projections and LoRA products are cuBLAS
    # matmuls, layer norms and residuals torch ops (rwkv-rs-stable_b200/cell_forward.py).  With N
    # GPUs the batch is split over the ranks (replicated weights, no collective in the forward).
    forward = None
    if not args.no_forward and (16 % world == 0):
        from rwkv_rs_stable_b200 import cell_forward as cf
        Lf, Cf, Hf, Ff, Vf, Bf, Tf = (2, 512, 8, 2048, 4096, 2, 1024) if args.small else (24, 2048, 32, 8192, 65536, 16, 8192)
        Bl = max(Bf // world, 1)
        with torch.no_grad():
            cells = [cf.random_cell(i, Cf, Hf, Ff, device=dev, seed=9, num_cells=Lf) for i in range(Lf)]
            gf = torch.Generator(device=dev)
            gf.manual_seed(99 + rank)
            emb = (torch.randn((Vf, Cf), generator=gf, device=dev) * 0.02).to(torch.bfloat16)
            headw = (torch.randn((Vf, Cf), generator=gf, device=dev) * 0.02).to(torch.bfloat16)
            fln = (torch.ones(Cf, device=dev, dtype=torch.bfloat16), torch.zeros(Cf, device=dev, dtype=torch.bfloat16))
            ids = torch.randint(0, Vf, (Bl, Tf), generator=gf, device=dev)
            cmws = torch.empty(int(pkg.lib().rwkv7_channel_mixer_workspace_bytes(Bl, Tf, Cf, Ff)) or 1,
                               dtype=torch.uint8, device=dev)
            floss = cf.prefill_forward(pkg, cells, emb, headw, fln, ids, Hf, cmws)   # warm-up
            sync_all()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n_fw = 2
            launches_before = pkg.kernel_launch_count()
            f0.record()
            for _ in range(n_fw):
                floss = cf.prefill_forward(pkg, cells, emb, headw, fln, ids, Hf, cmws)
            f1.record()
            sync_all()
            fw_launches = (pkg.kernel_launch_count() - launches_before) // n_fw
        tf_ms = torch.tensor([f0.elapsed_time(f1) / n_fw], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tf_ms, op=dist.ReduceOp.MAX)
        fms = float(tf_ms.item())
        forward = {"workload": f"L={Lf} C={Cf} H={Hf} F={Ff} V={Vf}, B={Bf} T={Tf} random token ids, bf16 random-init "
                               "weights, LM-head cross entropy on shifted targets",
                   "sharding": "none" if world == 1 else f"batch over {world} GPUs ({Bl} sequences each), weights replicated",
                   "scaling": "strong", "ms": fms, "tokens_per_s": Bl * world * Tf / (fms * 1e-3),
                   "library_kernel_launches_per_forward": int(fw_launches),
                   "mean_loss": float(floss.item()),
                   "dense_projections": "cuBLAS (torch.matmul), outside the hot path"}
        del cells, emb, headw, ids, cmws, floss
        torch.cuda.empty_cache()

    # ---- fused LM-head cross entropy at the configuration-2 shape (tensor-core-bound) -----
    # One GPU: the whole vocabulary.  N GPUs: the vocabulary is sharded over the ranks (strong
    # scaling of one LM head), every rank computes the partial triples of its shard, the triples
    # are all-gathered over NCCL and combined on every rank.
    lm_head = None
    if not args.no_lm_head:
        from rwkv_rs_stable_b200 import dist as rdist
        Rl, Cl, Vl = (8192, 2048, 16384) if args.small else (16 * 8192, 2048, 65536)
        xl, wl, tl = workloads.lm_head_inputs(Rl, Cl, Vl, seed=2, device=dev)   # same seed on every rank
        lo, hi = rdist.vocab_shard(Vl, rank, world)
        w_shard = wl[lo:hi].contiguous()
        if world > 1:
            del wl

        def lm_step():
            if world > 1:
                return rdist.lm_head_ce_sharded(pkg, xl, w_shard, tl, lo)
            return pkg.lm_head_ce(xl, w_shard, tl)

        for _ in range(2):
            lm_step()
        sync_all()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_lm = 3
        l0.record()
        for _ in range(n_lm):
            lse, loss = lm_step()
        l1.record()
        sync_all()
        tl_ms = torch.tensor([l0.elapsed_time(l1) / n_lm], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tl_ms, op=dist.ReduceOp.MAX)
        lms = float(tl_ms.item())
        flops = 2.0 * Rl * Cl * Vl
        tf_peak = 1653.6
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                tf_peak = float(json.load(f)["bf16_tflops"])
        except Exception:
            pass
        lm_head = {"workload": f"R={Rl} C={Cl} V={Vl} bf16, logits never materialised (configuration 2)",
                   "sharding": "none" if world == 1 else f"vocabulary over {world} GPUs, all-gather of [R,3] partials + combine",
                   "scaling": "strong",
                   "ms": lms, "tflops": flops / (lms * 1e-3) / 1e12, "peak_tflops": tf_peak * world,
                   "frac_of_bf16_peak": flops / (lms * 1e-3) / 1e12 / (tf_peak * world),
                   "frac_of_bf16_sustained_peak": flops / (lms * 1e-3) / 1e12 / (sustained_tflops() * world),
                   "mean_loss": float(loss.mean().item())}
        del xl, w_shard, tl

    # ---- channel mixer at the configuration-2 layer shape (two tensor-core projections) ---
    channel_mixer = None
    if not args.no_channel_mixer and rank == 0:
        Bc, Tc, Cc, Fc = (2, 4096, 2048, 8192) if args.small else (16, 8192, 2048, 8192)
        cx, cks, ckw, cvw = workloads.channel_mixer_inputs(Bc, Tc, Cc, Fc, seed=7, device=dev)
        cws = torch.empty(int(pkg.lib().rwkv7_channel_mixer_workspace_bytes(Bc, Tc, Cc, Fc)) or 1,
                          dtype=torch.uint8, device=dev)
        for _ in range(2):
            pkg.channel_mixer_custom(cx, cks, ckw, cvw, workspace=cws)
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_cm = 5
        c0.record()
        for _ in range(n_cm):
            cout = pkg.channel_mixer_custom(cx, cks, ckw, cvw, workspace=cws)
        c1.record()
        torch.cuda.synchronize()
        cms = c0.elapsed_time(c1) / n_cm
        cflops = 4.0 * Bc * Tc * Cc * Fc
        tf_peak_cm = 1653.6
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                tf_peak_cm = float(json.load(f)["bf16_tflops"])
        except Exception:
            pass
        channel_mixer = {"workload": f"B={Bc} T={Tc} C={Cc} F={Fc} bf16: token-shift mix, key projection with relu^2 "
                                     "epilogue, value projection",
                         "ms": cms, "tflops": cflops / (cms * 1e-3) / 1e12, "peak_tflops": tf_peak_cm,
                         "frac_of_bf16_peak": cflops / (cms * 1e-3) / 1e12 / tf_peak_cm,
                         # this leg runs right after the LM head, at the clocks of a sustained tensor load
                         "frac_of_bf16_sustained_peak": cflops / (cms * 1e-3) / 1e12 / sustained_tflops(),
                         "output_abs_mean": float(cout.float().abs().mean().item())}
        del cx, ckw, cvw, cws, cout

    # ---- configuration 4, second part: the vocabulary-sharded LM head (C2 on NCCL) ---------
    if cfg4_run:
        from rwkv_rs_stable_b200 import dist as rdist4
        R4, C4, V4 = 32768, 4096, 65536
        x4, _, t4 = workloads.lm_head_inputs(R4, C4, 8, seed=4, device=dev)        # same rows on every rank
        t4 = torch.randint(0, V4, (R4,), generator=torch.Generator(device=dev).manual_seed(44), device=dev)
        lo4, hi4 = rdist4.vocab_shard(V4, rank, world)
        g4 = torch.Generator(device=dev)
        g4.manual_seed(4000 + rank)
        w4 = (torch.randn((hi4 - lo4, C4), generator=g4, device=dev) * 0.02).to(torch.bfloat16)
        lm4_ms, (lse4, loss4) = timed_all(lambda: rdist4.lm_head_ce_sharded(pkg, x4, w4, t4, lo4), 3)
        lm4_flops = 2.0 * R4 * C4 * V4
        peak4, _ = measured_peaks()
        tfp4 = 1653.6
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                tfp4 = float(json.load(f)["bf16_tflops"])
        except Exception:
            pass
        wkv4_bytes = B4 * T4 * H4 * BYTES_PER_TOKEN_HEAD + B4 * H4 * STATE_BYTES
        cfg4 = {"workload": f"cfg4 layer: B={B4} T={T4} H={H4} N=64 bf16, heads sharded over {world} GPUs "
                            f"({Bl4} x {Hl4} = {Bl4 * Hl4} chains per rank), S0 = 0",
                "wkv7_ms": wkv4_ms, "wkv7_tokens_per_s": B4 * T4 / (wkv4_ms * 1e-3),
                "wkv7_gb_per_s": wkv4_bytes / (wkv4_ms * 1e-3) / 1e9,
                "wkv7_frac_of_hbm_peak": wkv4_bytes / (wkv4_ms * 1e-3) / 1e9 / (peak4 * world),
                "wkv7_hbm_roof_ms": wkv4_bytes / (peak4 * world * 1e9) * 1e3,
                "gather": "NCCL all-gather of the head-split y into [world,B,T,H_loc,N] on every rank + one strided copy into [B,T,H,N]",
                "gather_ms": gather_ms, "gather_bytes_full_tensor": y_bytes,
                "gather_bus_gb_per_s": y_bytes * (world - 1) / world / (gather_ms * 1e-3) / 1e9,
                "gather_checked": gather_ok,
                "lm_head": f"R={R4} of {B4 * T4} rows, C={C4}, V={V4} sharded {hi4 - lo4} columns per rank, "
                           "all-gather of [R,3] partials + combine on every rank",
                "lm_head_ms": lm4_ms, "lm_head_tflops": lm4_flops / (lm4_ms * 1e-3) / 1e12,
                "lm_head_frac_of_bf16_peak": lm4_flops / (lm4_ms * 1e-3) / 1e12 / (tfp4 * world),
                "lm_head_frac_of_bf16_sustained_peak": lm4_flops / (lm4_ms * 1e-3) / 1e12 / (sustained_tflops() * world),
                "lm_head_mean_loss": float(loss4.mean().item())}
        del x4, w4, t4
        torch.cuda.empty_cache()


    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    alg_bytes = B * T * H * BYTES_PER_TOKEN_HEAD + B * H * STATE_BYTES
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    if decode is not None:
        decode["frac_of_hbm_peak"] = decode["state_gb_per_s"] / (peak * world)
        decode["peak"] = f"{world} x {peak} GB/s {peak_kind}"
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES_CFG1 * (B / 8.0) if args.path != "sequential" else None,
                "traffic_source": NCU_TRAFFIC_SOURCE if args.path != "sequential" else None,
                "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": kernel_ms,
                "kernels": "one step = wkv7_chunk_operator_kernel (about 3/4 of the time) + wkv7_state_scan_kernel + two "
                           "flagged-chain kernels that exit at once; kernel_ms is the device time of the whole step"}
    if decode is not None:
        # the metric names two figures: the second one (decode state GB/s against the HBM peak) rides here
        roofline["decode_gb_per_s"] = decode["state_gb_per_s"]
        roofline["decode_frac"] = decode["frac_of_hbm_peak"]
        roofline["decode_ms_per_step"] = decode["ms_per_step"]
    cpu = None
    if not args.no_cpu_baseline:
        oracle = entry.load_oracle()
        oracle.build()
        cpu = cpu_baseline(oracle, workloads, torch)

    def pick(obj, *keys):
        return None if obj is None else {k: obj.get(k) for k in keys}

    # One line; the bulky per-leg objects come first and the compact figures last, so that a reader who
    # keeps only the end of the line still has every number the metric names.
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate, bf16 I/O", "data": "synthetic",
        "config": bench_config(B, T, H, N, args.path),
        "cfg2_forward": forward,
        "prefill_other_configs": prefill_other,
        "train": train,
        "streaming": streaming,
        "channel_mixer": channel_mixer,
        "lm_head_ce": lm_head,
        "decode": decode,
        "cfg4": cfg4,
        "host_copy": host_copy,
        "clocks": clocks,
        "gpu_launches": int(launches),
        "summary": {
            "prefill_cfg1": {"ms": kernel_ms, "tokens_per_s": value, "frac_of_hbm_peak": achieved / peak},
            "prefill_other": None if prefill_other is None else
                {k: {"ms": v["ms"], "frac_of_hbm_peak": v["frac_of_hbm_peak"]} for k, v in prefill_other.items()},
            "decode": pick(decode, "ms_per_step", "state_gb_per_s", "frac_of_hbm_peak", "tokens_per_s"),
            "lm_head_ce": pick(lm_head, "ms", "tflops", "frac_of_bf16_peak", "frac_of_bf16_sustained_peak"),
            "channel_mixer": pick(channel_mixer, "ms", "tflops", "frac_of_bf16_peak", "frac_of_bf16_sustained_peak"),
            "cfg2_forward": pick(forward, "ms", "tokens_per_s"),
            "train": pick(train, "forward_saved_ms", "forward_saved_frac_of_hbm_peak", "backward_ms",
                          "backward_frac_of_hbm_peak"),
            "streaming_frac_of_hbm_peak": None if streaming is None else
                {k: v["frac_of_hbm_peak"] for k, v in streaming.items() if isinstance(v, dict)},
            "cfg4": pick(cfg4, "wkv7_ms", "wkv7_frac_of_hbm_peak", "gather_ms", "lm_head_ms", "lm_head_frac_of_bf16_peak"),
            "host_copy": pick(host_copy, "h2d_gb_per_s_per_rank", "e2e_h2d_gb_per_s_per_rank", "e2e_bound"),
        },
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "timing": f"{e2e_steps} passes issued back to back from pinned host buffers, one device-timed "
                          "interval around all of them, only the last pass joined before the closing event "
                          "(a throughput figure, not the latency of one pass)"},
        "roofline": roofline,
    }
    if cpu is None:
        del out["cpu_baseline"]
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
