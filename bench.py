#!/usr/bin/env python
"""Benchmark of the attention forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one fused forward over the workload (default: causal GQA, B=8, Hq=32, Hkv=8,
S=4096, D=128, bf16).  Rank 0 prints ONE JSON line:

  value      effective TFLOP/s (unmasked pairs only) of the whole job, inputs resident in HBM,
             K steps back to back between one pair of CUDA events, max over ranks
  e2e        the same metric through the public variant API with HOST (pinned) tensors:
             host->device copies of q, k, v and the device->host copy of the result are inside
             the timed region of every step
  roofline   the attention kernel against the roof that bounds it, min(tensor, HBM): effective
             FLOPs (or compulsory bytes) per launch / mean launch duration from CUDA events
  workloads  (1 GPU) every benchmark configuration: time, TFLOP/s, the roof that bounds it and
             the fraction of it, plus the error against the fp32 oracle on a slice of the batch
  cpu_baseline  the reference's eager algorithm timed on this box's host cores on a bounded
             sample of the same workload (rank 0, 1 GPU only)

Several GPUs (torchrun, one rank per GPU): the FIXED workload is cut into contiguous slices of
its independent (batch, kv head) units (MSA rows for Evoformer), one slice per rank, placed on
the GPUs before timing: strong scaling.  There is no collective on the data path; NCCL carries
the start barrier and the max / sum of the timings.  `--impl reference` times the reference's
eager CPU implementation on the host cores and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "attention_fwd_effective_tflops"
UNIT = "TFLOP/s"
L2_BYTES = 126 * 1024 * 1024

# DRAM bytes (read + write) per launch of the attention kernel at the full size of the workload,
# from profiler captures of `dram__bytes_read.sum + dram__bytes_write.sum` on the workloads as they
# stand here (a capture of a smaller batch does not extrapolate: its working set sits in L2);
# None where no full-size capture exists.
NCU_TRAFFIC_BYTES = {
    "causal_gqa": 967e6, "softcap_causal": 718e6, "sliding_window": 782e6, "document_causal": 538e6,
    "evoformer": 190e6, "diff_attn": 470e6,
}


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="causal_gqa")
    ap.add_argument("--impl", default="flashlight_b200", choices=["flashlight_b200", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--batch", type=int, default=None,
                    help="override the workload's batch size (smaller cases for profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--no-workloads", action="store_true", help="skip the table of all workloads")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison in the workload table")
    ap.add_argument("--copy-ceiling", action="store_true",
                    help="measure what the platform gives N ranks copying the step's bytes in and out "
                         "of pinned host memory with no kernel, and print that instead")
    return ap.parse_args(argv)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json, burst)"
    return 1590.0, 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                clk, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            smax = mx
            if t0 - 0.05 <= ts <= t1 + 0.15:
                sm.append(clk)
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        if not sm:  # region shorter than the sampling period: fall back to all samples
            sm = [float(x[1].split(",")[1]) for x in self.lines if len(x[1].split(",")) >= 9]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, local, world


def bind_to_gpu_numa_node(local: int) -> str:
    """Pin this rank's threads to the CPUs next to its GPU (pinned host buffers are then allocated
    on that NUMA node and the copies do not cross sockets).  Best effort: says what it did."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (n_cpu + 63) // 64)
        cpus = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (wd >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return f"{len(cpus)} cpus near gpu {local}"
    except Exception as exc:  # no NVML, no permission: run unbound
        return f"unbound ({type(exc).__name__})"
    return "unbound"


# ------------------------------------------------------------------------------------------------
# reference arm and CPU baseline: the reference's own eager code when its compiled modules are
# present under oracle/_ref (see oracle/build_ref.py), else the oracle's restatement of it
# ------------------------------------------------------------------------------------------------
def cpu_runner(w):
    """Returns (fn(workload, tensors) -> output, kind) for the CPU legs."""
    from oracle.run_config import reference_runner, run_oracle
    ref = reference_runner(w)
    if ref is not None:
        return ref, "reference"
    return run_oracle, "port"


def cpu_sample(w, whole: bool):
    """The part of the workload one CPU step covers: all of it for the reference arm of the
    default workload (one sequence per call), a bounded slice elsewhere (seconds, not minutes)."""
    if w.variant == "vanilla":
        return w, "whole workload"
    if whole and w.variant == "causal":
        return w, f"whole workload, one of {w.N} sequences per call"
    if w.variant == "evoformer":
        n = min(w.N, 32)
        return w.scaled(N=n), f"{n} of {w.N} MSA rows"
    if w.variant == "document":
        heads = 4
        return w.scaled(Hq=heads, Hkv=heads), f"{heads} of {w.Hq} heads"
    return w.scaled(N=1), f"1 of {w.N} sequences (all heads)"


def run_cpu_step(fn, ws, t):
    """One CPU step; sequences go through the function one at a time to bound the fp32 scores."""
    if ws.variant in ("evoformer", "document") or ws.N == 1:
        return fn(ws, t)
    w1 = ws.scaled(N=1)
    for n in range(ws.N):
        fn(w1, {k: v[n:n + 1] for k, v in t.items()})


def reference_arm(args, rank, world):
    if rank != 0:
        return
    from flashlight_b200.workloads import WORKLOADS, effective_flops, make_inputs
    w = WORKLOADS[args.workload]
    if args.batch:
        w = w.scaled(N=args.batch)
    ws, sample = cpu_sample(w, whole=True)
    t = make_inputs(ws, seed=args.seed)
    flops = effective_flops(ws, t)
    torch.set_num_threads(os.cpu_count() or 1)
    fn, kind = cpu_runner(ws)
    for _ in range(args.warmup):
        run_cpu_step(fn, ws, t)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run_cpu_step(fn, ws, t)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    val = flops / dt / 1e12
    cores = torch.get_num_threads()
    what = "the reference's eager functions (compiled copies of its modules)" if kind == "reference" \
        else "oracle restatement of the reference's eager algorithm"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(w, world, note=f"CPU, {what}; per step: {sample}"),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(w, world, note=None):
    c = {"workload": w.name, "variant": w.variant, "batch": w.N, "q_heads": w.Hq, "kv_heads": w.Hkv,
         "seq_len": w.S, "head_dim": w.E, "v_head_dim": w.Ev, "causal": w.causal,
         "parallelism": (f"fixed workload cut into {world} contiguous slices of (batch, kv head) units, "
                         "no collective") if world > 1 else "one GPU"}
    c.update({k: v for k, v in w.extra.items()})
    if note:
        c["note"] = note
    return c


def reduce_over_ranks(ms: float, flops: float, dist, device) -> tuple:
    """Whole-job figures: the slowest rank's time and the work of all ranks (one all-reduce each)."""
    tm = torch.tensor([ms], dtype=torch.float64, device=device)
    fl = torch.tensor([flops], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(fl, op=dist.ReduceOp.SUM)
    return float(tm.item()), float(fl.item())


# ------------------------------------------------------------------------------------------------
# device-resident timing
# ------------------------------------------------------------------------------------------------
def device_copies(host_t, in_bytes):
    """Copies of the inputs on the device.  Inputs larger than L2 are their own flush; smaller ones
    are rotated over enough copies that twice the L2 lies between two uses of one copy."""
    n = 1 if in_bytes > L2_BYTES else min(64, math.ceil(2 * L2_BYTES / max(in_bytes, 1)) + 1)
    copies = [{k: v.cuda(non_blocking=True) for k, v in host_t.items()} for _ in range(n)]
    torch.cuda.synchronize()
    note = (f"inputs {in_bytes / 1e6:.0f} MB > L2 126 MB, no flush" if n == 1 else
            f"inputs {in_bytes / 1e6:.1f} MB < L2: steps rotate over {n} copies ({n * in_bytes / 1e6:.0f} MB)")
    return copies, note


def time_back_to_back(w, copies, steps, warmup, run_product, lib_count):
    """K forwards back to back between one event pair; returns (total ms, launches)."""
    out = None
    for i in range(warmup):
        out = run_product(w, copies[i % len(copies)])
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = lib_count()
    # A launch through Python costs tens of microseconds of host time.  The GPU first idles on a
    # spin kernel while the host queues all K launches, so that the events bracket K kernels
    # running back to back and not the host's launch rate (it matters for kernels below 0.1 ms).
    torch.cuda._sleep(int(2.0e6 * (0.5 + 0.1 * steps)))
    start.record()
    for i in range(steps):
        out = run_product(w, copies[i % len(copies)])
    end.record()
    torch.cuda.synchronize()
    del out
    return start.elapsed_time(end), lib_count() - n0


def time_per_launch(w, copies, steps, run_product, inside=None):
    """Duration of each of K launches from its own event pair (the kernel's figure for the roofline)."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    out = None
    for i, (a, b) in enumerate(evs):
        a.record()
        if inside is not None:
            inside()
        out = run_product(w, copies[i % len(copies)])
        b.record()
    torch.cuda.synchronize()
    del out
    return [a.elapsed_time(b) for a, b in evs]


def adjacent_rows(steps, peak_tf):
    """The operators either side of the forward variants, one line each: the backward pass at the default
    workload's shape (algorithmic FLOPs = 2.5 x the forward's: five matrix products for two), the product
    chain `(A @ B) @ C` at the reference's test shape (monkeypatch/template/fused_bmm.py:437-449) and
    invariant point attention at a structure module's sizes."""
    from flashlight_b200 import _lib, ops
    from flashlight_b200 import attention_variants as av
    from flashlight_b200.monkeypatch.template.fused_bmm import fused_bmm

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(int(2.0e6))
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    r = lambda *shape: torch.randn(*shape, device="cuda", dtype=torch.bfloat16)
    rows = {}
    N, Hq, Hkv, S, D = 8, 32, 8, 4096, 128
    q, k, v, dout = r(N, Hq, S, D), r(N, Hkv, S, D), r(N, Hkv, S, D), r(N, Hq, S, D)
    o, lse = ops.attn_fwd_lse(q, k, v, D ** -0.5, mask=_lib.MASK_CAUSAL)
    ms = timed(lambda: ops.attn_bwd(q, k, v, o, dout, lse, D ** -0.5, True))
    fl = 2.5 * 4 * D * N * Hq * (S * (S + 1) // 2)
    rows["backward_causal_gqa"] = {"shape": "B8 Hq32 Hkv8 S4096 D128 causal", "ms": ms, "flops": fl,
                                   "tflops": fl / ms / 1e9, "tensor_frac": fl / ms / 1e9 / peak_tf, "launches_per_step": 3}
    del q, k, v, dout, o, lse
    a, b, c = r(16, 4096, 128), r(16, 128, 4096), r(16, 4096, 128)
    ms = timed(lambda: fused_bmm(a, b, c))
    fl = 4.0 * 16 * 4096 * 4096 * 128
    rows["product_chain"] = {"shape": "b16 [4096,128]@[128,4096]@[4096,128]", "ms": ms, "flops": fl,
                             "tflops": fl / ms / 1e9, "tensor_frac": fl / ms / 1e9 / peak_tf, "launches_per_step": 1}
    del a, b, c
    B, H, Nr, C, Pq, Pv = 8, 12, 384, 16, 4, 8
    args = (r(B, H, Nr, C), r(B, H, Nr, C), r(B, H, Nr, C), r(B, H, Nr, Pq, 4), r(B, H, Nr, Pq, 4), r(B, H, Nr, Pv, 4),
            r(B, H, Nr, Nr))
    ms = timed(lambda: av.invariant_point_attention(*args, None, None, c_hidden=C, no_qk_points=Pq))
    fl = 2.0 * B * H * Nr * Nr * ((C + 4 * Pq) + (C + 4 * Pv))
    rows["invariant_point_attention"] = {"shape": "B8 H12 N384 C16 P_qk4 P_v8", "ms": ms, "flops": fl,
                                         "tflops": fl / ms / 1e9, "note": "operand assembly kernel + attention kernel",
                                         "launches_per_step": 2}
    return rows


def roof(flops, hbm_bytes, ms, peak_tf, peak_hbm):
    """The roof that bounds a launch, min(tensor, HBM), and the fraction of it that was reached."""
    t_tensor = flops / (peak_tf * 1e12)
    t_hbm = hbm_bytes / (peak_hbm * 1e9)
    tf = flops / (ms * 1e-3) / 1e12
    gbs = hbm_bytes / (ms * 1e-3) / 1e9
    if t_hbm > t_tensor:
        return {"bound": "hbm", "achieved": gbs, "peak": peak_hbm, "unit": "GB/s", "frac": gbs / peak_hbm,
                "tensor_frac": tf / peak_tf, "hbm_frac": gbs / peak_hbm}
    return {"bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf,
            "tensor_frac": tf / peak_tf, "hbm_frac": gbs / peak_hbm}


def parity_stats(w, dev_t, out, run_oracle):
    """Error of the kernel's result against the fp32 oracle evaluated on the device, on the first
    sequences (MSA rows) of the batch.  The oracle is the checker here, outside every timed region."""
    ws = w.scaled(N=min(w.N, 2))
    evo = w.variant == "evoformer"
    ts = {k: (v[:, :ws.N] if evo and v.size(1) == w.N else v if evo else v[:ws.N]) for k, v in dev_t.items()}
    ref = run_oracle(ws, ts)
    got = (out[:, :ws.N] if evo else out[:ws.N]).float()
    d = (got - ref.float()).abs()
    above = d > 2e-2
    n_above = int(above.sum())
    return {"max_abs": d.max().item(), "mean_abs": d.mean().item(), "n_above_2e-2": n_above,
            "largest_ref_above_2e-2": ref.float()[above].abs().max().item() if n_above else 0.0,
            "elements": d.numel(), "sample": f"first {ws.N} of {w.N} sequences"}


def copy_ceiling(args, rank, local, world, dist):
    """What the platform gives `world` ranks that each move their share of a step's bytes from and to
    pinned host memory at the same time, with no kernel in between: the ceiling of `e2e`."""
    from flashlight_b200.workloads import WORKLOADS, io_bytes, make_inputs, output_bytes, shard
    w_full = WORKLOADS[args.workload]
    w, host_t = shard(w_full, make_inputs(w_full, seed=args.seed), rank, world)
    in_b, out_b = io_bytes(w, host_t), output_bytes(w)
    src = torch.empty(in_b, dtype=torch.uint8).pin_memory()
    dst_h = torch.empty(out_b, dtype=torch.uint8).pin_memory()
    buf = torch.empty(in_b, dtype=torch.uint8, device="cuda")
    res = torch.empty(out_b, dtype=torch.uint8, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step():
        with torch.cuda.stream(s_in):
            buf.copy_(src, non_blocking=True)
        with torch.cuda.stream(s_out):
            dst_h.copy_(res, non_blocking=True)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    ms_max, bytes_all = reduce_over_ranks(ms, float(in_b + out_b), dist, "cuda")
    if rank == 0:
        print(json.dumps({"copy_ceiling": True, "n_gpus": world, "workload": w_full.name,
                          "ms_per_step": ms_max, "bytes_per_step_all_ranks": bytes_all,
                          "aggregate_gbs": bytes_all / (ms_max * 1e-3) / 1e9}), flush=True)


def main():
    args = parse_args()
    rank, local, world = dist_setup()
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import flashlight_b200
    from flashlight_b200.workloads import (WORKLOADS, effective_flops, hbm_bytes, io_bytes, make_inputs,
                                           output_bytes, run as run_product, shard)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    affinity = bind_to_gpu_numa_node(local) if world > 1 else "single rank"
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.copy_ceiling:
        copy_ceiling(args, rank, local, world, dist)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    w_full = WORKLOADS[args.workload]
    if args.batch:
        w_full = w_full.scaled(N=args.batch)
    peak_tf, peak_hbm, peak_src = load_peaks()

    # the fixed workload (same seed everywhere), this rank's contiguous slice of its units
    w, host_t = shard(w_full, make_inputs(w_full, seed=args.seed), rank, world)
    host_t = {k: v.pin_memory() for k, v in host_t.items()}
    flops = effective_flops(w, host_t)
    in_bytes = io_bytes(w, host_t)
    copies, resident_note = device_copies(host_t, in_bytes)
    warmup = max(args.warmup, 3)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)

    # ---- device-resident timing ----
    barrier()
    t_wall0 = time.time()
    total_ms, launches = time_back_to_back(w, copies, args.steps, warmup, run_product,
                                           flashlight_b200.launch_count)
    barrier()
    t_wall1 = time.time()
    flashlight_b200.check_status()
    per_launch = time_per_launch(w, copies, args.steps, run_product)
    region_ms_max, flops_all = reduce_over_ranks(total_ms, flops, dist, "cuda")
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

    # ---- end-to-end through the public API with host tensors ----
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(3):
            out_h = run_product(w, host_t)   # held across the next call, as in the timed loop
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(e2e_steps):
            out_h = run_product(w, host_t)     # H2D of q,k,v(+aux), kernel, D2H of the result
        e.record()
        barrier()
        e2e_ms, _ = reduce_over_ranks(s.elapsed_time(e) / e2e_steps, 0.0, dist, "cuda")
        assert out_h.device.type == "cpu"
        hb = torch.tensor([float(in_bytes), float(output_bytes(w))], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(hb)
        e2e = {"value": flops_all / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
               "ms_per_step": e2e_ms, "steps": e2e_steps,
               "h2d_bytes_per_step": int(hb[0].item()), "d2h_bytes_per_step": int(hb[1].item()),
               "host_gbs": (hb[0].item() + hb[1].item()) / (e2e_ms * 1e-3) / 1e9}

    # ---- every benchmark configuration (one GPU): time, roof, parity ----
    table = None
    if rank == 0 and world == 1 and not args.no_workloads:
        from oracle.run_config import run_oracle
        table = {}
        for name, wl in WORKLOADS.items():
            ht = make_inputs(wl, seed=args.seed)
            fl_w, by_w = effective_flops(wl, ht), hbm_bytes(wl, ht)
            cps, note = device_copies(ht, io_bytes(wl, ht))
            reps = max(args.steps, 10)
            ms_b2b, _ = time_back_to_back(wl, cps, reps, warmup, run_product, flashlight_b200.launch_count)
            pl = time_per_launch(wl, cps, reps, run_product)
            flashlight_b200.check_status()
            ms = ms_b2b / reps
            row = {"ms": ms, "ms_median_per_launch": statistics.median(pl), "tflops": fl_w / (ms * 1e-3) / 1e12,
                   "effective_flops": fl_w, "hbm_bytes": by_w, "traffic": NCU_TRAFFIC_BYTES.get(name), "l2": note}
            row.update(roof(fl_w, by_w, ms, peak_tf, peak_hbm))
            if wl.variant == "document":
                # the block map is cached per document_id tensor: also a step that rebuilds it
                pm = time_per_launch(wl, cps, reps, run_product, inside=flashlight_b200.clear_block_map_cache)
                row["ms_with_block_map_build"] = statistics.median(pm)
            if not args.no_parity:
                row["parity"] = parity_stats(wl, cps[0], run_product(wl, cps[0]), run_oracle)
            table[name] = row
            del cps

    adjacent = None
    if rank == 0 and world == 1 and not args.no_workloads:
        adjacent = adjacent_rows(max(3, min(args.steps, 10)), peak_tf)
        flashlight_b200.check_status()

    # ---- CPU baseline on a bounded sample ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ws, sample = cpu_sample(w_full, whole=False)
        ct = make_inputs(ws, seed=args.seed)
        torch.set_num_threads(os.cpu_count() or 1)
        fn, kind = cpu_runner(ws)
        t0 = time.perf_counter()
        run_cpu_step(fn, ws, ct)
        first = time.perf_counter() - t0
        reps = 1 if first > 10 else 2
        t0 = time.perf_counter()
        for _ in range(reps):
            run_cpu_step(fn, ws, ct)
        dt_cpu = (time.perf_counter() - t0) / reps
        cpu = {"value": effective_flops(ws, ct) / dt_cpu / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
               "kind": kind, "sample": sample, "seconds": dt_cpu}

    if rank == 0:
        kernel_ms = statistics.mean(per_launch)
        value = flops_all / (region_ms_max * 1e-3) * args.steps / 1e12
        rl = roof(flops, hbm_bytes(w, host_t), kernel_ms, peak_tf, peak_hbm)
        rl.update({"traffic": NCU_TRAFFIC_BYTES.get(w_full.name) if world == 1 and not args.batch else None,
                   "peak_source": peak_src, "kernel_ms": kernel_ms, "effective_flops_per_launch": flops,
                   "hbm_bytes_per_launch": hbm_bytes(w, host_t)})
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": region_ms_max / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": dict(workload_config(w_full, world), l2=resident_note, cpu_affinity=affinity),
            "per_gpu_tflops": value / world,
            "pct_of_bf16_peak": 100.0 * value / world / peak_tf,
            "roofline": rl,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if table is not None:
            line["workloads"] = table
        if adjacent is not None:
            line["adjacent_rows"] = adjacent
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
