#!/usr/bin/env python
"""Benchmark of the chunked HDLA operator, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg1|cfg0|cfg3]

One step = one forward + backward of the operator over one synthetic batch.  At N = 1 the
workload is B8 T4096 H16 K=V=128, bf16 inputs, fp32 accumulation/state, chunk 64 ("cfg1").  At
N > 1 (launched with torch.distributed.run, one rank per GPU) every rank processes its own cfg1
batch -- the (batch, head) pairs are independent, so the job shards with no collective on the
data path (weak scaling); ``--scaling strong`` shards the single cfg1 batch over the ranks instead.

The printed JSON line carries
  value / ms_per_step : tokens/s with the inputs resident in HBM, CUDA-event timed, max over ranks
  e2e                 : the same through the public entry point with pinned HOST buffers, the
                        host->device copies of all inputs and device->host copies of o and all
                        gradients inside the timed region
  roofline            : algorithmic FLOPs of one step / measured step time against the measured
                        bf16 tensor peak (MEASURED_PEAKS.json), with the HBM view beside it
  cpu_baseline        : the CPU oracle (a port of the reference algorithm) timed on this host
  clocks              : SM clocks and throttle reasons sampled with nvidia-smi during the timed region

``--impl reference`` times the reference algorithm's CPU implementation (the oracle port of
HRDPLR/naive.py plus explicit backward; the reference itself ships Triton-only kernels and a
torch "naive" path, and its checkout is not available on the GPU host) on all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "HDLA fwd+bwd tokens/s (B8 T4096 H16 D128 bf16)"
WORKLOADS = {
    # name: (B, T, H, K, V, C, dtype)
    "cfg1": (8, 4096, 16, 128, 128, 64, "bf16"),
    "cfg0": (2, 256, 4, 64, 64, 64, "f32"),
    # profiling case: cfg 1 with a quarter of the batch (inputs still larger than L2, ~2 GB on the device)
    "cfg1_small": (2, 4096, 16, 128, 128, 64, "bf16"),
    "cfg3": (1, 65536, 16, 128, 128, 64, "bf16"),
    # one layer of the 24-layer stack of cfg 4 (B32 sharded over the GPUs by batch): operator only
    "cfg4": (32, 4096, 16, 128, 128, 64, "bf16"),
    # decode: B sequences, one token per step, carried fp32 state [B,H,K,V]; T is unused
    "cfg2": (256, 1, 32, 128, 128, 0, "bf16"),
}
DECODE_METRIC = "HDLA fused-recurrent decode tokens/s (B256 H32 D128 bf16, fp32 state)"
R = 2
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# ------------------------------------------------------------------------------ work per unit
def macs_per_chunk_head(C: int, D: int) -> float:
    """Dense tile products of the algorithm per (chunk, head), no recompute, masked products dense."""
    fwd = 9 * C * C * D + (2 * C) ** 3 / 3 + 4 * C ** 3 + 4 * C * C * D + 2 * C * C * D + 5 * C * D * D \
        + (C * D * D + 3 * C * C * D)
    bwd = 5 * C * C * D + 5 * C * D * D + (C * D * D + C * C * D) + 6 * C * D * D + (28 * C ** 3 + 12 * C * C * D) \
        + 18 * C * C * D
    return fwd + bwd


def flops_per_token_head(C: int, D: int) -> float:
    return 2.0 * macs_per_chunk_head(C, D) / C


def bytes_per_token_head(C: int, D: int, elt: int) -> float:
    """Minimal HBM traffic: fwd reads 8D writes D; bwd reads 9D writes 8D; state checkpoints
    (K*V*2 bytes per chunk) written and read once each for S and dS."""
    return (8 * D + D) * elt + (9 * D + 8 * D) * elt + 4 * (D * D * 2 / C)


# Algorithmic HBM bytes per (chunk, head) of each kernel of the bf16 pipeline: every operand tile it
# needs read once, every result written once (KiB; bf16 tiles and un-gating factors, fp32 E; K = V = 128, chunk 64, R = 2).
# scan_tc_kernel is launched twice per step (forward 192.5, reverse 225).
KERNEL_KIB = {
    "prep_hat_kernel": 256.5, "gram_tc_kernel": 168.0, "inverse_tc_kernel": 64.0, "wu_tc_kernel": 192.0,
    "scan_tc_kernel": (192.5 + 225.0) / 2, "out_tc_kernel": 136.0, "dau_tc_kernel": 152.0,
    "wy_bwd_tc_kernel": 288.0, "grad_tc_kernel": 560.5,
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch (GB) at cfg 1: one ncu capture at B=2 (a quarter of
# cfg 1; traffic is proportional to the number of chunks), scaled by 4 -- see profiles/chunk_tc_pipeline_traffic.md
KERNEL_NCU_TRAFFIC_GB = {
    "prep_hat_kernel": 2.09, "gram_tc_kernel": 1.20, "inverse_tc_kernel": 0.33, "wu_tc_kernel": 1.39,
    "scan_tc_kernel": (1.51 + 1.79) / 2, "out_tc_kernel": 1.08, "dau_tc_kernel": 1.06, "wy_bwd_tc_kernel": 2.25,
    "grad_tc_kernel": 4.62,
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------ CPU oracle timing
def time_cpu_port(T_sample: int, H: int, K: int, V: int, C: int, repeats: int = 1):
    """Forward + explicit backward of the oracle port in fp32 on all host threads; tokens/s."""
    from oracle import hdla_oracle as orc
    from hdla_impl_b200.synthetic import make_inputs
    torch.set_num_threads(os.cpu_count() or 1)
    x = make_inputs(1, T_sample, H, K, V, R, seed=0)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        st = orc.staged_forward(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, K ** -0.5, None, C,
                                dtype=torch.float32)
        orc.staged_backward(st, x["do"], None)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return T_sample / best, best


def run_reference(args, rank, world):
    if rank != 0:
        return
    B, T, H, K, V, C, dt = WORKLOADS[args.workload]
    T_s = min(T, 256)
    times = []
    for i in range(args.warmup + args.steps):
        _, sec = time_cpu_port(T_s, H, K, V, C)
        if i >= args.warmup:
            times.append(sec)
    total = sum(times)
    val = T_s * args.steps / total
    cores = os.cpu_count() or 1
    sample = f"B=1 T={T_s} of {args.workload} (H={H} K={K} V={V} chunk {C}), fp32, per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "T": T, "H": H, "K": K, "V": V, "chunk": C, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ our arm
def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    import hdla_impl_b200 as HD
    from hdla_impl_b200 import _lib
    from hdla_impl_b200.sharding import shard_batch_heads
    from hdla_impl_b200.synthetic import make_inputs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, T, H, K, V, C, dt = WORKLOADS[args.workload]
    dtype = torch.bfloat16 if dt == "bf16" else torch.float32
    elt = 2 if dt == "bf16" else 4

    # this rank's units
    cp = args.workload == "cfg3" and world > 1           # long context: shard T, exchange boundary states
    if args.workload == "cfg4":
        args.scaling = "strong"                          # one B32 batch, sharded by batch over the ranks
    if cp:
        args.scaling = "strong"
    Tl = T // world if cp else T
    if cp:
        Bl, Hl = B, H
    elif args.scaling == "strong" and world > 1:
        b_lo, b_hi, h_lo, h_hi = shard_batch_heads(B, H, rank, world)
        Bl, Hl = b_hi - b_lo, h_hi - h_lo
    else:
        Bl, Hl = B, H
    x = make_inputs(Bl, Tl, Hl, K, V, R, seed=rank, dtype=dtype)
    names = ("q", "k", "v", "a", "b", "gk")
    from hdla_impl_b200.host import numa_local_to
    with numa_local_to(dev):                             # pinned buffers on the GPU's own NUMA node
        host = {n: x[n].pin_memory() for n in names + ("do",)}
    dev_in = {n: host[n].to(dev) for n in host}
    leaves = [dev_in[n].requires_grad_(True) for n in names]
    scale = K ** -0.5

    from hdla_impl_b200.context_parallel import cp_chunk_hrdplr_delta_rule

    def step(lv, do):
        if cp:
            o, _ = cp_chunk_hrdplr_delta_rule(*lv, R, scale=scale, chunk_size=C)
        else:
            o, _ = HD.chunk_hrdplr_delta_rule(*lv, R, scale=scale, chunk_size=C)
        grads = torch.autograd.grad(o, lv, do)
        return o, grads

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(leaves, dev_in["do"])
    barrier()
    l0 = _lib.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step(leaves, dev_in["do"])
    e1.record()
    barrier()
    launches = _lib.kernel_launches() - l0
    ms = e0.elapsed_time(e1)
    # per-kernel durations, live: the library brackets every launch with CUDA events on its stream
    ktimes = {}
    if rank == 0 or cp:                                  # with context parallelism every step is collective
        if rank == 0:
            _lib.timing_enable(True)
        for _ in range(3):
            step(leaves, dev_in["do"])
        torch.cuda.synchronize(dev)
        if rank == 0:
            _lib.timing_enable(False)
            ktimes = _lib.timing_report()
    if rank == 0 and not cp:
        # the timed region can be shorter than nvidia-smi's sampling period: keep the same load running
        # (untimed) until a few samples exist, so the clocks reported are clocks under this load
        t_end = time.time() + 5.0
        while len(sampler.rows) < 5 and time.time() < t_end:
            step(leaves, dev_in["do"])
            torch.cuda.synchronize(dev)
    elif cp:
        for _ in range(20):                              # same number of collective steps on every rank
            step(leaves, dev_in["do"])
        torch.cuda.synchronize(dev)
    clocks = sampler.stop() if rank == 0 else None

    # end to end: pinned host buffers in, host buffers out, through the package's host-tensor entry point
    # (slices of the batch pipelined over copy-in / compute / copy-out streams)
    from hdla_impl_b200.host import chunk_fwd_bwd_from_host
    out_host = {}
    e2e_steps = args.steps

    def e2e_step():
        if cp:                                           # sequence-sharded: one slice, collective step
            lv = [host[n].to(dev, non_blocking=True).requires_grad_(True) for n in names]
            do = host["do"].to(dev, non_blocking=True)
            o, grads = step(lv, do)
            outs = (o,) + tuple(grads)
            for i, t in enumerate(outs):
                if i not in out_host:
                    out_host[i] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                out_host[i].copy_(t, non_blocking=True)
        else:
            # enqueue only: successive steps stream through the copy engines (the copy-in of step s+1 runs under
            # the copy-out of step s); the clock stops after the last copy-out has completed
            chunk_fwd_bwd_from_host(host, out_host, R, dev, scale=scale, chunk_size=C, slice_batch=1, sync=False)

    with numa_local_to(dev) as numa:
        e2e_step()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(e2e_steps):
            e2e_step()
        f1.record()
        barrier()
        ms_e2e = f0.elapsed_time(f1)
    numa_node = numa.node
    h2d = sum(host[n].numel() * host[n].element_size() for n in host)
    d2h = sum(t.numel() * t.element_size() for t in out_host.values())

    if world > 1:
        tt = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()
    tokens_step = B * T * (world if args.scaling == "weak" else 1)
    ms_step = ms / args.steps
    value = tokens_step / (ms_step / 1e3)
    e2e_val = tokens_step / (ms_e2e / e2e_steps / 1e3)

    if rank == 0:
        peaks, how = load_peaks()
        heads_tokens = tokens_step * H / world            # per-GPU token-heads per step
        flops = heads_tokens * flops_per_token_head(C, K)
        byts = heads_tokens * bytes_per_token_head(C, K, elt)
        sec = ms_step / 1e3
        tf = flops / sec / 1e12
        gbs = byts / sec / 1e9
        peak_tf = peaks.get("bf16_tflops_sustained") or peaks.get("bf16_tflops")
        roof = {
            "bound": "tensor", "kernel": "chunked fwd+bwd pipeline (all launches of one step)",
            "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf, "traffic": None,
            "peak_source": f"{how} (bf16 sustained)", "flops_per_launch": flops,
            "hbm": {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                    "algorithmic_bytes": byts},
        }
        if ktimes and dt == "bf16":
            G = (B if (args.scaling == "weak" or cp) else B // world) * H * ((Tl + C - 1) // C)
            tot = sum(v[1] for v in ktimes.values())
            table = {}
            for name, (cnt, tms) in sorted(ktimes.items(), key=lambda kv: -kv[1][1]):
                avg = tms / cnt
                kib = KERNEL_KIB.get(name)
                table[name] = {"launches_per_step": cnt // 3, "avg_ms": avg, "share": tms / tot,
                               "algorithmic_GBps": (kib * 1024 * G / (avg / 1e3) / 1e9) if kib else None}
            top = next(iter(table))
            if KERNEL_KIB.get(top):
                a = table[top]["algorithmic_GBps"]
                roof = {
                    "bound": "hbm", "kernel": top, "achieved": a, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": a / peaks["hbm_gbs"], "traffic": KERNEL_NCU_TRAFFIC_GB.get(top),
                    "peak_source": f"{how} (copy)", "avg_launch_ms": table[top]["avg_ms"],
                    "algorithmic_bytes_per_launch": KERNEL_KIB[top] * 1024 * G,
                    "step": {"tensor": {"achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf,
                                        "flops_per_step": flops},
                             "hbm": {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                     "frac": gbs / peaks["hbm_gbs"], "algorithmic_bytes_per_step": byts}},
                    "kernels": table,
                }
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            T_s = min(T, 1024)
            val, sec_cpu = time_cpu_port(T_s, H, K, V, C)
            cpu = {"value": val, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                   "sample": f"B=1 T={T_s} of {args.workload} (H={H} K={K} V={V} chunk {C}) fp32, one pass, "
                             f"{sec_cpu:.1f} s"}
        line = {
            "metric": METRIC if args.workload == "cfg1" else
            f"HDLA fwd+bwd tokens/s (B{B} T{T} H{H} D{K} {dt})", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": args.workload, "B_per_step": B * (world if args.scaling == "weak" else 1), "T": T,
                       "H": H, "K": K, "V": V, "R": R, "chunk": C,
                       "sharding": ("context parallel: T/N per rank, all-gather of affine state maps (NCCL)" if cp
                                    else "batch x head, no collective"),
                       "backward": "saved forward intermediates" if HD.hrdplr.save_workspace_default() else "recompute",
                       "l2": "inputs (>1 GB per step) are larger than the 126 MB L2"},
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "host_numa_node": numa_node},
            "gpu_launches": int(launches), "roofline": roof, "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode(args, rank, world, local_rank):
    """cfg2: one token per sequence per step, state read-modify-write in HBM (bandwidth bound)."""
    import torch.distributed as dist
    import hdla_impl_b200 as HD
    from hdla_impl_b200 import _lib
    from hdla_impl_b200.synthetic import make_inputs
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, _, H, K, V, _, dt = WORKLOADS["cfg2"]
    steps, warm = args.steps, max(args.warmup, 3)
    ntok = 16                                            # distinct token inputs, cycled
    x = make_inputs(B, ntok, H, K, V, R, seed=rank, dtype=torch.bfloat16, h0_std=0.02)
    names = ("q", "k", "v", "a", "b", "gk")
    host = {n: x[n].pin_memory() for n in names}
    dv = {n: host[n].to(dev) for n in names}
    S = x["h0"].to(dev)
    scale = K ** -0.5

    def tok(src, t, n, r=1):
        return src[n][:, (t % ntok) * r:(t % ntok + 1) * r]

    def step(src, t):
        nonlocal S
        o, S = HD.fused_recurrent_dplr_delta_rule_fwd(tok(src, t, "q"), tok(src, t, "k"), tok(src, t, "v"),
                                                      tok(src, t, "a", R), tok(src, t, "b", R), tok(src, t, "gk"), R,
                                                      scale, S, True, inplace_state=True)
        return o

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for t in range(warm):
        step(dv, t)
    barrier()
    l0 = _lib.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for t in range(steps):
        step(dv, t)
    e1.record()
    barrier()
    launches = _lib.kernel_launches() - l0
    ms = e0.elapsed_time(e1)
    if rank == 0:
        t_end = time.time() + 5.0
        while len(sampler.rows) < 5 and time.time() < t_end:
            step(dv, 0)
            torch.cuda.synchronize(dev)
    clocks = sampler.stop() if rank == 0 else None
    # end to end: this step's token tensors come from pinned host memory, o goes back to the host
    o_host = torch.empty(B, 1, H, V, dtype=torch.bfloat16, pin_memory=True)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    f0.record()
    for t in range(steps):
        cur = {n: tok(host, t, n, R if n in ("a", "b") else 1).contiguous().to(dev, non_blocking=True) for n in names}
        o, S2 = HD.fused_recurrent_dplr_delta_rule_fwd(cur["q"], cur["k"], cur["v"], cur["a"], cur["b"], cur["gk"], R,
                                                       scale, S, True, inplace_state=True)
        o_host.copy_(o, non_blocking=True)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    h2d = B * H * (7 * K + V) * 2
    d2h = B * H * V * 2
    if world > 1:
        tt = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()
    if rank == 0:
        peaks, how = load_peaks()
        sec = ms / steps / 1e3
        byts = 2.0 * B * H * K * V * 4 + B * H * (7 * K + 2 * V) * 2      # state read+write, token I/O
        gbs = byts / sec / 1e9
        line = {
            "metric": DECODE_METRIC, "value": B * world / sec, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg2", "sequences_per_gpu": B, "H": H, "K": K, "V": V, "R": R,
                       "state": "fp32 [B,H,K,V] carried in HBM, updated in place",
                       "l2": "state (537 MB) is larger than the 126 MB L2"},
            "e2e": {"value": B * world / (ms_e2e / steps / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "recurrent_bulk_kernel", "achieved": gbs, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": f"{how} (copy)", "algorithmic_bytes": byts},
            "cpu_baseline": None, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "cfg2" and args.impl == "ours":
        if args.steps == 10:
            args.steps = 128
        run_decode(args, rank, world, local_rank)
    elif args.impl == "reference":
        if args.workload == "cfg2":
            args.workload = "cfg1"
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
