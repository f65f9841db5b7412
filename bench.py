#!/usr/bin/env python
"""Benchmark of the chunked HDLA operator, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg1|...]

One step = one forward + backward of the operator over one synthetic batch.  The workload is
B8 T4096 H16 K=V=128, bf16 inputs, fp32 accumulation/state, chunk 64 ("cfg1").  At N > 1 (launched
with torch.distributed.run, one rank per GPU) that ONE batch is sharded over the ranks by
(batch, head) pairs -- they are independent, so there is no collective on the data path -- and the
line reports ``"scaling": "strong"``; ``--scaling weak`` gives every rank its own cfg1 batch instead
(also reported under ``secondary.weak``).

The printed JSON line carries
  value / ms_per_step : tokens/s with the inputs resident in HBM, CUDA-event timed, max over ranks
  e2e                 : the same through the package's host-tensor entry point with pinned HOST buffers,
                        the host->device copies of all inputs and device->host copies of o and all
                        gradients inside the timed region
  roofline            : whole-step fractions -- the minimal HBM traffic of one step (8704 B per token
                        and head) / step time against the measured copy bandwidth, the algorithmic FLOPs
                        against the measured bf16 peak -- and, under ``kernels``, every kernel's own
                        CUDA-event time with the bytes the PIPELINE moves through it
  cpu_baseline        : the reference's own CPU implementation (HRDPLR/naive.py, installed under
                        oracle/_ref by oracle/install_ref.py; else the oracle port) on a bounded sample
  secondary           : decode (cfg2) and the fp32 CPU configuration (cfg0) on the GPU; at N > 1 the
                        weak-scaling number, the long-context configuration (cfg3) with context
                        parallelism, and ``cp_check``, the parity of the context-parallel path against
                        the single-GPU operator on the same inputs
  clocks              : SM clocks and throttle reasons sampled with nvidia-smi during the timed region

``--impl reference`` times that CPU implementation alone (rank 0; the other ranks exit).
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
    # what one GPU holds of cfg 1 when the batch is sharded over 2 / 8 GPUs (for profiling the sharded case on one GPU)
    "cfg1_shard2": (4, 4096, 16, 128, 128, 64, "bf16"),
    "cfg1_shard8": (1, 4096, 16, 128, 128, 64, "bf16"),
    "cfg3": (1, 65536, 16, 128, 128, 64, "bf16"),
    # one layer of the 24-layer stack of cfg 4 (B32 sharded over the GPUs by batch): operator only
    "cfg4": (32, 4096, 16, 128, 128, 64, "bf16"),
    # decode: B sequences, one token per step, carried fp32 state [B,H,K,V]; T is unused
    "cfg2": (256, 1, 32, 128, 128, 0, "bf16"),
}
DECODE_METRIC = "HDLA fused-recurrent decode tokens/s (B256 H32 D128 bf16, fp32 state)"
R = 2
NAMES = ("q", "k", "v", "a", "b", "gk")
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


# Bytes the PIPELINE moves through each kernel per (chunk, head): every operand tile the kernel reads, read once,
# every result it writes, written once -- inter-kernel intermediates included, which is why their sum is a multiple
# of the algorithmic minimum above (KiB; bf16 tiles and un-gating factors, fp32 E; K = V = 128, chunk 64, R = 2).
# scan_tc_kernel is launched twice per step (forward 192.5, reverse 225).
KERNEL_KIB = {
    "chunk_prep_tc_kernel": 424.5,
    "prep_hat_kernel": 256.5, "gram_tc_kernel": 168.0, "inverse_tc_kernel": 64.0, "wu_tc_kernel": 192.0,
    "scan_tc_kernel": (192.5 + 225.0) / 2, "out_tc_kernel": 136.0, "dau_tc_kernel": 152.0,
    "wy_bwd_tc_kernel": 288.0, "grad_tc_kernel": 560.5,
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch (GB) at cfg 1: one ncu capture at B=2 (a quarter of
# cfg 1; traffic is proportional to the number of chunks), scaled by 4 -- see profiles/
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


# ------------------------------------------------------------------------------ CPU reference timing
def cpu_reference_pass(H: int, K: int, V: int, C: int, T_sample: int, B_sample: int = 1, repeats: int = 1):
    """One sample definition for every CPU number this file prints: forward + backward in fp32 on all host
    threads over B_sample x T_sample tokens of the workload's head shape.  The reference's own naive.py
    (autograd backward, as its test_integrated.py does) when it is installed under oracle/_ref, else the oracle
    port (explicit backward).  Returns (tokens/s, seconds of the best pass, kind)."""
    from hdla_impl_b200.synthetic import make_inputs
    torch.set_num_threads(os.cpu_count() or 1)
    x = make_inputs(B_sample, T_sample, H, K, V, R, seed=0)
    from oracle import ref_naive
    sec = None
    if ref_naive.available():
        try:
            sec = ref_naive.time_fwd_bwd(x, R, C, repeats=repeats)
            kind = "reference"
        except Exception as e:                           # noqa: BLE001  (e.g. one of naive.py's imports is missing)
            print(f"bench: oracle/_ref/naive.py could not run ({type(e).__name__}: {e}); timing the oracle port",
                  file=sys.stderr)
    if sec is None:
        from oracle import hdla_oracle as orc
        sec = None
        for _ in range(repeats):
            t0 = time.perf_counter()
            st = orc.staged_forward(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, K ** -0.5, None, C,
                                    dtype=torch.float32)
            orc.staged_backward(st, x["do"], None)
            dt = time.perf_counter() - t0
            sec = dt if sec is None else min(sec, dt)
        kind = "port"
    return B_sample * T_sample / sec, sec, kind


def cpu_baseline_block(workload: str):
    """cpu_baseline of the JSON line: a bounded sample of the benchmark's own workload, best of 3, plus the
    CPU configuration (cfg0, B2 T256 H4 K=V=64) in full."""
    B, T, H, K, V, C, dt = WORKLOADS[workload]
    T_s = min(T, 512)
    val, sec, kind = cpu_reference_pass(H, K, V, C, T_s, 1, repeats=3)
    B0, T0, H0, K0, V0, C0, _ = WORKLOADS["cfg0"]
    val0, sec0, _ = cpu_reference_pass(H0, K0, V0, C0, T0, B0, repeats=3)
    what = "HRDPLR/naive.py (reference, autograd backward)" if kind == "reference" else "oracle port of HRDPLR/naive.py"
    return {"value": val, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": kind,
            "sample": f"{what}: B=1 T={T_s} of {workload} (H={H} K={K} V={V} chunk {C}) fp32 fwd+bwd, "
                      f"best of 3 passes, {sec:.2f} s per pass",
            "cfg0": {"value": val0, "unit": "tokens/s", "seconds_per_pass": sec0,
                     "sample": f"B={B0} T={T0} H={H0} K=V={K0} fp32 chunk {C0}, whole configuration, best of 3"}}


def run_reference(args, rank, world):
    if rank != 0:
        return
    wl = "cfg1" if args.workload == "cfg2" else args.workload
    B, T, H, K, V, C, dt = WORKLOADS[wl]
    T_s = min(T, 256)
    times, kind = [], "port"
    for i in range(args.warmup + args.steps):
        _, sec, kind = cpu_reference_pass(H, K, V, C, T_s, 1, repeats=1)
        if i >= args.warmup:
            times.append(sec)
    total = sum(times)
    val = T_s * args.steps / total
    cores = os.cpu_count() or 1
    what = "HRDPLR/naive.py (reference, autograd backward)" if kind == "reference" else "oracle port of HRDPLR/naive.py"
    sample = f"{what}: B=1 T={T_s} of {wl} (H={H} K={K} V={V} chunk {C}) fp32 fwd+bwd per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "B": B, "T": T, "H": H, "K": K, "V": V, "chunk": C, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ helpers of our arm
def timed_steps(step, steps, barrier):
    """K steps bracketed by barrier + synchronize on both sides; CUDA-event milliseconds of this rank."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    return e0.elapsed_time(e1)


def kernel_table(ktimes, passes, G):
    """Per-kernel CUDA-event times of `passes` steps -> table with the pipeline bytes each kernel moves."""
    tot = sum(v[1] for v in ktimes.values())
    table = {}
    for name, (cnt, tms) in sorted(ktimes.items(), key=lambda kv: -kv[1][1]):
        avg = tms / cnt
        kib = KERNEL_KIB.get(name)
        table[name] = {"launches_per_step": cnt / passes, "avg_ms": avg, "ms_per_step": tms / passes,
                       "share": tms / tot if tot else None,
                       "pipeline_KiB_per_chunk_head": kib,
                       "pipeline_GBps": (kib * 1024 * G / (avg / 1e3) / 1e9) if kib else None,
                       "ncu_dram_GB_per_launch_cfg1": KERNEL_NCU_TRAFFIC_GB.get(name)}
    return table


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    import hdla_impl_b200 as HD
    from hdla_impl_b200 import _lib
    from hdla_impl_b200.context_parallel import cp_chunk_hrdplr_delta_rule
    from hdla_impl_b200.host import chunk_fwd_bwd_from_host, join_host_streams, numa_local_to
    from hdla_impl_b200.sharding import shard_batch_heads, shard_time
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
    scale = K ** -0.5

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def op_step(lv, do, use_cp=False):
        if use_cp:
            o, _ = cp_chunk_hrdplr_delta_rule(*lv, R, scale=scale, chunk_size=C)
        else:
            o, _ = HD.chunk_hrdplr_delta_rule(*lv, R, scale=scale, chunk_size=C)
        return o, torch.autograd.grad(o, lv, do)

    # ---- this rank's units
    cp = args.workload == "cfg3" and world > 1           # long context: shard T, exchange boundary states
    scaling = args.scaling
    if cp or args.workload == "cfg4":
        scaling = "strong"
    if cp:
        Bl, Hl, Tl = B, H, T // world
    elif scaling == "strong" and world > 1:
        b_lo, b_hi, h_lo, h_hi = shard_batch_heads(B, H, rank, world)
        Bl, Hl, Tl = b_hi - b_lo, h_hi - h_lo, T
    else:
        Bl, Hl, Tl = B, H, T
    x = make_inputs(Bl, Tl, Hl, K, V, R, seed=rank, dtype=dtype)
    with numa_local_to(dev) as numa:                     # pinned buffers on the GPU's own NUMA node
        host = {n: x[n].pin_memory() for n in NAMES + ("do",)}
    dev_in = {n: host[n].to(dev) for n in host}
    leaves = [dev_in[n].requires_grad_(True) for n in NAMES]
    step = lambda: op_step(leaves, dev_in["do"], cp)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    l0 = _lib.kernel_launches()
    ms = timed_steps(step, args.steps, barrier)
    launches = _lib.kernel_launches() - l0
    # per-kernel durations, live: the library brackets every launch with CUDA events on its stream
    ktimes, kpasses = {}, 3
    if rank == 0:
        _lib.timing_enable(True)
    for _ in range(kpasses):                             # (with context parallelism every step is collective)
        step()
    torch.cuda.synchronize(dev)
    if rank == 0:
        _lib.timing_enable(False)
        ktimes = _lib.timing_report()
    # the timed region can be shorter than nvidia-smi's sampling period: keep the same load running (untimed)
    # until a few samples exist, so the clocks reported are clocks under this load
    for _ in range(60 if world > 1 else 400):
        if world == 1 and len(sampler.rows) >= 5:
            break
        step()
        if world == 1:
            torch.cuda.synchronize(dev)
    torch.cuda.synchronize(dev)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: pinned host buffers in, host buffers out, through the package's host-tensor entry point
    # (slices of the batch pipelined over copy-in / compute / copy-out streams; successive steps only enqueue, so
    # the copy-in of step s+1 runs under the copy-out of step s; the clock stops after the last copy-out)
    out_host = {}

    def e2e_step():
        if cp:                                           # sequence-sharded: one slice, collective step
            lv = [host[n].to(dev, non_blocking=True).requires_grad_(True) for n in NAMES]
            do = host["do"].to(dev, non_blocking=True)
            o, grads = op_step(lv, do, True)
            for i, t in enumerate((o,) + tuple(grads)):
                if i not in out_host:
                    out_host[i] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                out_host[i].copy_(t, non_blocking=True)
        else:
            # slices of up to four batch elements: while the kernels of a slice run, the copies of its neighbours
            # proceed at about half their rate (measured), so fewer and larger kernels cost the link less
            chunk_fwd_bwd_from_host(host, out_host, R, dev, scale=scale, chunk_size=C, slice_batch=4, sync=False)

    with numa_local_to(dev):
        e2e_step()
        torch.cuda.synchronize(dev)
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        f0.record()
        for _ in range(args.steps):
            e2e_step()
        if not cp:
            join_host_streams(dev)
        f1.record()
        barrier()
        ms_e2e = f0.elapsed_time(f1)
    h2d = sum(host[n].numel() * host[n].element_size() for n in host)
    d2h = sum(t.numel() * t.element_size() for t in out_host.values())

    if world > 1:
        tt = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()
    tokens_step = B * T * (world if scaling == "weak" else 1)
    ms_step = ms / args.steps
    value = tokens_step / (ms_step / 1e3)
    e2e_val = tokens_step / (ms_e2e / args.steps / 1e3)

    # ---- secondary measurements (all ranks take part in the collective ones)
    secondary = {}
    if not args.no_secondary and args.workload == "cfg1":
        del leaves, dev_in, host, out_host, x
        torch.cuda.empty_cache()

        def record(name, fn):
            # a secondary measurement must not take the headline line down with it (collective ones are entered by
            # every rank in the same order, so a failure on one rank fails them all at the same call)
            try:
                secondary[name] = fn()
            except Exception as e:                       # noqa: BLE001
                secondary[name] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        record("host_link", lambda: bench_host_link(dev, world, barrier))
        if world > 1:
            record("cp_check", lambda: cp_parity_check(dev, rank, world))
            record("cfg3", lambda: bench_cfg3(dev, rank, world, barrier))
            if scaling == "strong":
                record("weak", lambda: bench_weak(dev, rank, world, barrier))
        else:
            record("cfg3", lambda: bench_cfg3(dev, rank, world, barrier))
            record("cfg2_decode", lambda: bench_decode_small(dev))
            record("cfg0_fp32_gpu", lambda: bench_cfg0_gpu(dev))
            record("layer_call", lambda: bench_layer_call(dev))

    if rank == 0:
        peaks, how = load_peaks()
        heads_tokens = tokens_step * H / world            # per-GPU token-heads per step
        flops = heads_tokens * flops_per_token_head(C, K)
        byts = heads_tokens * bytes_per_token_head(C, K, elt)
        sec = ms_step / 1e3
        tf = flops / sec / 1e12
        gbs = byts / sec / 1e9
        peak_tf = peaks.get("bf16_tflops_sustained") or peaks.get("bf16_tflops")
        G = Bl * Hl * ((Tl + C - 1) // C)
        table = kernel_table(ktimes, kpasses, G) if (ktimes and dt == "bf16") else {}
        pipeline_kib = sum(v["pipeline_KiB_per_chunk_head"] * v["launches_per_step"] for v in table.values()
                           if v["pipeline_KiB_per_chunk_head"])
        alg_kib = bytes_per_token_head(C, K, elt) * C / 1024.0
        roof = {
            "bound": "hbm", "kernel": "all launches of one fwd+bwd step",
            "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
            "traffic": None,
            "peak_source": f"{how} (copy)",
            "algorithmic_bytes_per_step": byts,
            "algorithmic_KiB_per_chunk_head": alg_kib,
            "pipeline_KiB_per_chunk_head": pipeline_kib or None,
            "traffic_over_algorithmic": (pipeline_kib / alg_kib) if pipeline_kib else None,
            "tensor": {"achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf,
                       "flops_per_step": flops, "peak_source": f"{how} (bf16 sustained)",
                       "frac_of_burst_peak": tf / peaks["bf16_tflops"] if peaks.get("bf16_tflops") else None},
            "kernels_note": "per-kernel CUDA-event times of rank 0 with PIPELINE bytes (they include the "
                            "inter-kernel intermediates); event bracketing removes launch overlap, so their "
                            "sum can exceed ms_per_step slightly",
            "kernels": table,
        }
        ncu_total = sum((v["ncu_dram_GB_per_launch_cfg1"] or 0) * v["launches_per_step"] for v in table.values())
        if ncu_total and args.workload == "cfg1" and (world == 1 or scaling == "weak"):
            roof["traffic"] = ncu_total                   # GB per step, summed over the kernels' ncu captures
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline_block(args.workload)
        line = {
            "metric": METRIC if args.workload == "cfg1" else
            f"HDLA fwd+bwd tokens/s (B{B} T{T} H{H} D{K} {dt})", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": args.workload, "B_per_step": B * (world if scaling == "weak" else 1), "T": T,
                       "H": H, "K": K, "V": V, "R": R, "chunk": C,
                       "per_rank": {"B": Bl, "H": Hl, "T": Tl},
                       "sharding": ("context parallel: T/N per rank, all-gather of affine state maps (NCCL)" if cp
                                    else "batch x head, no collective"),
                       "backward": "saved forward intermediates" if HD.hrdplr.save_workspace_default() else "recompute",
                       "l2": "inputs (>1 GB per step) are larger than the 126 MB L2" if world == 1 or scaling == "weak"
                             else "each step rewrites a workspace larger than the 126 MB L2 between reuses of any input"},
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "host_numa_node": numa.node},
            "gpu_launches": int(launches), "roofline": roof, "cpu_baseline": cpu, "clocks": clocks,
            "secondary": secondary or None,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cp_parity_check(dev, rank, world):
    """The context-parallel operator (T = 4096 * world cut over the ranks, B1 H2, initial state and a loss on
    every rank's final state) against the single-GPU operator on the same inputs, forward and every gradient;
    max relative error over all tensors and ranks."""
    import torch.distributed as dist
    import hdla_impl_b200 as HD
    from hdla_impl_b200.context_parallel import cp_chunk_hrdplr_delta_rule
    from hdla_impl_b200.sharding import shard_time
    from hdla_impl_b200.synthetic import make_inputs
    C, K = 64, 128
    T = 4096 * world
    x = make_inputs(1, T, 2, K, K, R, seed=1234, dtype=torch.bfloat16, h0_std=0.1, with_dht=True)
    rr = lambda n: R if n in ("a", "b") else 1
    lo, hi = shard_time(T, rank, world, C)
    lv = [x[n][:, lo * rr(n):hi * rr(n)].to(dev).requires_grad_(True) for n in NAMES]
    h0 = x["h0"].to(dev).requires_grad_(True)
    o, ht = cp_chunk_hrdplr_delta_rule(*lv, R, initial_state=h0, output_final_state=True, chunk_size=C)
    dht = x["dht"].to(dev)
    loss = (o.float() * x["do"][:, lo:hi].to(dev).float()).sum() + (ht * dht * (0.5 + rank)).sum()
    grads = torch.autograd.grad(loss, lv + [h0], allow_unused=True)
    # truth: the same slices chained on this rank's GPU alone
    full = [x[n].to(dev).requires_grad_(True) for n in NAMES]
    h0f = x["h0"].to(dev).requires_grad_(True)
    state, lf, parts, ht_true = h0f, 0.0, [], None
    for r_ in range(world):
        l_, h_ = shard_time(T, r_, world, C)
        part = [t[:, l_ * rr(n):h_ * rr(n)] for t, n in zip(full, NAMES)]
        o_r, state = HD.chunk_hrdplr_delta_rule(*part, R, initial_state=state, output_final_state=True, chunk_size=C)
        lf = lf + (o_r.float() * x["do"][:, l_:h_].to(dev).float()).sum() + (state * dht * (0.5 + r_)).sum()
        parts.append(o_r)
        if r_ == rank:
            ht_true = state
    gf = torch.autograd.grad(lf, full + [h0f])
    of = torch.cat(parts, 1)

    def rel(a, b):
        return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))
    errs = [rel(o, of[:, lo:hi]), rel(ht, ht_true)]
    for g, gg, n in zip(grads[:6], gf[:6], NAMES):
        errs.append(rel(g, gg[:, lo * rr(n):hi * rr(n)]))
    if rank == 0:
        errs.append(rel(grads[6], gf[6]))
    e = torch.tensor([max(errs)], device=dev, dtype=torch.float64)
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    HD.check_status(dev, wait=True)
    err = float(e.item())
    return {"max_rel_err": err, "passed": bool(err < 2e-2), "world": world, "T": T, "tolerance": 2e-2,
            "what": "cp_chunk_hrdplr_delta_rule vs the single-GPU operator: o, final states, dq dk dv da db dgk, dh0"}


def bench_cfg3(dev, rank, world, barrier, steps=10):
    """Long context (B1 T65536 H16): one GPU, or T cut over the ranks with context parallelism."""
    import torch.distributed as dist
    import hdla_impl_b200 as HD
    from hdla_impl_b200.context_parallel import cp_chunk_hrdplr_delta_rule
    from hdla_impl_b200.synthetic import make_inputs
    B, T, H, K, V, C, _ = WORKLOADS["cfg3"]
    Tl = T // world
    x = make_inputs(B, Tl, H, K, V, R, seed=100 + rank, dtype=torch.bfloat16)
    lv = [x[n].to(dev).requires_grad_(True) for n in NAMES]
    do = x["do"].to(dev)
    del x

    def step():
        if world > 1:
            o, _ = cp_chunk_hrdplr_delta_rule(*lv, R, chunk_size=C)
        else:
            o, _ = HD.chunk_hrdplr_delta_rule(*lv, R, chunk_size=C)
        torch.autograd.grad(o, lv, do)
    for _ in range(10):                                  # (the first collective calls set up NCCL's channels)
        step()
    ms = timed_steps(step, steps, barrier)
    coll_ms = None
    if world > 1:
        # the collective alone, same sizes: forward packs [3,B,H,K,V], backward [2,B,H,K,V] fp32 per rank
        f32 = dict(dtype=torch.float32, device=dev)
        p3, p2 = torch.empty(3, B, H, K, V, **f32), torch.empty(2, B, H, K, V, **f32)
        g3, g2 = torch.empty(world, 3, B, H, K, V, **f32), torch.empty(world, 2, B, H, K, V, **f32)

        def coll():
            dist.all_gather_into_tensor(g3, p3)
            dist.all_gather_into_tensor(g2, p2)
        for _ in range(3):
            coll()
        coll_ms = timed_steps(coll, steps, barrier) / steps
        tt = torch.tensor([ms, coll_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, coll_ms = tt.tolist()
    ms_step = ms / steps
    HD.check_status(dev, wait=True)
    return {"workload": "cfg3: B1 T65536 H16 K=V=128 bf16 chunk 64, fwd+bwd", "n_gpus": world,
            "ms_per_step": ms_step, "value": B * T / (ms_step / 1e3), "unit": "tokens/s", "steps": steps,
            "collective": "all_gather (one per direction)" if world > 1 else None,
            "collective_bytes_per_rank_per_step": (5 * B * H * K * V * 4) if world > 1 else 0,
            "collective_ms_per_step": coll_ms}


def bench_weak(dev, rank, world, barrier, steps=5):
    """Every rank its own cfg1 batch: no sharding, no communication (the ceiling strong scaling is compared with)."""
    import torch.distributed as dist
    import hdla_impl_b200 as HD
    from hdla_impl_b200.synthetic import make_inputs
    B, T, H, K, V, C, _ = WORKLOADS["cfg1"]
    x = make_inputs(B, T, H, K, V, R, seed=200 + rank, dtype=torch.bfloat16)
    lv = [x[n].to(dev).requires_grad_(True) for n in NAMES]
    do = x["do"].to(dev)
    del x

    def step():
        o, _ = HD.chunk_hrdplr_delta_rule(*lv, R, chunk_size=C)
        torch.autograd.grad(o, lv, do)
    for _ in range(3):
        step()
    ms = timed_steps(step, steps, barrier)
    tt = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms_step = tt.item() / steps
    return {"scaling": "weak", "ms_per_step": ms_step, "value": B * T * world / (ms_step / 1e3), "unit": "tokens/s",
            "B_per_step": B * world, "steps": steps}


def bench_decode_small(dev, steps=128):
    """cfg2 on this GPU: 128 decode steps of B256 H32, state updated in place; tokens/s and HBM fraction."""
    import hdla_impl_b200 as HD
    from hdla_impl_b200.synthetic import make_inputs
    B, _, H, K, V, _, _ = WORKLOADS["cfg2"]
    ntok = 8
    x = make_inputs(B, ntok, H, K, V, R, seed=7, dtype=torch.bfloat16, h0_std=0.02)
    dv = {n: x[n].to(dev) for n in NAMES}
    S = x["h0"].to(dev)
    scale = K ** -0.5
    tok = lambda t, n, r=1: dv[n][:, (t % ntok) * r:(t % ntok + 1) * r]

    def step(t):
        nonlocal S
        _, S = HD.fused_recurrent_dplr_delta_rule_fwd(tok(t, "q"), tok(t, "k"), tok(t, "v"), tok(t, "a", R),
                                                      tok(t, "b", R), tok(t, "gk"), R, scale, S, True,
                                                      inplace_state=True)
    for t in range(5):
        step(t)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for t in range(steps):
        step(t)
    e1.record()
    torch.cuda.synchronize(dev)
    sec = e0.elapsed_time(e1) / steps / 1e3
    peaks, how = load_peaks()
    byts = 2.0 * B * H * K * V * 4 + B * H * (7 * K + 2 * V) * 2
    gbs = byts / sec / 1e9
    del S, dv
    torch.cuda.empty_cache()
    return {"workload": "cfg2: B256 H32 K=V=128 decode, one token per step, fp32 state in place", "steps": steps,
            "us_per_step": sec * 1e6, "value": B / sec, "unit": "tokens/s",
            "roofline": {"bound": "hbm", "kernel": "recurrent_bulk_kernel", "achieved": gbs, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "algorithmic_bytes_per_step": byts,
                         "peak_source": f"{how} (copy)", "l2": "state (537 MB) is larger than the 126 MB L2"}}


def bench_cfg0_gpu(dev, steps=20):
    """The CPU configuration (B2 T256 H4 K=V=64 fp32) on the GPU: fp32 CUDA-core pipeline, fwd+bwd."""
    import hdla_impl_b200 as HD
    from hdla_impl_b200.synthetic import make_inputs
    B, T, H, K, V, C, _ = WORKLOADS["cfg0"]
    x = make_inputs(B, T, H, K, V, R, seed=0)
    lv = [x[n].to(dev).requires_grad_(True) for n in NAMES]
    do = x["do"].to(dev)

    def step():
        o, _ = HD.chunk_hrdplr_delta_rule(*lv, R, chunk_size=C)
        torch.autograd.grad(o, lv, do)
    for _ in range(3):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / steps
    return {"workload": "cfg0: B2 T256 H4 K=V=64 fp32 chunk 64, fwd+bwd (fp32 CUDA-core pipeline; launch bound)",
            "ms_per_step": ms, "value": B * T / (ms / 1e3), "unit": "tokens/s", "steps": steps}


def bench_host_link(dev, world, barrier, nbytes=256 << 20, reps=8):
    """What the host link gives every rank while ALL ranks copy at once: pinned host <-> device copies of 256 MB,
    one direction alone and both directions together.  The end-to-end figure of the line is bounded by the last
    number (every step moves its inputs in and its gradients out); when the ranks' links share a host-side
    bottleneck it does not grow with the number of GPUs, whatever the kernels do."""
    import torch.distributed as dist
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_out = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def run(h2d, d2h):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        s_in.wait_stream(torch.cuda.current_stream(dev))
        s_out.wait_stream(torch.cuda.current_stream(dev))
        for _ in range(reps):
            if h2d:
                with torch.cuda.stream(s_in):
                    d_in.copy_(h_in, non_blocking=True)
            if d2h:
                with torch.cuda.stream(s_out):
                    h_out.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream(dev).wait_stream(s_in)
        torch.cuda.current_stream(dev).wait_stream(s_out)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return reps * nbytes / (ms.item() / 1e3) / 1e9

    run(True, True)                                       # warm-up
    one_in, one_out, both = run(True, False), run(False, True), run(True, True)
    return {"per_rank_GBps": {"h2d_alone": one_in, "d2h_alone": one_out, "each_way_when_both": both},
            "all_ranks_GBps_each_way_when_both": both * world, "ranks_copying_at_once": world,
            "bytes_per_copy": nbytes}


def bench_layer_call(dev, steps=10, workload="cfg1"):
    """The operator as the reference layer calls it (HRDPLR/hdla_custom.py:290-345), at the cfg 1 shape, fwd+bwd:
    parameterize_a_b + chunk_hrdplr_delta_rule as two calls against chunk_hdla_delta_rule (a and b formed inside the
    chunk-preparation kernel), and the layer's norm x gate epilogue on the operator's output."""
    import torch.nn.functional as F
    import hdla_impl_b200 as HD
    from hdla_impl_b200.layer_ops import chunk_hdla_delta_rule, parameterize_a_b, rms_norm_fused_gate
    B, T, H, K, V, C, _ = WORKLOADS[workload]
    g = torch.Generator().manual_seed(7)
    rn = lambda *s_: torch.randn(*s_, generator=g)
    bf = torch.bfloat16
    mk = lambda x: x.to(bf).to(dev).requires_grad_(True)
    q, k, v = mk(F.normalize(rn(B, T, H, K), dim=-1)), mk(F.normalize(rn(B, T, H, K), dim=-1)), mk(rn(B, T, H, V))
    beta, log_f = mk(2 * torch.sigmoid(rn(B, T, H, 1))), mk(F.logsigmoid(rn(B, T, H, K)) / 16)
    do = rn(B, T, H, V).to(bf).to(dev)
    lv = [q, k, v, beta, log_f]

    def two_calls():
        a, b = parameterize_a_b(beta, k, log_f)
        o, _ = HD.chunk_hrdplr_delta_rule(q, k, v, a, b, log_f, R, scale=1.0, chunk_size=C)
        torch.autograd.grad(o, lv, do)

    def one_call():
        o, _ = chunk_hdla_delta_rule(q, k, v, beta, log_f, scale=1.0)
        torch.autograd.grad(o, lv, do)

    x = rn(B * T, H * V).to(bf).to(dev).requires_grad_(True)
    gate = rn(B * T, H * V).to(bf).to(dev).requires_grad_(True)
    w = torch.ones(H * V, dtype=bf, device=dev, requires_grad=True)
    dn = rn(B * T, H * V).to(bf).to(dev)

    def norm():
        torch.autograd.grad(rms_norm_fused_gate(x, gate, w, 1e-5), [x, gate, w], dn)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / steps

    t2, t1, tn = timed(two_calls), timed(one_call), timed(norm)
    # the stand-alone layer kernels by themselves, straight through the C ABI (preallocated outputs, so that host-side
    # autograd bookkeeping does not show): algorithmic bytes (every element read or written once) / time
    from hdla_impl_b200 import _lib
    lib, st, P = _lib.load(), _lib.stream_ptr(dev), _lib.ptr
    es, n_ab, n_ng, dtc = 2, B * T * H * K, B * T * H * V, _lib.dtype_code(bf)
    with torch.no_grad():
        a, b = parameterize_a_b(beta, k, log_f)
        ga, gb = torch.randn_like(a), torch.randn_like(b)
        dbeta, dk_, dlf = torch.empty_like(beta), torch.empty_like(k), torch.empty_like(log_f)
        o_n, dx, dg = torch.empty_like(x), torch.empty_like(x), torch.empty_like(gate)
        dw = torch.zeros(H * V, dtype=torch.float32, device=dev)
        rows, D = x.shape

        def chk(rc):
            if rc != 0:
                raise RuntimeError(_lib.last_error())
        t_abf = timed(lambda: chk(lib.hdla_param_ab_fwd(P(beta), P(k), P(log_f), P(a), P(b), B, T, H, K, dtc, st)))
        t_abb = timed(lambda: chk(lib.hdla_param_ab_bwd(P(beta), P(k), P(log_f), P(ga), P(gb), P(dbeta), P(dk_), P(dlf),
                                                        B, T, H, K, dtc, st)))
        t_ngf = timed(lambda: chk(lib.hdla_norm_gate_fwd(P(x), P(gate), P(w), P(o_n), rows, D, 1e-5, dtc, st)))
        t_ngb = timed(lambda: chk(lib.hdla_norm_gate_bwd(P(x), P(gate), P(w), P(dn), P(dx), P(dg), P(dw), rows, D, 1e-5,
                                                         dtc, st)))
    peak = load_peaks()[0]["hbm_gbs"]
    kern = lambda ms, elems: {"ms": ms, "GBps": elems * es / ms / 1e6, "frac_of_hbm_peak": elems * es / ms / 1e6 / peak}
    return {"workload": f"{workload} shape (B{B} T{T} H{H} K{K} V{V}) as the layer calls the operator (q, k, v, beta, "
                        "log_f; scale 1), bf16, fwd+bwd",
            "two_calls_ms": t2, "one_call_ms": t1, "norm_gate_fwd_bwd_ms": tn,
            "one_call_tokens_per_s": B * T / (t1 / 1e3), "steps": steps,
            "kernels": {"param_ab_fwd": kern(t_abf, 6 * n_ab), "param_ab_bwd": kern(t_abb, 8 * n_ab),
                        "norm_gate_fwd": kern(t_ngf, 3 * n_ng), "norm_gate_bwd": kern(t_ngb, 5 * n_ng)}}


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
    host = {n: x[n].pin_memory() for n in NAMES}
    dv = {n: host[n].to(dev) for n in NAMES}
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
        cur = {n: tok(host, t, n, R if n in ("a", "b") else 1).contiguous().to(dev, non_blocking=True) for n in NAMES}
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
    from hdla_impl_b200.recurrent import check_recurrent_status
    check_recurrent_status(dev)
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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--layer-call", action="store_true",
                    help="only the layer-call measurement (secondary.layer_call of the default line) at --workload's shape")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.layer_call:
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
        print(json.dumps({"layer_call": bench_layer_call(dev, max(args.steps, 1), args.workload)}))
    elif args.workload == "cfg2" and args.impl == "ours":
        if args.steps == 20:
            args.steps = 128
        run_decode(args, rank, world, local_rank)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
