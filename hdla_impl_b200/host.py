"""Forward + backward of the chunked operator on HOST-resident tensors.

For callers whose activations live in pinned host memory (offloaded training, a data-loader side
process): the batch is cut into slices along B -- (batch, head) pairs are independent -- and the
slices are pipelined over three streams, so the host->device copies of slice i+1, the kernels of
slice i and the device->host copies of slice i-1 overlap.  The result is bound by the slower PCIe
direction rather than by the sum of copies and compute.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from .hrdplr import chunk_hrdplr_delta_rule

def _parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


class numa_local_to(object):
    """Context manager: run the calling thread on the CPUs of the NUMA node the GPU hangs off.

    Pinned host memory is placed on the node of the thread that allocates it, and a DMA that has to
    cross the socket interconnect runs at a fraction of the PCIe rate, so the pinned buffers of
    ``chunk_fwd_bwd_from_host`` should be allocated (and the copies issued) inside this context.
    Best effort: without NUMA information in sysfs, or when the node's CPUs are outside the allowed
    set, nothing changes.  ``node`` is the node bound to, or None.  The previous affinity is restored
    on exit."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.node = None
        self._saved = None

    def __enter__(self):
        try:
            pr = torch.cuda.get_device_properties(self.device)
            bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
                node = int(f.read().strip())
            if node < 0:
                return self
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = _parse_cpulist(f.read())
            allowed = os.sched_getaffinity(0)
            target = cpus & allowed
            if target and target != allowed:
                os.sched_setaffinity(0, target)
                self._saved = allowed
            if target:
                self.node = node
        except (OSError, ValueError, AttributeError, RuntimeError, AssertionError):
            pass
        return self

    def __exit__(self, *exc):
        if self._saved is not None:
            try:
                os.sched_setaffinity(0, self._saved)
            except OSError:
                pass
        return False


_IN = ("q", "k", "v", "a", "b", "gk")
_OUT = ("o", "dq", "dk", "dv", "da", "db", "dgk")


_copy_streams: Dict[int, tuple] = {}
_stages: Dict[tuple, dict] = {}      # (device index, slice shape key) -> dict(turn=int, slots=[slot0, slot1]), a slot = dict(bufs=..., done=Event|None)


def _streams(dev: torch.device):
    """One copy-in and one copy-out stream per device, kept across calls so that the copies of successive
    calls stay ordered among themselves."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _copy_streams:
        _copy_streams[idx] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _copy_streams[idx]


def join_host_streams(device) -> None:
    """Make the current stream of ``device`` wait for every copy that ``chunk_fwd_bwd_from_host(sync=False)`` has
    enqueued so far: work enqueued (or an event recorded) on the current stream afterwards is ordered after the
    results have reached host memory."""
    dev = torch.device(device)
    s_in, s_out = _streams(dev)
    cur = torch.cuda.current_stream(dev)
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)


def chunk_fwd_bwd_from_host(host_in: Dict[str, torch.Tensor], host_out: Optional[Dict[str, torch.Tensor]],
                            RANK_AB: int, device, scale: Optional[float] = None, chunk_size: int = 64,
                            slice_batch: int = 1, sync: bool = True) -> Dict[str, torch.Tensor]:
    """``host_in``: pinned CPU tensors q,k,v,a,b,gk and ``do`` (gradient of o), layouts as in
    ``chunk_hrdplr_delta_rule``.  Returns (and fills, if given) ``host_out`` with pinned CPU tensors
    o,dq,dk,dv,da,db,dgk.  With ``sync`` (default) the device is synchronised before returning.  With
    ``sync=False`` the call only enqueues and nothing waits for the copy-out: the copy-in and the kernels of a
    following call run under this call's copy-out (the device buffers of a slice are reused as soon as the
    kernels that read them are done, which an event tracks across calls).  The caller must not touch
    ``host_in`` / ``host_out`` before ``join_host_streams(device)`` plus a synchronisation of the current
    stream, or ``torch.cuda.synchronize(device)``."""
    dev = torch.device(device)
    B = host_in["q"].shape[0]
    if host_out is None:
        host_out = {}
    names_in = _IN + ("do",)
    for n in names_in:
        if not host_in[n].is_pinned():
            raise ValueError(f"host tensor '{n}' must be in pinned memory")
    ref = dict(o="v", dq="q", dk="k", dv="v", da="a", db="b", dgk="gk")
    for n in _OUT:
        if n not in host_out:
            src = host_in[ref[n]]
            host_out[n] = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = _streams(dev)
    bounds = [(i, min(i + slice_batch, B)) for i in range(0, B, slice_batch)]
    with torch.cuda.device(dev):
        for idx, (lo, hi) in enumerate(bounds):
            key = (dev.index, hi - lo) + tuple((n, tuple(host_in[n].shape[1:]), host_in[n].dtype) for n in names_in)
            stage = _stages.setdefault(key, dict(turn=0, slots=[dict(bufs=None, done=None), dict(bufs=None, done=None)]))
            slot = stage["slots"][stage["turn"] & 1]   # two sets of device input buffers, alternating from slice to
            stage["turn"] += 1                         # slice ACROSS calls too (a call may be a single slice)
            with torch.cuda.stream(s_in):
                if slot["done"] is not None:
                    s_in.wait_event(slot["done"])              # the kernels that last read these buffers are done
                if slot["bufs"] is None:
                    slot["bufs"] = {n: torch.empty((hi - lo,) + tuple(host_in[n].shape[1:]), dtype=host_in[n].dtype,
                                                   device=dev) for n in names_in}
                    for t in slot["bufs"].values():
                        t.record_stream(cur)                   # allocated on the copy stream, read by the kernels
                for n in names_in:
                    slot["bufs"][n].copy_(host_in[n][lo:hi], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            lv = [slot["bufs"][n].requires_grad_(True) for n in _IN]
            o, _ = chunk_hrdplr_delta_rule(*lv, RANK_AB, scale=scale, chunk_size=chunk_size)
            grads = torch.autograd.grad(o, lv, slot["bufs"]["do"])
            ev = torch.cuda.Event()
            ev.record(cur)
            slot["done"] = ev
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev)
                for n, t in zip(_OUT, (o.detach(),) + tuple(grads)):
                    t.record_stream(s_out)
                    host_out[n][lo:hi].copy_(t, non_blocking=True)
            for n in _IN:
                slot["bufs"][n].requires_grad_(False)
    if sync:
        torch.cuda.synchronize(dev)
    return host_out
