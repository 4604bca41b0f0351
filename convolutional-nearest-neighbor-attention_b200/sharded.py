"""Batch-sharded inference over the GPUs of one node (one process per GPU).

Every operation of the ConvNN path is per image, so ranks take contiguous slices of the
batch with replicated weights and no collective inside the model; the only exchange is
one all-gather of the logits (reference has no multi-GPU code at all).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split of ``n`` items: the first ``n % world`` ranks get one more."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shared_candidates(T: int, num_samples: int, device, seed: int = 0, group=None) -> torch.Tensor:
    """One random candidate set for all ranks (rank 0 draws, everyone receives it), so a
    sharded run selects from the same candidates as a single-GPU run of the whole batch."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    cand = torch.randperm(T, generator=g)[:num_samples].to(device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(cand, src=0, group=group)
    return cand


def gather_logits(local: torch.Tensor, total: int, group=None) -> torch.Tensor:
    """All-gather per-rank logits (n_r, classes) into (total, classes) in batch order."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    sizes = [shard_bounds(total, world, r) for r in range(world)]
    nmax = max(hi - lo for lo, hi in sizes)
    pad = local
    if local.shape[0] < nmax:
        pad = torch.zeros(nmax, local.shape[1], dtype=local.dtype, device=local.device)
        pad[: local.shape[0]] = local
    out = torch.empty(world * nmax, local.shape[1], dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, pad.contiguous(), group=group)
    if all(hi - lo == nmax for lo, hi in sizes):
        return out
    return torch.cat([out[r * nmax: r * nmax + (hi - lo)] for r, (lo, hi) in enumerate(sizes)], dim=0)


class LogitsGather:
    """Collects the logits of `batches_per_flush` consecutive batches and all-gathers them with ONE
    collective on a side stream, double-buffered, so that the exchange of one group of batches runs
    under the forwards of the next group instead of between them on the compute stream.  (A
    collective per batch costs its launch latency and a slice of the SMs every 2 ms; the logits of
    32 ViT-Tiny batches are 16 MB per rank.)  With one rank it only collects.  ``add`` may be called from
    different streams (batches in flight on several lanes): every add is ordered on the stream that is
    current at the call, and the flush waits for all of them."""

    def __init__(self, world, batches_per_flush, n_local, classes, dtype, dev):
        self.world, self.per, self.n_local = world, max(1, int(batches_per_flush)), n_local
        self.local = [torch.empty(self.per, n_local, classes, dtype=dtype, device=dev) for _ in range(2)]
        self.copied = [torch.cuda.Event() for _ in range(2)]
        self.added = [[torch.cuda.Event() for _ in range(self.per)] for _ in range(2)]
        self.done = [torch.cuda.Event() for _ in range(2)]
        self.slot, self.j = 0, 0
        self.last = None                         # (tensor with the most recent group's logits, event that says when)
        if world > 1:
            self.side = torch.cuda.Stream(dev)
            self.full = [torch.empty(world, self.per, n_local, classes, dtype=dtype, device=dev) for _ in range(2)]

    def add(self, logits):
        """Append one batch's logits; flushes when the group is complete.  Returns the (tensor, event)
        of the group this call completed, else None."""
        s = self.slot
        cur = torch.cuda.current_stream()
        cur.wait_event(self.done[s])             # whoever last read this slot has finished
        self.local[s][self.j].copy_(logits, non_blocking=True)
        self.added[s][self.j].record(cur)
        self.j += 1
        return self.flush() if self.j == self.per else None

    def flush(self):
        if self.j == 0:
            return self.last
        s, n = self.slot, self.j
        cur = torch.cuda.current_stream()
        for e in self.added[s][:n]:              # adds made on other streams
            cur.wait_event(e)
        self.copied[s].record(cur)
        if self.world > 1:
            with torch.cuda.stream(self.side):
                self.side.wait_event(self.copied[s])
                dist.all_gather_into_tensor(self.full[s], self.local[s])
                self.done[s].record(self.side)
            out = self.full[s][:, :n]            # (world, batches, n_local, classes)
        else:
            self.done[s].record(cur)
            out = self.local[s][:n]
        self.last = (out, self.done[s])
        self.slot, self.j = s ^ 1, 0
        return self.last

    def drain(self):
        self.flush()
        if self.world > 1:
            torch.cuda.current_stream().wait_stream(self.side)


@torch.no_grad()
def sharded_forward(model, images: torch.Tensor, group=None, gather: bool = True) -> torch.Tensor:
    """Run ``model`` on this rank's slice of ``images`` (the full batch, same on every rank)
    and return the full logits (or the local slice when ``gather`` is False)."""
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    lo, hi = shard_bounds(images.shape[0], world, rank)
    local = model(images[lo:hi])
    return gather_logits(local, images.shape[0], group) if gather else local


def bind_host_to_device(device) -> bool:
    """Restrict the calling process to the CPU cores next to `device` (NVML's ideal affinity for
    that GPU) so that pinned host buffers allocated afterwards come from the memory of the socket
    the GPU hangs off.  With eight ranks streaming input batches at the same time, host buffers on
    the far socket make every copy cross the inter-socket link.  Only the process's own CPU
    affinity changes (no GPU setting is touched).  Returns False, and changes nothing, when NVML
    or the PCI identity of the device is unavailable."""
    try:
        import pynvml
        props = torch.cuda.get_device_properties(device)
        bus = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        pynvml.nvmlDeviceSetCpuAffinity(handle)
        return True
    except Exception:
        return False
