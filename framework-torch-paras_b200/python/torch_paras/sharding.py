"""Sharding of the hot path over the GPUs of one box: one process per GPU, no collective on
the forward path.

Attention is independent per (batch, kv-head group), RMSNorm and SwiGLU per row, so each
rank takes a contiguous block of units and runs the single-GPU kernels on it.  The only
exchange the path ever needs is the optional re-assembly of the outputs, an all-gather
(NCCL over NVLink on GPUs; gloo on CPU for the tests).  The reference has no multi-device
logic beyond host-bounced copies (csrc/ops/tensor_ops.cpp:313-322); this module is new.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


def shard_bounds(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced block of `n_units` for `rank`: the first n % world ranks get one more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def attention_shard(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int):
    """Views of this rank's share of [B, Hq, L, D] / [B, Hkv, L, D] tensors and a description of
    the share.  Splits along the batch when there are at least `world` batches, otherwise along
    the kv heads (query heads follow their kv head, so GQA sharing stays inside one GPU)."""
    B, Hq, Hkv = q.shape[0], q.shape[1], k.shape[1]
    if Hkv == 0 or Hq % Hkv:
        raise ValueError("query heads must be a multiple of key/value heads")
    group = Hq // Hkv
    if B >= world:
        lo, hi = shard_bounds(B, rank, world)
        return q[lo:hi], k[lo:hi], v[lo:hi], ("batch", lo, hi)
    lo, hi = shard_bounds(Hkv, rank, world)
    return (q[:, lo * group:hi * group], k[:, lo:hi], v[:, lo:hi], ("kv_head", lo, hi))


def rows_shard(x: torch.Tensor, rank: int, world: int):
    """This rank's block of rows of a [rows, H] (or [..., H]) tensor, split on dim 0."""
    lo, hi = shard_bounds(x.shape[0], rank, world)
    return x[lo:hi], (lo, hi)


def as_cuda(t: torch.Tensor) -> torch.Tensor:
    """A torch.cuda tensor aliasing the memory of a contiguous `paras:N` tensor (N >= 1), so
    that torch.distributed's NCCL backend can send it.  The caller must synchronise the paras
    device before the CUDA side reads the data."""
    if t.device.type != "paras" or (t.device.index or 0) < 1:
        raise ValueError("as_cuda expects a tensor on paras:1..N")
    if not t.is_contiguous():
        raise ValueError("as_cuda expects a contiguous tensor")
    nbytes = t.numel() * t.element_size()

    class _Mem:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (t.data_ptr(), False),
                                    "version": 2}

    raw = torch.as_tensor(_Mem(), device=torch.device("cuda", t.device.index - 1))
    out = raw.view(t.dtype).view(t.shape)
    out._paras_owner = t  # keep the paras storage alive as long as the alias
    return out


def gather_shards(local: torch.Tensor, sizes: Sequence[int], dim: int = 0, group=None) -> torch.Tensor:
    """All-gathers per-rank blocks whose extent along `dim` is `sizes[rank]` and concatenates them.
    Works on CPU tensors (gloo) and CUDA tensors (NCCL); for `paras` tensors pass `as_cuda(t)`."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if len(sizes) != world:
        raise ValueError("sizes must have one entry per rank")
    moved = local.movedim(dim, 0).contiguous()
    biggest = max(sizes)
    padded = moved
    if moved.shape[0] != biggest:
        pad = torch.zeros((biggest - moved.shape[0],) + tuple(moved.shape[1:]), dtype=moved.dtype,
                          device=moved.device)
        padded = torch.cat([moved, pad], 0)
    bufs: List[torch.Tensor] = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded, group=group)
    out = torch.cat([b[:n] for b, n in zip(bufs, sizes)], 0)
    return out.movedim(0, dim)


# ---- failure detection on the host ---------------------------------------------------------
# The forward path has no collective, so a rank that dies only matters at the optional gather.
# Ranks announce each step in the rendezvous store before they enter a gather; a rank that finds a
# peer missing raises on the host instead of launching a collective that would wait for it.  (The
# other net is the process group's timeout, which turns a gather with a dead peer into an error.)
def announce_step(store, rank: int, step: int) -> None:
    """Records that `rank` has finished its work for `step` and is about to exchange results."""
    store.set(f"paras/step/{rank}", str(step))


def absent_ranks(store, world: int, step: int, wait_s: float = 2.0, poll_s: float = 0.02) -> List[int]:
    """Ranks that have not announced `step` within `wait_s` seconds (empty = everyone is there)."""
    import time
    deadline = time.monotonic() + wait_s
    missing = list(range(world))
    while missing:
        still = []
        for r in missing:
            try:
                ok = store.check([f"paras/step/{r}"]) and int(store.get(f"paras/step/{r}")) >= step
            except Exception:  # noqa: BLE001  (store gone with its owner: the peer is absent)
                ok = False
            if not ok:
                still.append(r)
        missing = still
        if not missing or time.monotonic() >= deadline:
            break
        time.sleep(poll_s)
    return missing


def gather_shards_checked(store, rank: int, step: int, local: torch.Tensor, sizes: Sequence[int], dim: int = 0,
                          group=None, wait_s: float = 2.0) -> torch.Tensor:
    """gather_shards for step `step`, entered only when every rank has announced that step."""
    import torch.distributed as dist
    announce_step(store, rank, step)
    gone = absent_ranks(store, dist.get_world_size(group), step, wait_s)
    if gone:
        raise RuntimeError(f"paras sharding: rank(s) {gone} did not reach step {step}; gather not started")
    return gather_shards(local, sizes, dim, group)


def _parse_cpulist(text: str) -> List[int]:
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_cpus(pci_bus_id: str, sysfs: str = "/sys") -> List[int]:
    """CPUs of the NUMA node a GPU hangs off, from sysfs (`pci_bus_id` like "0000:1b:00.0");
    empty when the platform does not say (single node, or no numa_node entry)."""
    import os
    dev = os.path.join(sysfs, "bus", "pci", "devices", pci_bus_id.lower())
    try:
        node = int(open(os.path.join(dev, "numa_node")).read())
        if node < 0:
            return []
        return _parse_cpulist(open(os.path.join(sysfs, "devices", "system", "node", f"node{node}", "cpulist")).read())
    except (OSError, ValueError):
        return []


def bind_host_to_gpu_node(gpu: int) -> List[int]:
    """Pins the calling process to the CPUs of the NUMA node of CUDA GPU `gpu`, so that the pinned
    host buffers it allocates afterwards (first touch) and the threads that fill them sit next to
    that GPU's PCIe root instead of across the socket link.  One rank per GPU feeding its GPU from
    host memory is bound by exactly that path.  Returns the CPUs bound to ([] = left as it was)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(gpu)).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        if len(bus.split(":")[0]) == 8:      # NVML prints an 8-digit domain, sysfs a 4-digit one
            bus = bus[4:]
        cpus = gpu_numa_cpus(bus)
        allowed = os.sched_getaffinity(0)
        cpus = [c for c in cpus if c in allowed]
        if cpus:
            os.sched_setaffinity(0, cpus)
        return cpus
    except Exception:  # noqa: BLE001  (no NVML, no sysfs entry, not permitted: stay unbound)
        return []
