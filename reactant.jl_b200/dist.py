"""Host-side plumbing for one-process-per-GPU meshes.

The engine itself only needs two byte strings moved between the processes of a
mesh: the NCCL unique id (rank 0 -> all) and the table of mailbox IPC handles
(all -> all).  Reactant moves such things through XLA's distributed key-value
store (src/xla/Distributed.jl:77-100); here any transport will do, and this
module uses torch.distributed (NCCL on GPUs, gloo on CPU-only test runs).
"""
from __future__ import annotations

import os


def shard_bounds(length: int, parts: int, index: int):
    """[lo, hi) of chunk `index` when a dimension of `length` is split into
    `parts` equal contiguous chunks in mesh order (src/xla/Sharding.jl:246-267).
    The engine requires divisibility (no padding rule)."""
    if length % parts:
        raise ValueError(f"dimension of length {length} is not divisible by the mesh size {parts}")
    step = length // parts
    return index * step, (index + 1) * step


class Dist:
    """Rendezvous, barrier, max/sum over ranks and byte exchange for a mesh of processes."""

    def __init__(self, world: int, backend: str = "nccl"):
        self.world = world
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.backend = backend
        self.dist = self.torch = None
        if world > 1:
            import torch
            import torch.distributed as dist
            kw = {}
            if backend == "nccl":
                torch.cuda.set_device(self.local_rank)
                kw["device_id"] = torch.device("cuda", self.local_rank)
            dist.init_process_group(backend, **kw)
            self.dist, self.torch = dist, torch

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
            if self.backend == "nccl":
                self.torch.cuda.synchronize()

    def reduce(self, v: float, op: str = "max") -> float:
        if self.world == 1:
            return v
        dev = "cuda" if self.backend == "nccl" else "cpu"
        t = self.torch.tensor([float(v)], dtype=self.torch.float64, device=dev)
        ops = {"max": self.dist.ReduceOp.MAX, "min": self.dist.ReduceOp.MIN, "sum": self.dist.ReduceOp.SUM}
        self.dist.all_reduce(t, op=ops[op])
        return float(t.item())

    def all_gather_bytes(self, b: bytes):
        if self.world == 1:
            return [b]
        out = [None] * self.world
        self.dist.all_gather_object(out, b)
        return out

    def broadcast_bytes(self, b):
        if self.world == 1:
            return b
        box = [b]
        self.dist.broadcast_object_list(box, src=0)
        return box[0]

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def connect_collectives(rx, client, dist: Dist, mode: str = "mailbox") -> str:
    """Give every process of the mesh what its client needs for all-reduce:
    the NVLink mailbox table (default) or the NCCL unique id."""
    if dist.world == 1:
        return "none"
    if mode in ("nccl", "mailbox+nccl"):
        uid = rx.collectives_unique_id() if dist.rank == 0 else None
        client.init_collectives(dist.broadcast_bytes(uid))
        if mode == "nccl":
            return "nccl"
    handles = dist.all_gather_bytes(client.mailbox_handles())
    client.open_mailboxes(b"".join(handles))
    # "mailbox+nccl": single words (loss, sharded sums) over the NVLink mailbox, vectors (gradients) over NCCL
    return "nvlink-mailbox" if mode == "mailbox" else "nvlink-mailbox + nccl"
