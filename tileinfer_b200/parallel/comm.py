"""Control-plane communicator used by the engine (sampling, server fan-out, barriers).

The reference talks to NCCL through free functions on the WORLD group (engine/parallel.py:19-200).
Here the engine sees a small object so that the same code runs on one process (`SingleComm`), on
torch.distributed ranks (`TorchDistComm`, nccl on GPUs / gloo on CPU) and inside unit tests
(`tileinfer_b200.parallel.fake_comm.FakeComm`, threads with injectable faults).  The hot
tensor-parallel reductions of the GPU model do not go through this class: they are fused into the
sm_100a kernels over peer memory (see parallel/symm_mem.py).
"""
from __future__ import annotations

import datetime
import os
import pickle

import torch


class SingleComm:
    rank, world_size = 0, 1

    def all_reduce(self, t):
        return t

    def all_gather(self, t):
        return [t]

    def broadcast(self, t, src=0):
        return t

    def broadcast_object(self, obj, src=0):
        return obj

    def barrier(self):
        pass


class TorchDistComm:
    """torch.distributed-backed communicator (one process per GPU, or gloo ranks on CPU)."""

    def __init__(self, group=None, device=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.device = device

    def all_reduce(self, t):
        self.dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t):
        t = t.contiguous()
        out = torch.empty((self.world_size,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        self.dist.all_gather_into_tensor(out.view(-1), t.view(-1), group=self.group)
        return list(out.unbind(0))

    def broadcast(self, t, src=0):
        self.dist.broadcast(t, src=src, group=self.group)
        return t

    def broadcast_object(self, obj, src=0):
        box = [obj if self.rank == src else None]
        self.dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def barrier(self):
        self.dist.barrier(group=self.group)


_COMM = SingleComm()


def get_comm():
    return _COMM


def init_distributed(tp_size: int = 1, timeout_s: float = 600.0, device: str = "cuda"):
    """Join the torchrun rendezvous when tp_size > 1 (reference: engine/parallel.py:19-56).

    Reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT from the environment.  Returns
    the communicator.  WORLD_SIZE must equal tp_size, as in the reference."""
    global _COMM
    if tp_size <= 1:
        _COMM = SingleComm()
        if device == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        return _COMM
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != tp_size:
        raise RuntimeError(f"tp_size={tp_size} but WORLD_SIZE={world}; launch with torchrun --nproc-per-node {tp_size}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if not dist.is_initialized():
        backend = "nccl" if device == "cuda" else "gloo"
        kw = {}
        if device == "cuda":
            local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", 0)))
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    _COMM = TorchDistComm(device=device)
    return _COMM


def shutdown_distributed():
    global _COMM
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    _COMM = SingleComm()
