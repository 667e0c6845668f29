"""Import shim for the reference's communicator module (engine/parallel.py:19-200): the same free functions on
top of `tileinfer_b200.parallel.comm`.  The hot tensor-parallel reductions do not go through these (they are
fused into the kernels over peer memory); they serve the control plane, the NCCL baseline path and user code."""
import torch

from tileinfer_b200.parallel.comm import get_comm, init_distributed, shutdown_distributed  # noqa: F401


def get_tp_rank() -> int:
    return get_comm().rank


def get_tp_world_size() -> int:
    return get_comm().world_size


def is_tp_enabled() -> bool:
    return get_comm().world_size > 1


def barrier():
    get_comm().barrier()


def tp_all_reduce(tensor):
    return get_comm().all_reduce(tensor)


def tp_all_reduce_async(tensor):
    """The reference returns a work handle; the reduction here is complete on return, the handle's wait() is a no-op."""
    get_comm().all_reduce(tensor)

    class _Done:
        def wait(self):
            return None
    return _Done()


def tp_broadcast(tensor, src: int = 0):
    return get_comm().broadcast(tensor, src)


def tp_distributed_argmax(local_logits, vocab_offset: int):
    """Arg-max over a vocabulary sharded across ranks: every rank contributes (max, global index)."""
    comm = get_comm()
    vals, idx = local_logits.float().max(dim=-1)
    idx = idx + vocab_offset
    if comm.world_size == 1:
        return idx
    all_v = torch.stack(comm.all_gather(vals.contiguous()))
    all_i = torch.stack(comm.all_gather(idx.contiguous()))
    best = all_v.argmax(dim=0, keepdim=True)
    return all_i.gather(0, best)[0]


tp_distributed_argmax_fused = tp_distributed_argmax


def shard_weight_col(weight, rank=None, world=None):
    """Output-dimension (row) shard of a [out, in] weight: column-parallel linear."""
    comm = get_comm()
    rank = comm.rank if rank is None else rank
    world = comm.world_size if world is None else world
    n = weight.shape[0] // world
    return weight[rank * n:(rank + 1) * n]


def shard_weight_row(weight, rank=None, world=None):
    """Input-dimension shard of a [out, in] weight: row-parallel linear (followed by an all-reduce)."""
    comm = get_comm()
    rank = comm.rank if rank is None else rank
    world = comm.world_size if world is None else world
    n = weight.shape[1] // world
    return weight[:, rank * n:(rank + 1) * n]


def shard_bias_col(bias, rank=None, world=None):
    return shard_weight_col(bias, rank, world)
