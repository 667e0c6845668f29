"""Symmetric peer buffers for the fused tensor-parallel kernels.

Two allocators sit behind `PeerComm`:

* `torch.distributed._symmetric_memory` (driver VMM allocations exchanged between the ranks and, where the
  GPUs and the driver support it, bound to an NVLS multicast object): gives a pointer table of every rank's
  buffer plus ONE multicast address through which `multimem.ld_reduce` sums all ranks' copies inside NVSwitch.
  Used for the large partial-sum buffers of the many-row all-reduce (ops/csrc/fused_ar.cu).
* plain `cudaMalloc` + CUDA IPC handles (no multicast): the packet buffers of the decode path, and the fallback
  for everything when NVLS is switched off (`TI_NVLS=0` or `NCCL_NVLS_ENABLE=0`) or unavailable.  Processes that
  may lose a peer must run in this mode: memory bound to a multicast object must not outlive a rank that dies.

Each rank owns (a) a packet buffer for the row-parallel all-reduce, laid out
[2 slots][tp sources][m_cap rows][N/2] 16-byte packet pairs, (b) a packet buffer for the top-k
candidate exchange [2][tp][m_cap][64] and (c) a step counter and a status word.  The buffers are
plain cudaMalloc memory; their CUDA-IPC handles travel over torch.distributed and every rank maps
all of them, so a kernel can store to / poll any rank's buffer over NVLink.  Tags are derived from
the device step counter (advanced by the embedding kernel once per forward) and the position of the
collective inside the step, so CUDA-graph replays need no host-side argument changes.

The reference has no counterpart; its communicator is NCCL only (engine/parallel.py:19-200).
"""
from __future__ import annotations

import ctypes
import os

import torch

from ..ops import functional as F


def nvls_wanted() -> bool:
    """Multicast (NVLS) data plane for this package's own kernels: on unless TI_NVLS=0 or NCCL's own switch is off
    (the tests in which a rank leaves run everything, NCCL included, without NVLS)."""
    return os.environ.get("TI_NVLS", "1") != "0" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"


class PeerComm:
    def __init__(self, comm, hidden: int, m_cap: int = 64, timeout_s: float = 2.0, device=None, ar_rows: int = 0):
        self.comm = comm
        self.tp, self.rank = comm.world_size, comm.rank
        self.m_cap = m_cap
        self.hidden = hidden
        self.timeout_ns = int(timeout_s * 1e9)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        # step counter + status live in ordinary torch memory (only this rank touches them)
        self.ctrl = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.step_ptr = self.ctrl.data_ptr()
        self.status_ptr = self.ctrl.data_ptr() + 4
        self.ll_bytes = 2 * self.tp * m_cap * (hidden // 2) * 16
        self.cand_bytes = 2 * self.tp * m_cap * 64 * 16
        self._local = []
        self._mapped = []
        self.ll_ptrs = self._exchange(self.ll_bytes)
        self.cand_ptrs = self._exchange(self.cand_bytes)
        # many-row all-reduce: two alternating partial-sum buffers [ar_rows, hidden] bf16 and one flag per source rank
        self.ar_rows = ar_rows
        self.part_ptrs, self.part_mc, self._symm_keep = [None, None], [0, 0], []
        self.flag_ptrs = self._exchange(256)
        self.nvls = False
        if ar_rows > 0 and self.tp > 1:
            nbytes = ar_rows * hidden * 2
            for i in range(2):
                got = self._symm_alloc(nbytes) if nvls_wanted() else None
                if got is None:
                    self.part_ptrs[i], self.part_mc[i] = self._exchange(nbytes), 0
                else:
                    self.part_ptrs[i], self.part_mc[i] = got
            self.nvls = all(mc != 0 for mc in self.part_mc)

    def _symm_alloc(self, nbytes: int):
        """(pointer table, multicast address) of a torch symmetric-memory allocation, or None when that allocator or
        multicast is not available here (all ranks then take the same fallback: the decision is agreed on)."""
        import torch.distributed as dist
        ok, out = 1, None
        try:
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
            hdl = symm.rendezvous(t, dist.group.WORLD.group_name)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            ptrs = [int(x) for x in hdl.buffer_ptrs]
            if mc == 0 or len(ptrs) != self.tp:
                ok = 0
            else:
                t.zero_()
                out = (t, hdl, ptrs, mc)
        except Exception:
            ok = 0
        flag = torch.tensor([ok], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0 or out is None:
            return None
        self._symm_keep.append(out[:2])
        torch.cuda.synchronize()
        self.comm.barrier()
        return out[2], out[3]

    def part_view(self, parity: int, rows: int) -> torch.Tensor:
        """This rank's partial-sum buffer `parity` as a [rows, hidden] bf16 tensor (the GEMM epilogue stores into it)."""
        assert rows <= self.ar_rows, f"{rows} rows exceed the all-reduce buffers ({self.ar_rows}); raise max_num_batched_tokens"
        key = ("part", parity)
        base = getattr(self, "_views", None)
        if base is None:
            base = self._views = {}
        if key not in base:
            base[key] = _tensor_from_ptr(self.part_ptrs[parity][self.rank], self.ar_rows * self.hidden, torch.bfloat16,
                                         self.device).view(self.ar_rows, self.hidden)
        return base[key][:rows]

    def _exchange(self, nbytes: int) -> list:
        lib = F.L()
        p = ctypes.c_void_p()
        F.check(lib.ti_symm_alloc(ctypes.byref(p), nbytes), "ti_symm_alloc")
        self._local.append(p.value)
        if self.tp == 1:
            return [p.value]
        hs = lib.ti_ipc_handle_size()
        buf = ctypes.create_string_buffer(hs)
        F.check(lib.ti_ipc_get_handle(p, buf), "ti_ipc_get_handle")
        import torch.distributed as dist
        handles = [None] * self.tp
        dist.all_gather_object(handles, bytes(buf.raw))
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(p.value)
                continue
            q = ctypes.c_void_p()
            F.check(lib.ti_ipc_open(ctypes.create_string_buffer(h, hs), ctypes.byref(q)), "ti_ipc_open")
            self._mapped.append(q.value)
            ptrs.append(q.value)
        torch.cuda.synchronize()
        self.comm.barrier()
        return ptrs

    SCRUB_PERIOD = 1 << 15

    def tick(self, steps: int = 1):
        """Called once per forward (eager or graph replay), by every rank in lockstep.  A tag is
        step * 65536 + position, so it recurs after 2^16 steps; a row of a packet buffer that was last
        written exactly that long ago (a batch size not used since) could then be mistaken for fresh
        data.  Every 2^15 steps all ranks therefore drain, zero their own buffers and meet again
        before any of them sends the next packet."""
        self._steps = getattr(self, "_steps", 0) + steps
        if self.tp > 1 and self._steps >= self.SCRUB_PERIOD:
            self._steps = 0
            self.scrub()

    def scrub(self):
        lib = F.L()
        torch.cuda.synchronize()
        self.comm.barrier()                   # nobody is still sending into anybody's buffer
        for ptr, n in zip(self._local, (self.ll_bytes, self.cand_bytes)):
            F.check(lib.ti_memset_async(ctypes.c_void_p(ptr), 0, n, None), "ti_memset_async")
        # The flags of the many-row all-reduce are compared modulo 2^32 ("at least this tag"): a flag left behind by a
        # collective more than 2^15 steps ago would look AHEAD of the next tags.  All ranks are at the same step here:
        # every flag is put just behind the tags that come next (the block counter of the two-shot form stays zero).
        if self.tp > 1:
            flags = _tensor_from_ptr(self.flag_ptrs[self.rank], 64, torch.int32, self.device)
            vals = torch.full((64,), flag_rebase_value(int(self.ctrl[0].item())), dtype=torch.int32)
            vals[FLAG_COUNTER_WORD] = 0
            flags.copy_(vals.to(self.device))
        torch.cuda.synchronize()
        self.comm.barrier()                   # nobody sends before every buffer is clean
        self.scrubs = getattr(self, "scrubs", 0) + 1

    def status(self) -> int:
        """Error bits raised by kernels (1 = a peer wait timed out).  Synchronises."""
        return int(self.ctrl[1].item())

    def clear_status(self):
        self.ctrl[1] = 0

    def close(self, collective: bool = True):
        """Unmaps the peers' buffers and frees the local ones.  collective=False skips the barrier between the two
        (a peer is gone: nobody will write into the local buffers any more, and nobody can answer a barrier)."""
        lib = F.L()
        torch.cuda.synchronize()
        for q in self._mapped:
            lib.ti_ipc_close(ctypes.c_void_p(q))
        self._mapped = []
        if self.tp > 1 and collective:
            self.comm.barrier()
        for p in self._local:
            lib.ti_symm_free(ctypes.c_void_p(p))
        self._local = []


FLAG_COUNTER_WORD = 16      # 2 * kMaxRanks in ops/csrc/fused_ar.cu: finished blocks of the two-shot reduce kernel


def flag_rebase_value(step: int) -> int:
    """The int32 bit pattern of step * 65536: the largest value every tag of this and of later steps (step * 65536 +
    position + 1, modulo 2^32) still counts as 'not reached'."""
    v = (step * 65536) & 0xFFFFFFFF
    return v - (1 << 32) if v >= (1 << 31) else v


class _PtrOwner:
    """Exposes raw device memory through __cuda_array_interface__ so that torch can wrap it without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _tensor_from_ptr(ptr: int, numel: int, dtype, device) -> torch.Tensor:
    nbytes = numel * torch.empty(0, dtype=dtype).element_size()
    return torch.as_tensor(_PtrOwner(ptr, nbytes), device=device).view(dtype)


class LocalRanks:
    """Several emulated ranks on ONE GPU (tests): same buffer layout, plain device pointers.  Kernels
    of all ranks must then run inside a single cooperative launch (`ti_gemv_ranks`)."""

    def __init__(self, tp: int, hidden: int, m_cap: int = 16, timeout_s: float = 1.0, device="cuda"):
        self.tp, self.m_cap, self.hidden = tp, m_cap, hidden
        self.timeout_ns = int(timeout_s * 1e9)
        n = 2 * tp * m_cap * (hidden // 2) * 4     # 16-byte pairs as int32 x4
        self.bufs = [torch.zeros(n, dtype=torch.int32, device=device) for _ in range(tp)]
        self.ctrl = torch.zeros(4, dtype=torch.int32, device=device)
        self.ctrl[0] = 1
        self.step_ptr = self.ctrl.data_ptr()
        self.status_ptr = self.ctrl.data_ptr() + 4
        self.ll_ptrs = [b.data_ptr() for b in self.bufs]

    def view(self, rank: int):
        class _V:
            pass
        v = _V()
        v.tp, v.rank, v.m_cap = self.tp, rank, self.m_cap
        v.ll_ptrs, v.step_ptr, v.status_ptr, v.timeout_ns = self.ll_ptrs, self.step_ptr, self.status_ptr, self.timeout_ns
        return v
