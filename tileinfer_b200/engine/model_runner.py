"""Execution runtime: builds the executor, owns the KV / DeltaNet pools and turns scheduled
sequences into one forward step.

Responsibilities match the reference's ModelRunner (engine/model_runner.py:48-1169): weight
loading and sharding, cache sizing and allocation, DeltaNet slot allocation, prefix-state
snapshots (host copies, LRU of max_prefix_states), batch building, sampling, and an OOM retry that
drops the last sequence of the batch (engine/model_runner.py:726-750).

What is different:
* the model is an explicit executor object (`TorchHybridModel` on CPU, `B200HybridModel` on the GPU)
  instead of monkey-patched HuggingFace layers;
* one step may mix prefill chunks of several sequences with decode tokens (variable-length batch);
* swap-out / swap-in of KV blocks plus DeltaNet state to host memory is implemented;
* DeltaNet snapshots are taken at the prompt positions the scheduler asks for, also inside a chunk.
"""
from __future__ import annotations

import logging
from collections import OrderedDict, deque

import torch

from ..models.reference_cpu import Batch, TorchHybridModel
from ..models.weights import make_weight_source
from .config import Config
from .sampler import Sampler
from .sequence import Sequence

log = logging.getLogger("tileinfer_b200")


class SimulatedOOM(RuntimeError):
    """Raised by tests (fault injection) in place of torch.cuda.OutOfMemoryError."""


class ModelRunner:
    def __init__(self, config: Config, comm):
        self.config = config
        self.comm = comm
        self.mc = config.model_config
        self.block_size = config.kvcache_block_size
        Sequence.block_size = self.block_size
        self.tp_size, self.tp_rank = config.tp_size, comm.rank
        self.model = None
        self.sampler = None
        self.num_slots = config.max_num_seqs + 1
        self.free_deltanet_slots: deque = deque()
        self.seq_to_slot: dict = {}
        self.oom_preempted: list = []
        self.prefix_state_cache: OrderedDict = OrderedDict()    # node_id -> (rec, conv) host tensors
        self.pinned_prefix_states: dict = {}                    # seq_id -> node_id it has yet to restore
        self.pending_snapshots: dict = {}                        # (seq_id, abs tokens) -> (rec, conv)
        self.max_prefix_states = config.max_prefix_states
        self.on_prefix_state_dropped = None                      # callable(node_id)
        self.swapped: dict = {}                                  # seq_id -> (kv host tensor, state)
        self.fault_hook = None                                   # tests: callable(seqs) may raise
        self.steps = 0
        self.last_batch_tokens = 0

    # ---- model / cache ----------------------------------------------------
    def load_model(self):
        cfg = self.config
        if cfg.device == "cuda":
            from ..models.hybrid_b200 import B200HybridModel
            src = make_weight_source(self.mc, cfg.weights, cfg.model, device="cuda")
            self.model = B200HybridModel(self.mc, src, quant=cfg.quantization, tp=self.tp_size,
                                         rank=self.tp_rank, comm=self.comm, config=cfg)
        else:
            src = make_weight_source(self.mc, cfg.weights, cfg.model, device="cpu")
            self.model = TorchHybridModel(self.mc, src, quant=cfg.quantization if cfg.quantization == "w8a16" else "none",
                                          tp=self.tp_size, rank=self.tp_rank, comm=self.comm)
        self.sampler = Sampler(self.comm, self.model.vocab_start, cfg.eos, seed=0,
                               full_vocab_gather=cfg.baseline_full_vocab_gather)
        self.sampler._v_local = getattr(self.model, "v_local", self.mc.vocab_size // self.tp_size)
        return self.model

    def allocate_kv_cache(self):
        cfg = self.config
        n = cfg.num_kvcache_blocks
        if n is None or n <= 0:
            if cfg.device == "cuda":
                n = self.model.auto_num_blocks(cfg.gpu_memory_utilization, self.block_size, self.num_slots,
                                               cfg.max_num_seqs, cfg.max_model_len)
            else:
                n = max(64, 2 * cfg.max_num_seqs * ((min(cfg.max_model_len, 4096) + self.block_size - 1) // self.block_size) // 8)
            cfg.num_kvcache_blocks = n
        self.model.alloc_cache(n, self.block_size, self.num_slots)
        # the last slot is reserved for CUDA-graph padding rows
        self.padding_deltanet_slot = self.num_slots - 1
        self.free_deltanet_slots = deque(range(self.num_slots - 1))
        log.info("kv cache: %d blocks x %d tokens, %d DeltaNet slots", n, self.block_size, self.num_slots)
        return n

    def block_bytes(self) -> int:
        return self.model.cache_bytes_per_block()

    def capture_decode_graphs(self):
        if self.config.device == "cuda" and not self.config.enforce_eager:
            self.model.capture_decode_graphs(self.config.max_num_seqs, self.config.cuda_graph_max_batch_size,
                                             self.config.max_model_len, self.padding_deltanet_slot)

    # ---- DeltaNet slots ---------------------------------------------------
    def allocate_slot(self, seq: Sequence) -> int:
        slot = self.seq_to_slot.get(seq.seq_id)
        if slot is None:
            if not self.free_deltanet_slots:
                raise RuntimeError("no free DeltaNet state slot (more sequences than max_num_seqs)")
            slot = self.free_deltanet_slots.popleft()
            self.seq_to_slot[seq.seq_id] = slot
            self.model.zero_state(slot)
        seq.deltanet_state_slot = slot
        return slot

    def free_deltanet_slot(self, seq_id: int):
        slot = self.seq_to_slot.pop(seq_id, None)
        if slot is not None:
            self.free_deltanet_slots.append(slot)
        self.swapped.pop(seq_id, None)
        self.pinned_prefix_states.pop(seq_id, None)
        for key in [k for k in self.pending_snapshots if k[0] == seq_id]:
            del self.pending_snapshots[key]

    def reset_state(self, seq: Sequence):
        """Recompute preemption: the sequence restarts from an empty recurrent state."""
        self.free_deltanet_slot(seq.seq_id)
        seq.deltanet_state_slot = -1

    # ---- prefix-cache state snapshots --------------------------------------
    def save_prefix_state(self, seq: Sequence, node_id: int, num_tokens: int) -> bool:
        snap = self.pending_snapshots.pop((seq.seq_id, num_tokens), None)
        if snap is None:
            return False
        self.prefix_state_cache[node_id] = snap
        self.prefix_state_cache.move_to_end(node_id)
        # LRU, except snapshots a scheduled sequence still has to restore (its first chunk may run a step later)
        pinned = set(self.pinned_prefix_states.values())
        over = len(self.prefix_state_cache) - self.max_prefix_states
        for old in [k for k in self.prefix_state_cache if k not in pinned and k != node_id][:max(0, over)]:
            del self.prefix_state_cache[old]
            if self.on_prefix_state_dropped is not None:
                self.on_prefix_state_dropped(old)
        return True

    def has_prefix_state(self, seq: Sequence, node_id: int, num_tokens: int) -> bool:
        if node_id in self.prefix_state_cache:
            self.prefix_state_cache.move_to_end(node_id)
            self.pinned_prefix_states[seq.seq_id] = node_id
            return True
        return False

    def drop_prefix_state(self, node_id: int):
        if node_id not in self.pinned_prefix_states.values():
            self.prefix_state_cache.pop(node_id, None)

    # ---- swap ------------------------------------------------------------------
    def swap_out(self, seq: Sequence, dev_blocks: list, host_blocks: list):
        slot = self.seq_to_slot.get(seq.seq_id)
        kv = self.model.blocks_out(dev_blocks)
        st = self.model.state_out(slot) if slot is not None else None
        self.swapped[seq.seq_id] = (kv, st)
        if slot is not None:
            del self.seq_to_slot[seq.seq_id]
            self.free_deltanet_slots.append(slot)
            seq.deltanet_state_slot = -1

    def swap_in(self, seq: Sequence, host_blocks: list, dev_blocks: list):
        kv, st = self.swapped.pop(seq.seq_id)
        self.model.blocks_in(dev_blocks, kv)
        slot = self.allocate_slot(seq)
        if st is not None:
            self.model.state_in(slot, st)

    # ---- one step ---------------------------------------------------------------
    def run(self, seqs: list, is_prefill: bool = False) -> list:
        """Execute one step; returns a token id per sequence (-1: nothing sampled).  On an
        out-of-memory error the last sequence of the batch is dropped (recorded in
        `oom_preempted`) and the step retried, at most twice."""
        seqs = list(seqs)
        dropped = 0
        while True:
            try:
                out = self._run_impl(seqs)
                return out + [-1] * dropped
            except (torch.cuda.OutOfMemoryError, SimulatedOOM) as e:
                if dropped >= 2 or len(seqs) <= 1:
                    raise RuntimeError(
                        f"out of memory running a batch of {len(seqs)} sequences after {dropped} retries; "
                        "lower max_num_seqs / max_num_batched_tokens or gpu_memory_utilization") from e
                if torch.cuda.is_available():
                    torch.cuda.empty_cache()
                self.oom_preempted.append(seqs.pop())
                dropped += 1

    def build_batch(self, seqs: list) -> Batch:
        bs = self.block_size
        ids, pos, slots = [], [], []
        cu, ctx, tables, sslots, snaps = [0], [], [], [], []
        for seq in seqs:
            slot = self.allocate_slot(seq)
            if seq.prefix_restore_key is not None:
                self.model.state_in(slot, self.prefix_state_cache[seq.prefix_restore_key])
                seq.prefix_restore_key = None
                self.pinned_prefix_states.pop(seq.seq_id, None)
            start, n = seq.num_cached_tokens, seq.num_scheduled_tokens
            ids.extend(seq.token_ids[start:start + n])
            pos.extend(range(start, start + n))
            bt = seq.block_table
            slots.extend(bt[p // bs] * bs + p % bs for p in range(start, start + n))
            cu.append(cu[-1] + n)
            ctx.append(start + n)
            tables.append(bt)
            sslots.append(slot)
            snaps.append(list(seq.snapshot_points) if seq.is_prefill else [])
        return Batch(torch.tensor(ids, dtype=torch.long), torch.tensor(pos, dtype=torch.long), cu, ctx, tables,
                     torch.tensor(slots, dtype=torch.long), sslots, snaps)

    def _run_impl(self, seqs: list) -> list:
        if self.fault_hook is not None:
            self.fault_hook(seqs)
        self.steps += 1
        batch = self.build_batch(seqs)
        self.last_batch_tokens = batch.cu_seqlens[-1]
        sample_rows = [i for i, s in enumerate(seqs) if s.num_cached_tokens + s.num_scheduled_tokens >= s.num_tokens]
        sample_seqs = [seqs[i] for i in sample_rows]
        fast = getattr(self.model, "forward_and_sample", None)
        k = self.sampler.num_candidates(sample_seqs) if sample_rows else 1
        edits = self.sampler.edit_rows(sample_seqs) if sample_rows else []
        if (fast is not None and sample_rows and not self.sampler.full_vocab_gather
                and k <= self.sampler.max_device_candidates and len(edits) <= self.model.EDIT_SLOTS):
            # GPU path: lm_head, logit edits, per-rank top-k (+ candidate exchange) and the draw itself run as
            # kernels; what comes back is the chosen token id per row and the peer status word
            spec = self.sampler.device_spec(sample_seqs, edits)
            toks = fast(batch, sample_rows, k, spec)
            self._collect_snapshots(seqs)
        else:
            # host path: more than 64 candidates or more edited rows than the device buffers hold, the
            # full-vocabulary-gather baseline, and the CPU executor
            hidden = self.model.forward(batch)
            self._collect_snapshots(seqs)
            toks = []
            if sample_rows:
                logits = self.model.logits(hidden[torch.tensor(sample_rows, device=hidden.device)])
                toks = self.sampler.sample(logits, sample_seqs)
        out = [-1] * len(seqs)
        for r, t in zip(sample_rows, toks):
            out[r] = int(t)
        return out

    def _collect_snapshots(self, seqs):
        for (si, abs_tokens), snap in self.model.take_snapshots().items():
            self.pending_snapshots[(seqs[si].seq_id, abs_tokens)] = snap
