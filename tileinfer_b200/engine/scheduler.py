"""Continuous-batching scheduler: decode-first, chunked varlen prefill, true mixed batches,
SWAP (or RECOMPUTE) preemption, prefix reuse and multi-step decode.

Semantics kept from the reference (engine/scheduler.py:68-293): running sequences are scheduled
for one decode token each before any prefill; a victim is the most recently admitted running
sequence and at most max_num_seqs//4 are preempted per step; prompts are prefilled in chunks of at
most max_prefill_chunk_tokens inside the max_num_batched_tokens budget; EOS / max_tokens / grammar
completion / stop strings finish a sequence.

Deliberate differences:
* a step may contain prefill chunks of several sequences AND decode tokens; the runner executes
  them as one variable-length batch (the reference schedules such a batch but runs every sequence
  as a 1-token decode, engine/model_runner.py:776-798);
* preemption swaps KV blocks and DeltaNet state to host memory when swap space is configured,
  and falls back to recompute otherwise;
* non-final prefill chunks end on a block boundary, DeltaNet snapshots are requested at
  deterministic prompt positions, only prefilled blocks are registered in the prefix cache and a
  cached prefix never covers the whole prompt (at least one token is always computed);
* `finish_reason` records "stop" or "length".
"""
from __future__ import annotations

from collections import OrderedDict, deque

from .block_manager import BlockManager
from .config import Config
from .constraints import advance_constraint, constraint_complete
from .prefix_cache import PrefixCache
from .sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config: Config, tokenizer=None, block_bytes: int = 0):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.max_prefill_chunk_tokens = config.max_prefill_chunk_tokens
        self.eos = list(config.eos or [])
        self.block_size = config.kvcache_block_size
        self.state_stride = config.prefix_state_stride
        ncpu = config.swap_space_bytes // block_bytes if block_bytes > 0 else 0
        self.block_manager = BlockManager(config.num_kvcache_blocks, self.block_size, ncpu)
        self.waiting: deque = deque()
        self.running: OrderedDict = OrderedDict()
        self.swapped: deque = deque()
        self.tokenizer = tokenizer
        self.max_preempt_count = max(1, config.max_num_seqs // 4)
        self.enable_prefix_caching = config.enable_prefix_caching
        self.prefix_cache = PrefixCache(self.block_size, self.block_manager)
        if self.enable_prefix_caching:
            self.block_manager.evictor = self.prefix_cache.evict
            self.block_manager.evictable = self.prefix_cache.num_evictable
        # callbacks wired by the engine
        self.on_preempt = None          # (seq)                       recompute preemption: drop state
        self.on_swap_out = None         # (seq, dev_blocks, host_blocks)
        self.on_swap_in = None          # (seq, host_blocks, dev_blocks)
        self.on_prefix_hit = None       # (seq, node_id, num_tokens) -> bool
        self.on_prefix_save = None      # (seq, node_id, num_tokens) -> bool
        self.on_block_freed = None
        self.block_manager.on_block_freed = self._on_block_freed
        # counters
        self.num_preemptions = 0
        self.num_swaps_out = 0
        self.num_swaps_in = 0
        self.num_recomputes = 0

    # ---- queue helpers -----------------------------------------------------
    def is_finished(self):
        return not self.waiting and not self.running and not self.swapped

    def add(self, seq: Sequence):
        self.waiting.append(seq)

    def _on_block_freed(self, block_id: int):
        if self.on_block_freed is not None:
            self.on_block_freed(block_id)

    def deallocate(self, seq: Sequence):
        self.block_manager.deallocate(seq)

    # ---- scheduling --------------------------------------------------------
    def schedule(self):
        """Returns (scheduled_seqs, is_prefill): prefill chunks first, then decode sequences.

        `is_prefill` is True only when no decode sequence is in the step (reference contract).
        Each sequence carries `num_scheduled_tokens` and `is_prefill`.
        """
        bm = self.block_manager
        decode_seqs, prefill_seqs = [], []
        budget = self.max_num_batched_tokens
        preempted = 0

        # 0) bring swapped sequences back first (FIFO), before admitting new work
        while self.swapped and len(self.running) < self.max_num_seqs:
            seq = self.swapped[0]
            if not bm.can_swap_in(seq):
                break
            self.swapped.popleft()
            host, dev = bm.swap_in(seq)
            if self.on_swap_in is not None:
                self.on_swap_in(seq, host, dev)
            seq.status = SequenceStatus.RUNNING
            self.running[seq.seq_id] = seq
            self.num_swaps_in += 1

        # 1) decode: one token for every running sequence that has finished its prefill
        for seq in list(self.running.values()):
            if seq.seq_id not in self.running:        # preempted earlier in this loop
                continue
            if seq.is_prefill:
                continue                               # prompt not finished (handled below)
            if len(decode_seqs) >= self.max_num_seqs or budget <= 0:
                break
            ok = True
            while not bm.can_append(seq):
                if preempted >= self.max_preempt_count or not self._preempt_victim(seq, decode_seqs):
                    ok = False
                    break
                preempted += 1
            if not ok:
                # nothing else to evict: preempt this sequence itself and stop
                self._preempt_seq(seq)
                break
            seq.num_scheduled_tokens = 1
            seq.is_prefill = False
            bm.may_append(seq)
            decode_seqs.append(seq)
            budget -= 1

        # 2) prefill: running sequences with an unfinished prompt first, then new arrivals
        partial = [s for s in self.running.values() if s.is_prefill and s.num_cached_tokens < s.num_tokens]
        for seq in partial:
            if budget <= 0:
                break
            budget -= self._schedule_chunk(seq, budget, prefill_seqs)
        while (self.waiting and budget > 0 and not self.swapped and preempted == 0
               and len(self.running) < self.max_num_seqs):
            seq = self.waiting[0]
            if not seq.block_table and not self._allocate_blocks_for_new_seq(seq):
                break
            self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            seq.is_prefill = True
            self.running[seq.seq_id] = seq
            budget -= self._schedule_chunk(seq, budget, prefill_seqs)

        scheduled = prefill_seqs + decode_seqs
        return scheduled, bool(scheduled) and not decode_seqs

    def _schedule_chunk(self, seq: Sequence, budget: int, out: list) -> int:
        remaining = seq.num_tokens - seq.num_cached_tokens
        chunk = min(remaining, budget, self.max_prefill_chunk_tokens)
        if chunk < remaining:
            # a non-final chunk ends on a block boundary
            end = (seq.num_cached_tokens + chunk) // self.block_size * self.block_size
            chunk = end - seq.num_cached_tokens
            if chunk <= 0:
                return 0
        seq.num_scheduled_tokens = chunk
        seq.is_prefill = True
        seq.snapshot_points = self._snapshot_points(seq, seq.num_cached_tokens, seq.num_cached_tokens + chunk)
        out.append(seq)
        return chunk

    def _snapshot_points(self, seq: Sequence, lo: int, hi: int) -> list:
        """Prompt positions in (lo, hi] at which the DeltaNet state is captured for prefix reuse:
        stride * 2^j, block-aligned chunk ends, and the last block boundary below the prompt end."""
        if not self.enable_prefix_caching or seq.num_completion_tokens > 0:
            return []
        bs, pts = self.block_size, set()
        p = self.state_stride
        while p <= hi:
            if p > lo:
                pts.add(p)
            p *= 2
        if hi % bs == 0:
            pts.add(hi)
        last = (seq.num_prompt_tokens - 1) // bs * bs
        if lo < last <= hi:
            pts.add(last)
        return sorted(x for x in pts if 0 < x <= seq.num_prompt_tokens)

    def _allocate_blocks_for_new_seq(self, seq: Sequence) -> bool:
        bm = self.block_manager
        if self.enable_prefix_caching and seq.num_completion_tokens == 0:
            chain, n = self.prefix_cache.find_longest_prefix(seq.token_ids, seq.num_tokens - 1)
            if chain:
                # Take the chain's references BEFORE the capacity check: once shared, these blocks are no longer
                # evictable, so they must not be counted among the blocks the remainder of the prompt may take.
                bm.share_blocks(seq, [c.block_id for c in chain])
                if bm.can_append(seq) and (self.on_prefix_hit is None
                                           or self.on_prefix_hit(seq, chain[-1].node_id, n)):
                    bm.allocate_extra(seq)
                    seq.num_cached_tokens = n
                    seq.prefix_restore_key = chain[-1].node_id
                    return True
                bm.deallocate(seq)          # give the references back; the cache still holds its own
        if bm.can_allocate(seq):
            bm.allocate(seq)
            return True
        return False

    def advance_decode(self, seqs: list) -> list:
        """Between the sub-steps of multi-step decode: reserve the next KV slot of each sequence.
        Returns the sequences that can continue (others were preempted)."""
        alive = []
        for seq in seqs:
            if seq.seq_id not in self.running:
                continue
            if not self.block_manager.can_append(seq):
                if not self._preempt_victim(seq, alive):
                    self._preempt_seq(seq)
                    continue
                if not self.block_manager.can_append(seq):
                    self._preempt_seq(seq)
                    continue
            seq.num_scheduled_tokens = 1
            seq.is_prefill = False
            self.block_manager.may_append(seq)
            alive.append(seq)
        return [s for s in alive if s.seq_id in self.running]

    # ---- preemption ----------------------------------------------------------
    def _preempt_victim(self, exclude: Sequence, protected=()) -> bool:
        for sid in reversed(self.running):
            victim = self.running[sid]
            if victim is not exclude and victim.block_table and all(victim is not p for p in protected):
                self._preempt_seq(victim)
                return True
        return False

    def _preempt_seq(self, seq: Sequence):
        bm = self.block_manager
        self.running.pop(seq.seq_id, None)
        self.num_preemptions += 1
        seq.num_preemptions += 1
        seq.num_scheduled_tokens = 0
        fully_prefilled = seq.num_cached_tokens >= seq.num_tokens - 1
        if fully_prefilled and bm.can_swap_out(seq):
            dev, host = bm.swap_out(seq)
            if self.on_swap_out is not None:
                self.on_swap_out(seq, dev, host)
            seq.status = SequenceStatus.SWAPPED
            self.swapped.append(seq)
            self.num_swaps_out += 1
            return
        # RECOMPUTE: drop everything, re-prefill prompt + generated tokens later
        self.num_recomputes += 1
        seq.status = SequenceStatus.WAITING
        seq.is_prefill = True
        seq.num_cached_tokens = 0
        seq.prefix_restore_key = None
        bm.deallocate(seq)
        if self.on_preempt is not None:
            self.on_preempt(seq)
        self.waiting.appendleft(seq)

    def preempt(self, seq: Sequence):
        self._preempt_seq(seq)

    # ---- post-processing -----------------------------------------------------
    def postprocess(self, seqs: list, token_ids: list, is_prefill: bool = False):
        """Advance counters, register prefilled blocks, append sampled tokens, finish sequences.
        `token_ids[i]` is -1 for a sequence that did not sample (non-final prefill chunk)."""
        for i, seq in enumerate(seqs):
            if seq.status != SequenceStatus.RUNNING:
                continue                                    # preempted while the step ran
            was_prefill = seq.is_prefill
            seq.num_cached_tokens += seq.num_scheduled_tokens
            seq.num_scheduled_tokens = 0
            if was_prefill and self.enable_prefix_caching and seq.num_completion_tokens == 0:
                self._register_prefix(seq)
            if seq.num_cached_tokens < seq.num_tokens:
                continue                                    # more prompt chunks to go
            token_id = token_ids[i] if i < len(token_ids) else -1
            if token_id is None or token_id < 0:
                continue
            seq.is_prefill = False
            seq.append_token(token_id)
            advance_constraint(seq, token_id)
            reason = None
            if not seq.ignore_eos and token_id in self.eos:
                reason = "stop"
            elif constraint_complete(seq):
                reason = "stop"
            elif seq.stop and self.tokenizer is not None and self._hit_stop_string(seq):
                reason = "stop"
            if reason is None and seq.num_completion_tokens >= seq.max_tokens:
                reason = "length"
            if reason is not None:
                seq.finish_reason = reason
                seq.status = SequenceStatus.FINISHED
                self.block_manager.deallocate(seq)
                self.running.pop(seq.seq_id, None)

    def _hit_stop_string(self, seq: Sequence) -> bool:
        # only the tail can contain a new match: decode a bounded window, not the whole completion
        longest = max(len(s) for s in seq.stop)
        tail = seq.completion_token_ids[-(longest + 8):]
        text = self.tokenizer.decode(tail, skip_special_tokens=True)
        return any(s in text for s in seq.stop)

    def _register_prefix(self, seq: Sequence):
        bs = self.block_size
        n_full = min(seq.num_cached_tokens, seq.num_prompt_tokens) // bs
        if n_full == 0:
            return
        chain = self.prefix_cache.insert(seq.token_ids, seq.block_table, n_full)
        for p in seq.snapshot_points:
            if p % bs == 0 and 0 < p // bs <= len(chain) and p <= seq.num_cached_tokens:
                node = chain[p // bs - 1]
                if not node.has_state and self.on_prefix_save is not None:
                    if self.on_prefix_save(seq, node.node_id, p):
                        node.has_state = True
        seq.snapshot_points = []
