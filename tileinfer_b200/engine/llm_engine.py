"""Engine orchestrator: request intake, the step loop, multi-step decode and the generate APIs.

Public surface and start-up order follow the reference (engine/llm_engine.py:30-331): Config ->
init_distributed -> tokenizer -> ModelRunner.load_model -> allocate_kv_cache -> barrier ->
capture_decode_graphs -> barrier -> Scheduler with callbacks.  `generate` returns dicts with
text / prompt / token_ids / prompt_token_ids, `generate_stream` yields (index, text, finished).

Additions: prompts may be token-id lists, each result also carries `finish_reason`, `stats()`
reports counters and latency percentiles, and multi-step decode keeps running sequences that are
preempted or finish in the middle of the multi-step window out of the next sub-step.
"""
from __future__ import annotations

import logging
import time

from ..parallel.comm import init_distributed
from ..utils.tokenizer import load_tokenizer
from .config import Config
from .constraints import make_constraint
from .model_runner import ModelRunner
from .sampling_params import SamplingParams
from .scheduler import Scheduler
from .sequence import Sequence, SequenceStatus
from .stats import EngineStats

log = logging.getLogger("tileinfer_b200")


class LLMEngine:
    def __init__(self, model: str, comm=None, **kwargs):
        self.config = Config(model, **kwargs)
        cfg = self.config
        self._owns_process_group = comm is None and cfg.tp_size > 1      # close() then also destroys the process group
        self.comm = comm if comm is not None else init_distributed(cfg.tp_size, cfg.nccl_timeout, cfg.device)
        if self.comm.world_size != cfg.tp_size:
            raise RuntimeError(f"communicator has {self.comm.world_size} ranks, tp_size={cfg.tp_size}")
        self.tokenizer = load_tokenizer(cfg)
        if not cfg.eos and getattr(self.tokenizer, "eos_token_id", None) is not None:
            cfg.eos = [self.tokenizer.eos_token_id]
        self.model_runner = ModelRunner(cfg, self.comm)
        self.model_runner.load_model()
        self.model_runner.allocate_kv_cache()
        self.comm.barrier()
        self.model_runner.capture_decode_graphs()
        self.comm.barrier()
        self.scheduler = Scheduler(cfg, self.tokenizer, block_bytes=self.model_runner.block_bytes())
        r, s = self.model_runner, self.scheduler
        s.on_preempt = r.reset_state
        s.on_swap_out = r.swap_out
        s.on_swap_in = r.swap_in
        s.on_prefix_hit = r.has_prefix_state
        s.on_prefix_save = r.save_prefix_state
        s.prefix_cache.on_node_evicted = r.drop_prefix_state
        r.on_prefix_state_dropped = lambda node_id: s.prefix_cache.mark_state(node_id, False)
        self._all_seqs = {}
        self._stats = EngineStats()
        # host-side peer watchdog (tensor parallelism): a dead rank is noticed before the next launch
        self.watchdog = None
        if cfg.tp_size > 1 and cfg.heartbeat_interval > 0:
            from ..parallel.watchdog import Heartbeat, default_store
            store = default_store()
            if store is not None:
                self.watchdog = Heartbeat(store, self.comm.rank, self.comm.world_size, interval_s=cfg.heartbeat_interval,
                                          timeout_s=cfg.heartbeat_timeout).start()

    # ---- requests ---------------------------------------------------------
    def add_request(self, prompt, sampling_params: SamplingParams | None = None) -> Sequence:
        sp = sampling_params or SamplingParams()
        if isinstance(prompt, str):
            token_ids = self.tokenizer.encode(prompt, add_special_tokens=True)
        else:
            token_ids = [int(t) for t in prompt]
        max_len = self.config.max_model_len
        if len(token_ids) > max_len:
            raise ValueError(f"Prompt has {len(token_ids)} tokens, exceeds max_model_len={max_len}. "
                             "Truncate the prompt or increase max_model_len.")
        if len(token_ids) == 0:
            raise ValueError("Prompt produced no tokens after tokenization")
        vs = self.config.model_config.vocab_size
        if any(t < 0 or t >= vs for t in token_ids):
            raise ValueError(f"prompt token id outside [0, {vs})")
        seq = Sequence(token_ids, sp)
        seq.max_tokens = min(sp.max_tokens, max(1, max_len - len(token_ids)))
        seq.constraint = make_constraint(sp, self.tokenizer)
        self.scheduler.add(seq)
        self._all_seqs[seq.seq_id] = seq
        return seq

    # ---- stepping ---------------------------------------------------------
    def step(self) -> list:
        """One scheduling step.  Returns the sequences that finished in it."""
        if self.watchdog is not None:
            self.watchdog.check()                     # raises PeerLostError: no launch that would wait for a dead rank
        seqs, is_prefill = self.scheduler.schedule()
        if not seqs:
            return []
        if (not is_prefill and self.config.num_scheduler_steps > 1
                and all(not s.is_prefill for s in seqs)):
            return self._multi_step_decode(seqs)
        return self._run_and_post(seqs, is_prefill)

    def _run_and_post(self, seqs, is_prefill) -> list:
        t0 = time.perf_counter()
        self.model_runner.oom_preempted.clear()
        npre = sum(s.num_scheduled_tokens for s in seqs if s.is_prefill)
        ndec = sum(1 for s in seqs if not s.is_prefill)
        before = [s.num_tokens for s in seqs]
        token_ids = self.model_runner.run(seqs, is_prefill)
        self._handle_preempted()
        self.scheduler.postprocess(seqs, token_ids, is_prefill)
        now = time.perf_counter()
        for s, b in zip(seqs, before):
            if s.num_tokens > b:
                self._stats.on_token(s, now)
        self._stats.on_step(npre, ndec, (now - t0) * 1e3)
        return self._finalize_finished(seqs)

    def _handle_preempted(self):
        for seq in self.model_runner.oom_preempted:
            self._stats.oom_retries += 1
            if seq.status == SequenceStatus.RUNNING:
                self.scheduler.running.pop(seq.seq_id, None)
                seq.status = SequenceStatus.WAITING
                seq.is_prefill = True
                seq.num_cached_tokens = 0
                seq.num_scheduled_tokens = 0
                seq.prefix_restore_key = None
                self.scheduler.deallocate(seq)
                self.model_runner.reset_state(seq)
                self.scheduler.waiting.appendleft(seq)
        self.model_runner.oom_preempted.clear()

    def _finalize_finished(self, seqs) -> list:
        finished = [s for s in seqs if s.is_finished]
        for seq in finished:
            self.model_runner.free_deltanet_slot(seq.seq_id)
            self._all_seqs.pop(seq.seq_id, None)
            self._stats.finished += 1
        return finished

    def _multi_step_decode(self, seqs) -> list:
        batch, finished = list(seqs), []
        for k in range(self.config.num_scheduler_steps):
            if not batch:
                break
            finished.extend(self._run_and_post(batch, False))
            batch = [s for s in batch if s.status == SequenceStatus.RUNNING]
            if batch and k + 1 < self.config.num_scheduler_steps:
                batch = self.scheduler.advance_decode(batch)
        return finished

    # ---- generation APIs ------------------------------------------------------
    def _submit(self, prompts, sampling_params):
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        return [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]

    def _drain(self):
        idle = 0
        while not self.scheduler.is_finished():
            before = self.model_runner.steps
            self.step()
            idle = idle + 1 if self.model_runner.steps == before else 0
            if idle > 1000:
                raise RuntimeError("scheduler made no progress for 1000 steps (KV cache too small for one request?)")

    def generate(self, prompts, sampling_params=None) -> list:
        seqs = self._submit(prompts, sampling_params)
        try:
            self._drain()
        finally:
            self._cleanup_seqs(seqs)
        outs = []
        for seq in seqs:
            ids = seq.completion_token_ids
            outs.append({
                "text": self.tokenizer.decode(ids, skip_special_tokens=True),
                "prompt": self.tokenizer.decode(seq.prompt_token_ids, skip_special_tokens=True),
                "token_ids": ids,
                "prompt_token_ids": seq.prompt_token_ids,
                "finish_reason": seq.finish_reason or "stop",
            })
        return outs

    def generate_stream(self, prompts, sampling_params=None):
        """Yields (sequence index, token text, is_finished) as tokens are produced."""
        seqs = self._submit(prompts, sampling_params)
        done_idx = {}
        yielded = [0] * len(seqs)
        try:
            while not self.scheduler.is_finished():
                self.step()
                for i, seq in enumerate(seqs):
                    ids = seq.completion_token_ids
                    while yielded[i] < len(ids):
                        tok = ids[yielded[i]]
                        yielded[i] += 1
                        last = seq.is_finished and yielded[i] == len(ids)
                        yield (i, self.tokenizer.decode([tok], skip_special_tokens=True), last)
        finally:
            self._cleanup_seqs(seqs)

    def generate_token_ids(self, prompts, sampling_params=None) -> list:
        seqs = self._submit(prompts, sampling_params)
        try:
            self._drain()
        finally:
            self._cleanup_seqs(seqs)
        return [seq.completion_token_ids for seq in seqs]

    def _cleanup_seqs(self, seqs):
        for seq in seqs:
            if not seq.is_finished:
                # aborted (exception / generator closed): release everything the request holds
                self.scheduler.running.pop(seq.seq_id, None)
                for q in (self.scheduler.waiting, self.scheduler.swapped):
                    try:
                        q.remove(seq)
                    except ValueError:
                        pass
                self.scheduler.deallocate(seq)
                seq.status = SequenceStatus.FINISHED
                seq.finish_reason = seq.finish_reason or "abort"
            self.model_runner.free_deltanet_slot(seq.seq_id)
            self._all_seqs.pop(seq.seq_id, None)

    def close(self):
        """Orderly shutdown (every rank calls it): captured decode graphs go first (graphs that captured NCCL
        collectives must not outlive the communicator), then the peer-memory buffers, then the process group this
        engine created.  Safe to call twice; the CPU executor has nothing to release."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        if self.watchdog is not None and hasattr(self.watchdog, "stop"):
            self.watchdog.stop()
        model = getattr(self.model_runner, "model", None)
        if hasattr(model, "release_graphs"):
            model.release_graphs()
        peer = getattr(model, "peer", None)
        if peer is not None:
            peer.close()
            model.peer = None
        if getattr(self, "_owns_process_group", False):
            import torch.distributed as dist
            if dist.is_initialized():
                dist.barrier()
                dist.destroy_process_group()

    def stats(self) -> dict:
        return self._stats.snapshot(self.scheduler, self.model_runner)
