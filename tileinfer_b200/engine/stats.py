"""Engine counters and latency histograms (the reference only prints; see engine/parallel.py:56,
engine/model_runner.py:184-185,295-299).  `EngineStats.snapshot()` is what `LLM.stats()` returns."""
from __future__ import annotations

import time


def _pct(xs, q):
    if not xs:
        return None
    xs = sorted(xs)
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


class EngineStats:
    def __init__(self):
        self.start = time.perf_counter()
        self.steps = 0
        self.prefill_tokens = 0
        self.decode_tokens = 0
        self.generated_tokens = 0
        self.finished = 0
        self.batch_sizes = []
        self.ttft_ms = []
        self.itl_ms = []
        self.step_ms = []
        self.oom_retries = 0

    def on_step(self, num_prefill_tokens, num_decode, ms):
        self.steps += 1
        self.prefill_tokens += num_prefill_tokens
        self.decode_tokens += num_decode
        self.batch_sizes.append(num_prefill_tokens + num_decode)
        self.step_ms.append(ms)
        if len(self.batch_sizes) > 100000:
            del self.batch_sizes[:50000], self.step_ms[:50000]

    def on_token(self, seq, now):
        self.generated_tokens += 1
        if seq.first_token_time is None:
            seq.first_token_time = now
            self.ttft_ms.append((now - seq.arrival_time) * 1e3)
        elif seq.token_times:
            self.itl_ms.append((now - seq.token_times[-1]) * 1e3)
        seq.token_times.append(now)

    def snapshot(self, scheduler=None, runner=None) -> dict:
        d = {
            "uptime_s": time.perf_counter() - self.start,
            "steps": self.steps,
            "prefill_tokens": self.prefill_tokens,
            "decode_tokens": self.decode_tokens,
            "generated_tokens": self.generated_tokens,
            "finished_requests": self.finished,
            "mean_batch_tokens": (sum(self.batch_sizes) / len(self.batch_sizes)) if self.batch_sizes else 0.0,
            "ttft_ms_p50": _pct(self.ttft_ms, 0.5), "ttft_ms_p99": _pct(self.ttft_ms, 0.99),
            "itl_ms_p50": _pct(self.itl_ms, 0.5), "itl_ms_p99": _pct(self.itl_ms, 0.99),
            "step_ms_p50": _pct(self.step_ms, 0.5),
            "oom_retries": self.oom_retries,
        }
        if scheduler is not None:
            bm = scheduler.block_manager
            d.update({
                "waiting": len(scheduler.waiting), "running": len(scheduler.running), "swapped": len(scheduler.swapped),
                "free_blocks": bm.num_free_blocks, "total_blocks": bm.num_blocks,
                "preemptions": scheduler.num_preemptions, "swaps_out": scheduler.num_swaps_out,
                "swaps_in": scheduler.num_swaps_in, "recomputes": scheduler.num_recomputes,
                "prefix_cache_nodes": len(scheduler.prefix_cache), "prefix_hits": scheduler.prefix_cache.hits,
                "prefix_hit_tokens": scheduler.prefix_cache.hit_tokens, "prefix_queries": scheduler.prefix_cache.queries,
            })
        if runner is not None:
            d["prefix_states"] = len(runner.prefix_state_cache)
        return d
