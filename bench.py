"""Headline benchmark: batch-1 greedy decode of the Qwen3.6-27B architecture in W8A16 at TP = N.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 2 --steps 64 --warmup 8

A step is one decode token after a 128-token prompt (random token ids, random-init weights).
`value` is decode tokens/s timed on the device with CUDA events around exactly K steps (CUDA-graph
replays whose inputs advance on the device), max over ranks.  `e2e` is the same metric through
`LLM.generate_token_ids`, every step including the pinned-host -> device copy of its inputs and the
device -> host read of the sampled token; like the reference's own harness
(tests/bench_multi_gpu.py:57-115) it subtracts a max_tokens=1 call from a full call.
`--impl reference` runs the unmodified reference package from baseline/_ref instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_TOK_S = 36.6          # reference README: INT8 W8A16 decode at TP=2 on 2x A100-40GB
PROMPT_LEN = 128


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t0=None, t1=None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if (t0 is None or t >= t0) and (t1 is None or t <= t1)] or [r for _, r in self.rows]
        sm, mx, reasons = [], None, set()
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    from tileinfer_b200.models.reference_cpu import Batch

    n = args.gpus
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    K, W = args.steps, args.warmup
    total_len = PROMPT_LEN + 2 * (K + W) + 64
    llm = LLM(args.model, quantization="w8a16", tp_size=n, max_num_seqs=2, max_model_len=max(1024, total_len),
              num_kvcache_blocks=max(256, 3 * (total_len // 16 + 2)), enable_prefix_caching=False,
              gpu_memory_utilization=0.9)
    model = llm.model_runner.model
    comm = llm.comm
    g = torch.Generator().manual_seed(1234)
    vocab = llm.config.model_config.vocab_size

    def prompt():
        return torch.randint(0, vocab - 1, (PROMPT_LEN,), generator=g).tolist()

    # ---------------- device-timed: prefill, then K graph replays with on-device input advance
    nblk = total_len // 16 + 2
    table = list(range(nblk))                       # blocks of an otherwise idle cache
    p = prompt()
    model.zero_state(0)
    ids = torch.tensor(p)
    slots = torch.arange(PROMPT_LEN)
    first = model.forward_and_sample(
        Batch(ids, torch.arange(PROMPT_LEN), [0, PROMPT_LEN], [PROMPT_LEN], [table], slots, [0]), [0], 1)[0]
    b = Batch(torch.tensor([first]), torch.tensor([PROMPT_LEN]), [0, 1], [PROMPT_LEN + 1], [table],
              torch.tensor([PROMPT_LEN]), [0])
    model.forward_and_sample(b, [0], 1)
    gr = model.decode_graph(1, 1)
    x = gr.x

    def advance():
        # next token = the id the in-graph sample kernel chose (the same on every rank); positions and KV slots move on
        x.ids.copy_(gr.samp.tok[:1])
        x.positions.add_(1)
        x.slot_mapping.add_(1)

    for _ in range(W):
        advance()
        gr.graph.replay()
    torch.cuda.synchronize()
    comm.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    t0 = time.perf_counter()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
    evs[0].record()
    for i in range(K):
        advance()
        gr.graph.replay()
        evs[i + 1].record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    comm.barrier()
    clocks = sampler.stop(t0, t1)
    dev_ms = evs[0].elapsed_time(evs[K])
    step_ms = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(K))
    p50_ms, p99_ms = step_ms[K // 2], step_ms[min(K - 1, int(0.99 * K))]
    status = model.peer_status()

    # ---------------- end to end through the public API (H2D inputs + D2H token every step)
    sp1 = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    spk = SamplingParams(temperature=0.0, max_tokens=K + 1, ignore_eos=True)
    llm.generate_token_ids([prompt()], SamplingParams(temperature=0.0, max_tokens=W + 1, ignore_eos=True))   # warm-up

    def timed(sp):
        pr = prompt()
        torch.cuda.synchronize()
        comm.barrier()
        a, bb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = llm.generate_token_ids([pr], sp)
        bb.record()
        torch.cuda.synchronize()
        return a.elapsed_time(bb), out

    pre_ms, _ = timed(sp1)
    full_ms, out = timed(spk)
    assert len(out[0]) == K + 1
    e2e_ms = full_ms - pre_ms

    # max over ranks
    if n > 1:
        t = torch.tensor([dev_ms, e2e_ms, pre_ms, p50_ms, p99_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms, pre_ms, p50_ms, p99_ms = (float(v) for v in t.tolist())
    host = gr.host
    h2d = sum(v.numel() * v.element_size() for v in host.values()) + \
        gr.samp.h_fpar.numel() * 4 + gr.samp.h_ipar.numel() * 4
    d2h = gr.samp.h_tok.numel() * 4                    # the chosen token id + the peer status word
    checksum = 0
    for tkn in out[0]:
        checksum = (checksum * 1000003 + int(tkn)) % 2147483647
    from tileinfer_b200.models.weights import weight_bytes_per_rank
    wbytes = weight_bytes_per_rank(llm.config.model_config, n, "w8a16")
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    ms_step = dev_ms / K
    value = K / (dev_ms / 1e3)
    res = {
        "metric": "decode_tok_s", "value": round(value, 2), "unit": "tok/s", "n_gpus": n, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(value / BASELINE_TOK_S, 3),
        "dtype": "bf16 (W8A16: int8 weights; each bf16 activation row enters the integer tensor cores as a 16-bit "
                 "fixed-point number with one power-of-two exponent per row, int32 accumulate, bf16 scales)",
        "data": "synthetic: uniform-random prompt tokens, random-init N(0,0.02) weights",
        "config": {"model": llm.config.model_config.name, "global_batch": 1, "seq_len": PROMPT_LEN,
                   "decode_tokens": K, "parallelism": f"tp{n}", "cuda_graph": True,
                   "l2": "each step streams %.1f GB of weights per GPU, far more than the 126 MB L2" % (wbytes / 1e9)},
        "mean_itl_ms": round(ms_step, 4), "p50_itl_ms": round(p50_ms, 4), "p99_itl_ms": round(p99_ms, 4),
        "clocks": clocks,
        "e2e": {"value": round(K / (e2e_ms / 1e3), 2), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "itl_ms": round(e2e_ms / K, 4), "prefill_ms_128_tokens": round(pre_ms, 2),
                "vs_baseline": round(K / (e2e_ms / 1e3) / BASELINE_TOK_S, 3), "tokens_checksum": checksum},
        "gpu_launches": model.launches_per_decode_step * K,
        "launches_per_step": model.launches_per_decode_step,
        "hbm_roofline": {"weight_bytes_per_gpu": wbytes, "floor_ms": round(wbytes / (hbm * 1e6), 4),
                         "fraction_of_measured_hbm": round(wbytes / (hbm * 1e6) / ms_step, 3)},
        "peer_status": status,
        "impl": "tileinfer_b200",
    }
    return res if rank == 0 else None


def run_reference(args) -> dict:
    from baseline.run_reference import run
    return run(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="preset:qwen3.6-27b")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        try:
            res = run_reference(args)
        except Exception as e:      # the reference arm must never take the driver down
            res = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}".replace("\n", " ")}
        if res is not None:
            print(json.dumps(res), flush=True)
        return
    res = run_ours(args)
    if res is not None:
        print(json.dumps(res), flush=True)
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
