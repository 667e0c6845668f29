"""Batched decode sweep: tokens/s and inter-token latency statistics of the CUDA-graph decode step for batch sizes
1 .. 64 (every graph bucket), at a fixed context length.

Counterpart of the reference's tests/bench_batched_decode.py and of the statistics block of
model/generate.py:362-387 (mean / median / p95 / p99 over CUDA-event timings).  Every step is timed with its own pair
of CUDA events; between steps the inputs advance on the device (positions, KV slots, sampled ids), so a step is what
the engine replays minus the host scheduling.  Prints one JSON line per batch size and, with --out, a JSON file.

    python benchmarks/bench_batched_decode.py --model preset:qwen3.6-27b --ctx 1024 --steps 40
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_batched_decode.py
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from tileinfer_b200.engine.llm import LLM  # noqa: E402
from tileinfer_b200.models.reference_cpu import Batch  # noqa: E402


def stats(ms: list) -> dict:
    s = sorted(ms)
    pick = lambda q: s[min(len(s) - 1, int(q * len(s)))]
    return {"mean_ms": round(sum(s) / len(s), 4), "p50_ms": round(pick(0.5), 4), "p95_ms": round(pick(0.95), 4),
            "p99_ms": round(pick(0.99), 4), "min_ms": round(s[0], 4), "max_ms": round(s[-1], 4)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="preset:qwen3.6-27b")
    ap.add_argument("--tp", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--batches", default="1,2,4,8,16,32,64")
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--quantization", default="w8a16")
    ap.add_argument("--sample", action="store_true", help="temperature 0.6 / top-k 50 instead of greedy")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    batches = [int(b) for b in args.batches.split(",")]
    bmax = max(batches)
    per_seq = (args.ctx + args.steps + args.warmup + 32) // 16 + 2
    llm = LLM(args.model, tp_size=args.tp, quantization=args.quantization, max_num_seqs=bmax,
              max_model_len=args.ctx + args.steps + args.warmup + 64, num_kvcache_blocks=bmax * per_seq + 8,
              enable_prefix_caching=False, gpu_memory_utilization=0.9)
    model, comm = llm.model_runner.model, llm.comm
    vocab = llm.config.model_config.vocab_size
    k = 64 if args.sample else 1
    rows = []
    for B in batches:
        tables = [list(range(s * per_seq, (s + 1) * per_seq)) for s in range(B)]
        pos = args.ctx - 1
        batch = Batch(torch.randint(0, vocab - 1, (B,)), torch.full((B,), pos), list(range(B + 1)), [pos + 1] * B, tables,
                      torch.tensor([t[pos // 16] * 16 + pos % 16 for t in tables]), list(range(B)))
        spec = model._default_spec(B)
        if args.sample:
            spec.update(temperature=[0.6] * B, top_k=[50] * B, u=torch.rand(B).tolist())
        model.forward_and_sample(batch, list(range(B)), k, spec)
        gr = model.decode_graph(B, k)
        x = gr.x

        def advance():
            x.ids[:B].copy_(gr.samp.tok[:B])
            x.positions[:B].add_(1)
            x.slot_mapping[:B].add_(1)
        for _ in range(args.warmup):
            advance()
            gr.graph.replay()
        torch.cuda.synchronize()
        comm.barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        evs[0].record()
        for i in range(args.steps):
            advance()
            gr.graph.replay()
            evs[i + 1].record()
        torch.cuda.synchronize()
        ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
        total = evs[0].elapsed_time(evs[args.steps])
        if args.tp > 1:
            import torch.distributed as dist
            t = torch.tensor([total], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total = float(t)
        row = {"metric": "batched_decode_tok_s", "batch": B, "value": round(B * args.steps / (total / 1e3), 1),
               "unit": "tok/s", "n_gpus": args.tp, "context": args.ctx, "steps": args.steps,
               "sampling": "temperature 0.6, top-k 50" if args.sample else "greedy", "itl": stats(ms),
               "launches_per_step": gr.launches, "peer_status": model.peer_status()}
        rows.append(row)
        if comm.rank == 0:
            print(json.dumps(row), flush=True)
    if comm.rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    if args.tp > 1:
        import torch.distributed as dist
        dist.barrier()
        model.release_graphs()
        torch.cuda.synchronize()
        if model.peer is not None:
            model.peer.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
