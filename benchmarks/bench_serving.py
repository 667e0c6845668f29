"""Continuous-batching benchmark: many concurrent requests through the public API (`LLM.generate_token_ids`).

Workload of the serving configuration: `--requests` prompts of 512..2048 random tokens that share a
`--prefix`-token prefix, `--max-tokens` sampled tokens each (temperature 0.6, top-k 50), swap space on,
multi-step scheduling.  Prints one JSON line on rank 0: aggregate generated tokens/s (wall clock bracketed by
device synchronisation, max over ranks), TTFT / ITL percentiles and scheduler counters from `LLM.stats()`.

    python benchmarks/bench_serving.py --model preset:qwen3.6-27b-8l --requests 16
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_serving.py --tp 2
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from tileinfer_b200.engine.llm import LLM  # noqa: E402
from tileinfer_b200.engine.sampling_params import SamplingParams  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="preset:qwen3.6-27b")
    ap.add_argument("--tp", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--min-prompt", type=int, default=512)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--prefix", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--scheduler-steps", type=int, default=4)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--swap-gb", type=float, default=8.0)
    ap.add_argument("--quantization", default="w8a16")
    ap.add_argument("--prefix-share", type=float, default=0.5, help="fraction of the requests that start with the shared prefix")
    ap.add_argument("--kv-blocks", type=int, default=-1, help="size of the KV pool in 16-token pages (default: from free memory); "
                                                               "a small pool forces preemption by swapping")
    args = ap.parse_args()

    llm = LLM(args.model, tp_size=args.tp, quantization=args.quantization, max_num_seqs=min(64, args.requests),
              max_model_len=args.max_prompt + args.max_tokens + 16, max_prefill_chunk_tokens=args.chunk,
              max_num_batched_tokens=args.chunk + 64, num_scheduler_steps=args.scheduler_steps,
              swap_space_bytes=int(args.swap_gb * (1 << 30)), gpu_memory_utilization=0.85,
              num_kvcache_blocks=args.kv_blocks)
    vocab = llm.config.model_config.vocab_size
    cuda = torch.cuda.is_available() and llm.config.device != "cpu"
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    g = torch.Generator().manual_seed(7)
    prefix = torch.randint(0, vocab - 1, (args.prefix,), generator=g).tolist()
    prompts = []
    for i in range(args.requests):
        n = int(torch.randint(args.min_prompt, args.max_prompt + 1, (1,), generator=g))
        shared = (i % 100) < int(100 * args.prefix_share)       # e.g. every other request for 0.5
        if args.prefix_share == 0.5:
            shared = i % 2 == 0
        head = prefix if shared else torch.randint(0, vocab - 1, (args.prefix,), generator=g).tolist()
        prompts.append(head + torch.randint(0, vocab - 1, (max(1, n - args.prefix),), generator=g).tolist())
    sp = SamplingParams(temperature=0.6, top_k=50, max_tokens=args.max_tokens, ignore_eos=True)
    # warm-up: compiles nothing, but touches every graph bucket's first replay and the allocator
    llm.generate_token_ids([prompts[0][:64]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    sync()
    llm.comm.barrier()
    t0 = time.perf_counter()
    outs = llm.generate_token_ids(prompts, sp)
    sync()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], device="cuda" if cuda else "cpu")
    if args.tp > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t)
    st = llm.stats()
    if llm.comm.rank == 0:
        gen = sum(len(o) for o in outs)
        keys = ("steps", "prefill_tokens", "mean_batch_tokens", "ttft_ms_p50", "ttft_ms_p99", "itl_ms_p50", "itl_ms_p99",
                "step_ms_p50", "preemptions", "swaps_out", "swaps_in", "recomputes", "prefix_hits", "prefix_hit_tokens")
        print(json.dumps({"metric": "serving_generated_tok_s", "value": round(gen / dt, 1), "unit": "tok/s",
                          "n_gpus": args.tp, "wall_s": round(dt, 3), "generated_tokens": gen,
                          "prompt_tokens": sum(len(p) for p in prompts),
                          "total_tok_s": round((gen + sum(len(p) for p in prompts)) / dt, 1),
                          "config": {"model": args.model, "requests": args.requests, "prompt": [args.min_prompt, args.max_prompt],
                                     "shared_prefix": args.prefix, "prefix_share": args.prefix_share, "kv_blocks": llm.config.num_kvcache_blocks, "max_tokens": args.max_tokens, "temperature": 0.6, "top_k": 50,
                                     "scheduler_steps": args.scheduler_steps, "chunk": args.chunk, "parallelism": f"tp{args.tp}"},
                          "stats": {k: st.get(k) for k in keys}}), flush=True)
    if args.tp > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
