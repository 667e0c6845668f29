"""Runs INSIDE the reference's own package tree (PYTHONPATH = baseline/_ref, nothing of tileinfer_b200 on
the path): builds the reference's LLM on a checkpoint directory and times decode the way the reference's
own harness does (tests/bench_multi_gpu.py:57-115): a max_tokens=1 call and a full call, CUDA events,
decode = full - prefill.  Prints one JSON line on rank 0."""
import argparse
import json
import os
import sys
import time


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--model-name", default="qwen3.6-27b")
    args = ap.parse_args()
    import torch
    from engine.llm import LLM
    from engine.sampling_params import SamplingParams
    rank = int(os.environ.get("RANK", "0"))
    t0 = time.time()
    llm = LLM(args.ckpt, tp_size=args.gpus, max_model_len=2048, max_num_seqs=4, enable_prefix_caching=False)
    load_s = time.time() - t0
    g = torch.Generator().manual_seed(1234)
    vocab = llm.config.hf_config.vocab_size

    def prompt():
        ids = torch.randint(0, vocab - 1, (args.prompt_len,), generator=g).tolist()
        return " ".join(f"t{i}" for i in ids)

    def timed(max_tokens):
        p = prompt()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b), len(out[0]["token_ids"])

    timed(args.warmup + 1)
    timed(1)
    pre_ms, _ = timed(1)
    full_ms, n = timed(args.steps + 1)
    dec_ms = full_ms - pre_ms
    t = torch.tensor([dec_ms, pre_ms], device="cuda")
    if args.gpus > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dec_ms, pre_ms = (float(v) for v in t.tolist())
    if rank == 0:
        K = n - 1
        print("REF_RESULT " + json.dumps({
            "metric": "decode_tok_s", "value": round(K / (dec_ms / 1e3), 2), "unit": "tok/s", "n_gpus": args.gpus,
            "steps": K, "warmup": args.warmup, "ms_per_step": round(dec_ms / K, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": round(K / (dec_ms / 1e3) / 36.6, 3), "dtype": "bf16 activations, int8 weights",
            "data": "synthetic: uniform-random prompt tokens, random-init N(0,0.02) weights",
            "config": {"model": args.model_name, "global_batch": 1, "seq_len": args.prompt_len,
                       "parallelism": f"tp{args.gpus}", "cuda_graph": True},
            "e2e": {"value": round(K / (dec_ms / 1e3), 2), "unit": "tok/s"}, "prefill_ms": round(pre_ms, 2),
            "load_s": round(load_s, 1), "impl": "reference"}), flush=True)


if __name__ == "__main__":
    main()
