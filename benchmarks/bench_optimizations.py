"""What each optimisation buys, measured through the public API (the counterpart of the reference's
tests/bench_optimizations.py:43-211: prefill throughput, decode throughput with and without CUDA graphs, the fused
lm_head + arg-max against lm_head + selection, memory in use).

Every variant runs in its own process (several switches are read once when the kernel library loads), builds an `LLM`,
times a prefill-dominated request (`max_tokens=1`) and a decode-dominated one, and prints one JSON line; the parent
prints them with the ratio to the default configuration.

    python benchmarks/bench_optimizations.py [--model preset:qwen3.6-27b] [--prompt-len 512] [--max-tokens 128]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_optimizations.py --tp 2
    python benchmarks/bench_optimizations.py --model preset:tiny-hybrid --device cpu --quick       # plumbing check without a GPU
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

# name -> (extra engine kwargs, extra environment)
VARIANTS = {
    "default": ({}, {}),
    "eager (no CUDA graphs)": ({"enforce_eager": True}, {}),
    "lm_head + selection instead of the arg-max epilogue": ({}, {"TI_FUSED_ARGMAX": "0"}),
    "no programmatic dependent launch": ({}, {"TI_PDL": "0"}),
    "one GEMV launch per product (no chain)": ({}, {"TI_GEMV_CHAIN": "0"}),
    "direct-load decode attention": ({}, {"TI_ATTN_PIPE": "0"}),
    "multi-step scheduling x4": ({"num_scheduler_steps": 4}, {}),
    "NCCL collectives instead of the fused ones (tp > 1)": ({"fused_collectives": False}, {}),
}


def sync():
    import torch
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def run_variant(args):
    import torch
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    kwargs, _ = VARIANTS[args.variant]
    if args.tp == 1:
        kwargs = {k: v for k, v in kwargs.items() if k != "fused_collectives"}
    llm = LLM(args.model, tp_size=args.tp, device=args.device, max_model_len=args.prompt_len + args.max_tokens + 64,
              max_num_seqs=4, **kwargs)
    g = torch.Generator().manual_seed(0)
    vocab = llm.model_runner.model_config.vocab_size if hasattr(llm.model_runner, "model_config") else 1000
    prompt = torch.randint(0, min(vocab, 1000) - 1, (args.prompt_len,), generator=g).tolist()
    one = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    many = SamplingParams(temperature=0.0, max_tokens=args.max_tokens, ignore_eos=True)
    # distinct first tokens keep the prefix cache from turning the repeats into cache hits
    def timed(sp, salt):
        p = [salt % 900 + 1] + prompt[1:]
        sync()
        t0 = time.perf_counter()
        out = llm.generate_token_ids([p], sp)
        sync()
        return time.perf_counter() - t0, out
    for w in range(args.warmup):
        timed(one, 100 + w)
    t_pre = min(timed(one, 200 + i)[0] for i in range(args.runs))
    timed(many, 300)
    t_dec = min(timed(many, 400 + i)[0] for i in range(args.runs))
    decode_s = max(t_dec - t_pre, 1e-9)
    res = {"variant": args.variant, "tp": args.tp, "prefill_tok_s": round(args.prompt_len / t_pre, 1),
           "decode_tok_s": round((args.max_tokens - 1) / decode_s, 2), "prefill_s": round(t_pre, 4),
           "request_s": round(t_dec, 4)}
    if torch.cuda.is_available() and args.device != "cpu":
        res["gpu_mem_gb"] = round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)
    if llm.comm.rank == 0:
        print("VARIANT_RESULT " + json.dumps(res), flush=True)
    llm.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="preset:qwen3.6-27b")
    ap.add_argument("--tp", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--device", default="auto")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--quick", action="store_true", help="short prompt, few tokens, two variants")
    ap.add_argument("--variant", default=None, help="(internal) run this one variant in this process")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    if args.quick:
        args.prompt_len, args.max_tokens, args.runs = 48, 8, 1
    if args.variant is not None:
        return run_variant(args)
    if args.tp > 1 and "RANK" in os.environ:
        raise SystemExit("run the parent without torchrun: it starts one torchrun per variant itself (--tp N)")
    names = list(VARIANTS)
    if args.quick:
        names = names[:2]
    if args.tp == 1:
        names = [n for n in names if "tp > 1" not in n]
    rows = []
    for i, name in enumerate(names):
        env = dict(os.environ, **VARIANTS[name][1])
        child = [os.path.abspath(__file__), "--variant", name, "--model", args.model, "--tp", str(args.tp), "--device", args.device,
                 "--prompt-len", str(args.prompt_len), "--max-tokens", str(args.max_tokens), "--runs", str(args.runs),
                 "--warmup", str(args.warmup)]
        if args.tp > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.tp),
                   "--master-addr", "127.0.0.1", "--master-port", str(29800 + i)] + child
        else:
            cmd = [sys.executable] + child
        r = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=3600)
        line = [l for l in r.stdout.splitlines() if l.startswith("VARIANT_RESULT ")]
        if r.returncode != 0 or not line:
            rows.append({"variant": name, "error": (r.stderr or r.stdout)[-300:]})
            continue
        rows.append(json.loads(line[0][len("VARIANT_RESULT "):]))
    base = next((r for r in rows if r.get("variant") == "default" and "error" not in r), None)
    for r in rows:
        if base is not None and "error" not in r:
            r["decode_vs_default"] = round(r["decode_tok_s"] / base["decode_tok_s"], 3)
            r["prefill_vs_default"] = round(r["prefill_tok_s"] / base["prefill_tok_s"], 3)
        print(json.dumps(r), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
