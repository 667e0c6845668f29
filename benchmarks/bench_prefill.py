"""Long-prompt prefill benchmark through the public API: `--prompts` prompts of `--prompt-len` random tokens,
chunked prefill (`--chunk`), optionally `--decoders` short requests decoding alongside (mixed batches).

Prints one JSON line on rank 0: prompt tokens/s (wall clock between device synchronisations, max over ranks)
and the engine's step statistics.  `--quantization bf16` runs the unquantised weights (tcgen05 kind::f16 GEMM).

    python benchmarks/bench_prefill.py --model preset:qwen3.6-27b --prompts 2 --prompt-len 32768 --chunk 8192
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_prefill.py \
        --quantization bf16 --prompts 8 --prompt-len 32768 --chunk 8192 --decoders 32
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
    ap.add_argument("--prompts", type=int, default=2)
    ap.add_argument("--prompt-len", type=int, default=32768)
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--decoders", type=int, default=0)
    ap.add_argument("--decode-tokens", type=int, default=64)
    ap.add_argument("--quantization", default="w8a16")
    args = ap.parse_args()

    llm = LLM(args.model, tp_size=args.tp, quantization=args.quantization, max_num_seqs=max(8, args.decoders + args.prompts),
              max_model_len=args.prompt_len + 256, max_prefill_chunk_tokens=args.chunk,
              max_num_batched_tokens=args.chunk + 256, enable_prefix_caching=False, gpu_memory_utilization=0.85)
    vocab = llm.config.model_config.vocab_size
    cuda = torch.cuda.is_available() and llm.config.device != "cpu"
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    g = torch.Generator().manual_seed(11)
    longs = [torch.randint(0, vocab - 1, (args.prompt_len,), generator=g).tolist() for _ in range(args.prompts)]
    shorts = [torch.randint(0, vocab - 1, (32,), generator=g).tolist() for _ in range(args.decoders)]
    llm.generate_token_ids([longs[0][:256]], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))   # warm-up
    sync()
    llm.comm.barrier()
    t0 = time.perf_counter()
    # the decoders go first so that they are decoding while the long prompts are being prefilled
    sp_short = SamplingParams(temperature=0.0, max_tokens=args.decode_tokens, ignore_eos=True)
    sp_long = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    for p in shorts:
        llm.add_request(p, sp_short)
    for p in longs:
        llm.add_request(p, sp_long)
    while not llm.scheduler.is_finished():
        llm.step()
    sync()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], device="cuda" if cuda else "cpu")
    if args.tp > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t)
    st = llm.stats()
    if llm.comm.rank == 0:
        ptoks = args.prompts * args.prompt_len
        print(json.dumps({"metric": "prefill_tok_s", "value": round(ptoks / dt, 1), "unit": "tok/s", "n_gpus": args.tp,
                          "wall_s": round(dt, 3), "prompt_tokens": ptoks,
                          "config": {"model": args.model, "quantization": args.quantization, "prompts": args.prompts,
                                     "prompt_len": args.prompt_len, "chunk": args.chunk, "decoders": args.decoders,
                                     "decode_tokens": args.decode_tokens, "parallelism": f"tp{args.tp}"},
                          "stats": {k: st.get(k) for k in ("steps", "prefill_tokens", "decode_tokens", "mean_batch_tokens",
                                                           "step_ms_p50", "itl_ms_p50", "itl_ms_p99")}}), flush=True)
    if args.tp > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
