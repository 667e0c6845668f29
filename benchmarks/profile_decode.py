"""Decode-step driver for profilers: builds the model, captures the CUDA-graph decode step for one
batch size and replays it.  Meant to be run as is (prints ms/step), under
`ncu --metrics gpu__time_duration.sum --clock-control none` for a per-kernel launch list, or with
`--torch-profiler`, which runs eager decode steps under torch.profiler, prints the kernel time per category
(GEMV / GEMM / attention / DeltaNet / sampling / communication / ...) and the top kernels, and with `--trace FILE`
writes a Chrome trace.  That mode is the counterpart of the reference's tests/profile_decode.py:71-114,188-191.
`TI_NVTX=1` adds an NVTX range per layer and block for external timeline tools.

    python benchmarks/profile_decode.py --model preset:qwen3.6-27b-8l --batch 1 --ctx 256 --steps 3
    python benchmarks/profile_decode.py --model preset:qwen3.6-27b-8l --torch-profiler --trace decode_trace.json
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from tileinfer_b200.models.config import get_preset  # noqa: E402
from tileinfer_b200.models.hybrid_b200 import B200HybridModel  # noqa: E402
from tileinfer_b200.models.reference_cpu import Batch  # noqa: E402
from tileinfer_b200.models.weights import RandomWeights  # noqa: E402


def prefill(m, cfg, args):
    """One sequence, one chunk of --prefill tokens, eager (the path a prefill step takes)."""
    T = args.prefill
    nblk = T // 16 + 2
    m.alloc_cache(nblk + 1, 16, 2)
    batch = Batch(torch.randint(0, cfg.vocab_size - 1, (T,)), torch.arange(T), [0, T], [T], [list(range(nblk))],
                  torch.arange(T), [0])
    m.forward(batch)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        m.forward(batch)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(f"model={cfg.name} prefill tokens={T} ms/forward={ms:.3f} tok/s={T / ms * 1e3:.0f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="preset:qwen3.6-27b-8l")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=256)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--quant", default="w8a16")
    ap.add_argument("--prefill", type=int, default=0, help="run eager prefill forwards of this many tokens instead")
    ap.add_argument("--torch-profiler", action="store_true", help="category buckets + top kernels through torch.profiler")
    ap.add_argument("--trace", default=None, help="with --torch-profiler: write a Chrome trace here")
    args = ap.parse_args()
    cfg = get_preset(args.model)
    torch.cuda.set_device(0)
    m = B200HybridModel(cfg, RandomWeights(cfg, 0, device="cuda"), quant=args.quant)
    if args.prefill:
        return prefill(m, cfg, args)
    B = args.batch
    nblk_seq = args.ctx // 16 + 2
    m.alloc_cache(B * nblk_seq + 1, 16, B + 1)
    m.capture_decode_graphs(B, B, args.ctx + 16, B)
    tables = [list(range(s * nblk_seq, (s + 1) * nblk_seq)) for s in range(B)]
    pos = args.ctx - 1
    batch = Batch(torch.randint(0, cfg.vocab_size - 1, (B,)), torch.full((B,), pos), list(range(B + 1)), [pos + 1] * B,
                  tables, torch.tensor([t[pos // 16] * 16 + pos % 16 for t in tables]), list(range(B)))
    m._decode_graph_step(batch, 1)
    torch.cuda.synchronize()
    if args.torch_profiler:
        from tileinfer_b200.utils.trace import format_profile, profile_call

        def steps():
            for _ in range(args.steps):
                h = m.forward(batch)                # eager: every kernel shows up by name (a graph replay is one node)
                m.logits(h)
        steps()
        res = profile_call(steps, trace_path=args.trace)
        print(f"model={cfg.name} batch={B} ctx={args.ctx}: {args.steps} eager decode steps")
        print(format_profile(res))
        return
    g = m.decode_graph(m.buckets[-1], 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        g.graph.replay()
    e1.record()
    torch.cuda.synchronize()
    print(f"model={cfg.name} batch={B} ctx={args.ctx} launches/step={g.launches} ms/step={e0.elapsed_time(e1) / args.steps:.4f}")


if __name__ == "__main__":
    main()
