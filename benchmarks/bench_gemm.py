"""Prefill GEMM micro-benchmark (tcgen05 kind::i8 W8A16): time, int8 tensor throughput of the two limb
products and weight-streaming bandwidth per shape.  Weight copies are rotated so each launch streams from HBM.

    python benchmarks/bench_gemm.py [--M 32 64 128 512 2048]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from tileinfer_b200.ops import functional as F  # noqa: E402

SHAPES = {"in_proj": (16480, 5120, F.GEPI_STORE), "gate_up": (34816, 5120, F.GEPI_SWIGLU),
          "down": (5120, 17408, F.GEPI_ROWPAR), "out_proj": (5120, 6144, F.GEPI_ROWPAR)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, nargs="*", default=[32, 64, 128, 512, 2048])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    for name, (N, K, epi) in SHAPES.items():
        if args.only and name != args.only:
            continue
        ncopy = max(2, int(300e6 // (N * K)) + 1)
        Ws = [F.LinearW(torch.randn(N, K, device="cuda") * 0.05, True) for _ in range(ncopy)]
        for M in args.M:
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            limbs = F.quant_rows(x)
            resid = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
            out = torch.zeros(M, N // 2 if epi == F.GEPI_SWIGLU else N, dtype=torch.bfloat16, device="cuda")
            for i in range(3):
                F.gemm_w8a16(Ws[i % ncopy], limbs, out=out, epi=epi, resid=resid)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.iters):
                F.gemm_w8a16(Ws[i % ncopy], limbs, out=out, epi=epi, resid=resid)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / args.iters
            tops = 2 * 2.0 * M * N * K / us / 1e6          # two int8 limb products
            print(f"{name:9s} M={M:5d} N={N:6d} K={K:6d}  {us:9.1f} us  {tops:8.1f} int8 TOP/s  "
                  f"{2.0 * M * N * K / us / 1e6:8.1f} TFLOP/s bf16-equivalent  weights {N * K / us / 1e3:7.1f} GB/s")


if __name__ == "__main__":
    main()
