"""GEMV micro-benchmark: achieved weight-streaming bandwidth per shape, with an optional per-CTA
timeline (globaltimer stamps written by the kernel).  Weights are rotated over several copies so
that every launch streams from HBM, not from the 126 MB L2.

    python benchmarks/bench_gemv.py [--timeline]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from tileinfer_b200.ops import functional as F  # noqa: E402

SHAPES = {   # name: (N, K, xmode, epi)
    "in_proj": (16480, 5120, F.XNORM, F.EPI_STORE),
    "gate_up": (34816, 5120, F.XNORM, F.EPI_SWIGLU),
    "down": (5120, 17408, F.XGLOBAL, F.EPI_ROWPAR),
    "out_proj": (5120, 6144, F.XGLOBAL, F.EPI_ROWPAR),
    "down_tp8": (5120, 2176, F.XGLOBAL, F.EPI_ROWPAR),
    "tiny_norm": (64, 5120, F.XNORM, F.EPI_STORE),
    "tiny_glob": (64, 6144, F.XGLOBAL, F.EPI_ROWPAR),
    "big_norm": (4 * 34816, 5120, F.XNORM, F.EPI_SWIGLU),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--timeline", action="store_true")
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--iters", type=int, default=40)
    args = ap.parse_args()
    M = args.M
    ws = F.GemvWorkspace()
    for name, (N, K, xmode, epi) in SHAPES.items():
        ncopy = max(2, int(400e6 // (N * K)) + 1)
        Ws = [F.LinearW(torch.randn(N, K, device="cuda") * 0.05, True) for _ in range(ncopy)]
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        nw = torch.zeros(K, dtype=torch.bfloat16, device="cuda")
        resid = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        dbg = torch.zeros(148 * 8, dtype=torch.int64, device="cuda")
        ps = []
        for W in Ws:
            p = F.make_gemv_params(W, x, out, M, xmode=xmode, epi=epi, norm_w=nw, resid=resid, ws=ws)
            if args.timeline:
                p.dbg = dbg.data_ptr()
            ps.append(p)
        for i in range(5):
            F.gemv_launch(ps[i % ncopy], F.W_INT8, xmode, epi)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(args.iters):
                F.gemv_launch(ps[i % ncopy], F.W_INT8, xmode, epi)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.iters
        p0 = ps[0]
        print(f"{name:10s} N={N:6d} K={K:6d} M={M} R={p0.R} tps={p0.tps} stages={p0.stages} "
              f"{us:7.2f} us  {N * K / us / 1e3:7.1f} GB/s")
        if args.timeline:
            t = dbg.view(148, 8).cpu().double()
            t0 = t[:, 0].min()
            names = ["start", "ring primed", "x staged", "first chunk", "last unit", "end"]
            for j, nm in enumerate(names):
                c = (t[:, j] - t0) / 1e3
                print(f"      {nm:12s} min {c.min():7.2f}  mean {c.mean():7.2f}  max {c.max():7.2f} us")


if __name__ == "__main__":
    main()
