"""GEMV micro-benchmark: achieved weight-streaming bandwidth per shape, with an optional per-CTA
timeline (globaltimer stamps written by the kernel).  Weights are rotated over several copies so
that every launch streams from HBM, not from the 126 MB L2.

    python benchmarks/bench_gemv.py [--timeline] [--chain]

--chain times the four dependent products of a decoder layer (out_proj -> gate_up+SwiGLU -> down -> next
in_proj, 27B shapes) in ONE launch, as the decode step runs them.
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


def _print_timeline(dbg, n_ops):
    t = dbg.view(148, 32).cpu().double()
    t0 = t[:, 0].min()

    def row(nm, j):
        c = (t[:, j] - t0) / 1e3
        print(f"      {nm:22s} min {c.min():7.2f}  mean {c.mean():7.2f}  max {c.max():7.2f} us")
    row("start", 0)
    row("ring primed", 1)
    for op in range(n_ops):
        for k, nm in enumerate(("marker reached", "barrier passed", "x staged", "last unit done")):
            row(f"op{op} {nm}", 8 + 4 * op + k)
    for op in range(1, min(n_ops, 4)):
        row(f"all warps of the CTA at barrier before op{op}", 1 + op)
    for op in range(min(n_ops, 2)):
        for k, nm in enumerate(("unit popped", "first chunk arrived", "tiles done")):
            row(f"op{op} warp0 last unit: {nm}", 24 + 4 * op + k)
    row("end", 5)


def bench_chain(args):
    """One launch = out_proj, gate_up, down, in_proj of the 27B layer; weights rotate over copies > L2."""
    tp = args.tp_shapes          # per-rank shapes of a tensor-parallel group of this size, without the collectives
    M, H, I, KO, NI = args.M, 5120, 17408 // tp, 6144 // tp, 16480 // tp // 8 * 8
    ws = F.GemvWorkspace()
    ncopy = 3
    mk = lambda n, k: F.LinearW(torch.randn(n, k, device="cuda") * 0.05, True)
    sets = [(mk(H, KO), mk(2 * I, H), mk(H, I), mk(NI, H)) for _ in range(ncopy)]
    x = torch.randn(M, KO, device="cuda").to(torch.bfloat16)
    h0 = torch.randn(M, H, device="cuda").to(torch.bfloat16)
    h1, h2 = torch.zeros_like(h0), torch.zeros_like(h0)
    act = torch.zeros(M, I, dtype=torch.bfloat16, device="cuda")
    proj = torch.zeros(M, NI, dtype=torch.bfloat16, device="cuda")
    nw = torch.zeros(H, dtype=torch.bfloat16, device="cuda")
    dbg = torch.zeros(148 * 32, dtype=torch.int64, device="cuda")
    chains = []
    tm = [int(t) for t in args.teams.split(",")] if args.teams else [None] * 4
    for Wo, Wgu, Wd, Wi in sets:
        ps = [F.make_gemv_params(Wo, x, h1, M, xmode=F.XGLOBAL, epi=F.EPI_ROWPAR, resid=h0, ws=ws, team=tm[0]),
              F.make_gemv_params(Wgu, h1, act, M, xmode=F.XNORM, epi=F.EPI_SWIGLU, norm_w=nw, ws=ws, team=tm[1]),
              F.make_gemv_params(Wd, act, h2, M, xmode=F.XGLOBAL, epi=F.EPI_ROWPAR, resid=h1, ws=ws, team=tm[2]),
              F.make_gemv_params(Wi, h2, proj, M, xmode=F.XNORM, epi=F.EPI_STORE, norm_w=nw, ws=ws, team=tm[3])]
        if args.timeline:
            ps[0].dbg = dbg.data_ptr()
        chains.append(ps)
    for i in range(4):
        F.gemv_chain_launch(chains[i % ncopy], F.W_INT8)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(args.iters):
            F.gemv_chain_launch(chains[i % ncopy], F.W_INT8)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.iters
    nbytes = sum(W.nbytes() for W in sets[0])
    print(f"chain of 4 (27B layer, 1/{tp} shard) M={M} stages={chains[0][0].stages} T={[p.T for p in chains[0]]}: {us:7.2f} us  {nbytes / us / 1e3:7.1f} GB/s "
          f"({nbytes / 1e6:.0f} MB)")
    if args.timeline:
        _print_timeline(dbg, 4)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--timeline", action="store_true")
    ap.add_argument("--chain", action="store_true")
    ap.add_argument("--tp-shapes", type=int, default=1)
    ap.add_argument("--teams", default=None, help="team sizes of the four chained products, e.g. 2,2,16,1 (default: planner)")
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--iters", type=int, default=40)
    args = ap.parse_args()
    M = args.M
    if args.chain:
        return bench_chain(args)
    ws = F.GemvWorkspace()
    for name, (N, K, xmode, epi) in SHAPES.items():
        ncopy = max(2, int(400e6 // (N * K)) + 1)
        Ws = [F.LinearW(torch.randn(N, K, device="cuda") * 0.05, True) for _ in range(ncopy)]
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        nw = torch.zeros(K, dtype=torch.bfloat16, device="cuda")
        resid = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        dbg = torch.zeros(148 * 32, dtype=torch.int64, device="cuda")
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
            _print_timeline(dbg, 1)


if __name__ == "__main__":
    main()
