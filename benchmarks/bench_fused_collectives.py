"""Row-parallel product + all-reduce + residual: the fused peer-memory kernel against the NCCL baseline.

One rank per GPU (torchrun).  For the row-parallel shapes of the 27B layer (o_proj / out_proj K = 6144 / tp,
down K = 17408 / tp, N = 5120) and M decode rows:

  fused     ONE launch: W8A16 GEMV whose epilogue sends the partial sums as tagged packets into every rank's
            buffer over NVLink, collects them at the product boundary, sums in rank order and adds the residual
  baseline  the reference's structure (engine/parallel.py:98-125 around kernels/splitk_gemv.py): GEMV -> NCCL
            all_reduce -> residual add, three launches, eager

Both are timed with CUDA events over `--iters` iterations after warm-up, weights rotated over copies larger
than L2, max over ranks.  The fused kernel is also timed inside a CUDA graph (how the decode step runs it).
Roofline per row: max(weight bytes / measured HBM bandwidth, bytes that must cross NVLink / 770 GB/s).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_fused_collectives.py
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from tileinfer_b200.ops import functional as F  # noqa: E402
from tileinfer_b200.parallel.comm import init_distributed  # noqa: E402
from tileinfer_b200.parallel.symm_mem import PeerComm  # noqa: E402

HBM_GBS, NVLINK_GBS = 6536.0, 770.0
BF16 = torch.bfloat16


def timed(fn, iters, warm=5):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(warm + i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--rows", default="1,8")
    args = ap.parse_args()
    comm = init_distributed(int(os.environ.get("WORLD_SIZE", "1")), timeout_s=120)
    tp, rank = comm.world_size, comm.rank
    N = 5120
    peer = PeerComm(comm, N, m_cap=64)
    ws = F.GemvWorkspace()
    results = []
    for name, Kfull in (("o_proj", 6144), ("down", 17408)):
        K = Kfull // tp // 64 * 64
        ncopy = max(2, int(300e6 // (N * K)) + 1)
        Ws = [F.LinearW(torch.randn(N, K, device="cuda") * 0.05, True) for _ in range(ncopy)]
        for M in [int(m) for m in args.rows.split(",")]:
            x = torch.randn(M, K, device="cuda").to(BF16)
            resid = torch.randn(M, N, device="cuda").to(BF16)
            out_f = torch.zeros(M, N, dtype=BF16, device="cuda")
            part = torch.zeros(M, N, dtype=BF16, device="cuda")
            out_b = torch.zeros(M, N, dtype=BF16, device="cuda")
            # consecutive collectives alternate between the two packet slots (order 0 / 1), as inside a decode step
            fused_p = [[F.make_gemv_params(W, x, out_f, M, epi=F.EPI_ROWPAR, resid=resid, ws=ws, comm=peer, order=o)
                        for o in (0, 1)] for W in Ws]
            base_p = [F.make_gemv_params(W, x, part, M, epi=F.EPI_STORE, ws=ws) for W in Ws]

            def fused(i):
                peer.ctrl[0:1].add_(1)                      # the step counter the tags are derived from
                F.gemv_launch(fused_p[i % ncopy][i & 1], F.W_INT8)

            def baseline(i):
                F.gemv_launch(base_p[i % ncopy], F.W_INT8)
                dist.all_reduce(part)
                torch.add(resid, part, out=out_b)

            us_base = timed(baseline, args.iters)
            us_fused = timed(fused, args.iters)
            # the fused launch inside a CUDA graph: 2 * ncopy launches per replay
            g = torch.cuda.CUDAGraph()
            n_in_graph = 2 * ncopy
            with torch.cuda.graph(g):
                for i in range(n_in_graph):
                    fused(i)
            us_graph = timed(lambda i: g.replay(), max(10, args.iters // n_in_graph), warm=2) / n_in_graph
            ok = bool(peer.status() == 0)
            # correctness of one fused call against the baseline result
            peer.ctrl[0:1].add_(1)
            F.gemv_launch(fused_p[0][0], F.W_INT8)
            F.gemv_launch(base_p[0], F.W_INT8)
            dist.all_reduce(part)
            torch.add(resid, part, out=out_b)
            torch.cuda.synchronize()
            err = float((out_f.float() - out_b.float()).abs().max())
            wbytes = N * K
            link_bytes = (tp - 1) * M * N * 8                # 8-byte packets to every peer
            floor_us = max(wbytes / (HBM_GBS * 1e3), link_bytes / (NVLINK_GBS * 1e3))
            results.append({"op": name, "tp": tp, "M": M, "K_per_rank": K, "fused_us": round(us_fused, 2),
                            "fused_graph_us": round(us_graph, 2), "nccl_baseline_us": round(us_base, 2),
                            "speedup_eager": round(us_base / us_fused, 2), "floor_us": round(floor_us, 2),
                            "fraction_of_roofline_graph": round(floor_us / us_graph, 3), "max_abs_diff": round(err, 4),
                            "peer_status_ok": ok})
            if rank == 0:
                print(json.dumps(results[-1]), flush=True)
    dist.barrier()
    peer.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
