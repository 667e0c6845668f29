"""Fused compute + collective kernels against the NCCL structure they replace, at the 27B shapes.

One rank per GPU (torchrun), M = 1, 8, 64, 256 rows.

Op 1  row-parallel W8A16 product (N = 5120, K = 17408 / tp: the MLP down projection; int8 weights uniform in
      [-127, 127], bf16 scales, activations N(0, 1)) + all-reduce + residual add + RMSNorm.
        fused, M <= 16   ONE GEMV launch whose epilogue sends the partial sums as tagged packets into every rank's
                         buffer over NVLink and collects them at the product boundary (+ residual); the RMSNorm is a
                         separate launch HERE (in the model it is the prologue of the consuming GEMV and costs none)
        fused, M > 16    activation limbs -> tcgen05 GEMM storing bf16 partials into the symmetric buffer -> ONE kernel:
                         sum over ranks (multimem.ld_reduce through NVSwitch, or peer loads) + residual + RMSNorm
        baseline         the reference's structure (engine/parallel.py:98-125, kernels/residual_rmsnorm.py): the same
                         product -> NCCL all_reduce -> residual+RMSNorm kernel
Op 2  lm_head product over the vocabulary shard (248320 / tp rows, bf16) + per-rank top-k (64 kept, 50 asked) + exchange
      of the candidates through peer memory, against gathering the full-vocabulary logits with NCCL and torch.topk.

Timed with CUDA events over `--iters` iterations after warm-up, weights rotated over copies larger than L2, max over
ranks.  Roofline = the slowest of weight bytes / measured copy bandwidth, FLOPs / measured bf16 throughput and the
bytes that must cross NVLink / 770 GB/s (measured peer copy, per direction); peaks from MEASURED_PEAKS.json.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_fused_collectives.py
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from tileinfer_b200.ops import functional as F  # noqa: E402
from tileinfer_b200.parallel.comm import init_distributed  # noqa: E402
from tileinfer_b200.parallel.symm_mem import PeerComm  # noqa: E402

NVLINK_GBS = 770.0
BF16 = torch.bfloat16


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


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


def graph_timed(fn, n_in_graph, iters):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_in_graph):
            fn(i)
    return timed(lambda i: g.replay(), max(5, iters // n_in_graph), warm=2) / n_in_graph


def op1(peer, comm, args, out):
    tp, rank = comm.world_size, comm.rank
    hbm, tflops, how = peaks()
    N, K = 5120, 17408 // tp // 64 * 64
    ncopy = max(2, int(300e6 // (N * K)) + 1)
    ws = F.GemvWorkspace()
    mk = lambda: torch.randint(-127, 128, (N, K), device="cuda").float() * 0.01
    Ws = [F.LinearW(mk(), True) for _ in range(ncopy)]
    nw = torch.zeros(N, dtype=BF16, device="cuda")
    for M in args.rows:
        x = torch.randn(M, K, device="cuda").to(BF16)
        resid = torch.randn(M, N, device="cuda").to(BF16)
        h_f = torch.zeros(M, N, dtype=BF16, device="cuda")
        n_f = torch.zeros(M, N, dtype=BF16, device="cuda")
        part = torch.zeros(M, N, dtype=BF16, device="cuda")
        h_b = torch.zeros(M, N, dtype=BF16, device="cuda")
        n_b = torch.zeros(M, N, dtype=BF16, device="cuda")
        order = [0]
        if M <= 16:
            fused_p = [[F.make_gemv_params(W, x, h_f, M, epi=F.EPI_ROWPAR, resid=resid, ws=ws, comm=peer, order=o)
                        for o in (0, 1)] for W in Ws]
            base_p = [F.make_gemv_params(W, x, part, M, epi=F.EPI_STORE, ws=ws) for W in Ws]

            def fused(i):
                peer.ctrl[0:1].add_(1)                      # the step counter the tags are derived from
                F.gemv_launch(fused_p[i % ncopy][i & 1], F.W_INT8)
                F.rmsnorm(h_f, nw, 1e-6, out=n_f)

            def baseline(i):
                F.gemv_launch(base_p[i % ncopy], F.W_INT8)
                dist.all_reduce(part)
                F.rmsnorm(part, nw, 1e-6, add=resid, out=n_b, r_out=h_b)
            link_bytes = (tp - 1) * M * N * 8                # 8-byte packets to every peer
            form = "gemv+packets"
        else:
            limbs = F.Limbs(M, K, "cuda")

            def fused(i):
                peer.ctrl[0:1].add_(1)
                F.quant_rows(x, out=limbs)
                F.gemm_w8a16(Ws[i % ncopy], limbs, out=peer.part_view(i & 1, M), epi=F.GEPI_STORE)
                F.ar_rows(peer, i & 1, M, N, resid, h_f, order=i & 1, mode=F.AR_BF16, norm_w=nw, xn=n_f)

            def baseline(i):
                F.quant_rows(x, out=limbs)
                F.gemm_w8a16(Ws[i % ncopy], limbs, out=part, epi=F.GEPI_STORE)
                dist.all_reduce(part)
                F.rmsnorm(part, nw, 1e-6, add=resid, out=n_b, r_out=h_b)
            link_bytes = (tp - 1) * M * N * 2                # every rank reads every peer's bf16 partial rows once
            form = "gemm+multimem" if peer.nvls else "gemm+peer-loads"
        us_base = timed(baseline, args.iters)
        us_fused = timed(fused, args.iters)
        us_graph = graph_timed(fused, 2 * ncopy, args.iters)
        ok = bool(peer.status() == 0)
        fused(0)
        baseline(0)
        torch.cuda.synchronize()
        err = float((n_f.float() - n_b.float()).abs().max())
        floor_us = max(N * K / (hbm * 1e3), 2.0 * M * N * K / (tflops * 1e6), link_bytes / (NVLINK_GBS * 1e3))
        out.append({"op": "down+allreduce+residual+rmsnorm", "form": form, "tp": tp, "M": M, "K_per_rank": K,
                    "fused_us": round(us_fused, 2), "fused_graph_us": round(us_graph, 2),
                    "nccl_baseline_us": round(us_base, 2), "baseline_over_fused_graph": round(us_base / us_graph, 2),
                    "floor_us": round(floor_us, 2), f"fraction_of_roofline_{how}": round(floor_us / us_graph, 3),
                    "nvlink_bytes_per_rank": link_bytes, "max_abs_diff_vs_baseline": round(err, 4), "peer_status_ok": ok})
        if rank == 0:
            print(json.dumps(out[-1]), flush=True)


def op2(peer, comm, args, out):
    tp, rank = comm.world_size, comm.rank
    hbm, tflops, how = peaks()
    V, H, k = 248320 // tp, 5120, 64
    ncopy = 2
    Ws = [F.LinearW(torch.randn(V, H, device="cuda") * 0.02, False) for _ in range(ncopy)]
    nw = torch.zeros(H, dtype=BF16, device="cuda")
    ws = F.GemvWorkspace()
    max_chunks = min(128, 8192 // k)
    cs = max(256, -(-(-(-V // max_chunks)) // 256) * 256)
    chunks = -(-V // cs)
    for M in args.rows:
        hid = torch.randn(M, H, device="cuda").to(BF16)
        logits = torch.zeros(M, V, dtype=torch.float32, device="cuda")
        mcap = peer.m_cap
        tks = []
        for m0 in range(0, M, mcap):
            m = min(mcap, M - m0)
            t = F.TopkParams()
            keep = [torch.empty(m * chunks * k, dtype=torch.float32, device="cuda"),
                    torch.empty(m * chunks * k, dtype=torch.int32, device="cuda"),
                    torch.empty(m, tp * k, dtype=torch.float32, device="cuda"),
                    torch.empty(m, tp * k, dtype=torch.int32, device="cuda")]
            t.logits, t.ws_val, t.ws_idx, t.out_val, t.out_idx = (logits[m0:m0 + m].data_ptr(), keep[0].data_ptr(),
                                                                   keep[1].data_ptr(), keep[2].data_ptr(), keep[3].data_ptr())
            t.M, t.V, t.ld, t.k, t.chunks, t.chunk_size, t.vocab_start = m, V, V, k, chunks, cs, rank * V
            t.tp, t.rank, t.order, t.m_cap = tp, rank, 65000 + m0 // mcap, mcap
            for r in range(tp):
                t.peer_buf[r] = peer.cand_ptrs[r]
            t.step_ptr, t.status, t.timeout_ns = peer.step_ptr, peer.status_ptr, peer.timeout_ns
            tks.append((t, keep))

        def head(i):
            W = Ws[i % ncopy]
            if M <= 8:
                F.gemv(W, hid, out=logits, xmode=F.XNORM, epi=F.EPI_F32, norm_w=nw, ws=ws)
            else:
                xs = F.rmsnorm(hid, nw, 1e-6)
                F.gemm_bf16(W, xs, out=logits, epi=F.GEPI_F32)

        def fused(i):
            peer.ctrl[0:1].add_(1)
            head(i)
            for t, _ in tks:
                F.topk(t)

        full = torch.empty(tp, M, V, dtype=torch.float32, device="cuda")

        def baseline(i):
            head(i)
            dist.all_gather_into_tensor(full.view(-1), logits.view(-1))
            torch.topk(full.permute(1, 0, 2).reshape(M, tp * V), 50, dim=-1)

        us_base = timed(baseline, max(10, args.iters // 4))
        us_fused = timed(fused, max(10, args.iters // 4))
        ok = bool(peer.status() == 0)
        floor_us = max(V * H * 2 / (hbm * 1e3), 2.0 * M * V * H / (tflops * 1e6))
        out.append({"op": "lm_head+top-k+candidate exchange", "tp": tp, "M": M, "vocab_per_rank": V,
                    "fused_us": round(us_fused, 2), "full_vocab_gather_baseline_us": round(us_base, 2),
                    "baseline_over_fused": round(us_base / us_fused, 2), "floor_us": round(floor_us, 2),
                    f"fraction_of_roofline_{how}": round(floor_us / us_fused, 3),
                    "nvlink_bytes_per_rank": (tp - 1) * M * k * 16,
                    "baseline_nvlink_bytes_per_rank": (tp - 1) * M * V * 4, "peer_status_ok": ok})
        if rank == 0:
            print(json.dumps(out[-1]), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--rows", default="1,8,64,256")
    ap.add_argument("--ops", default="1,2")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    args.rows = [int(m) for m in args.rows.split(",")]
    comm = init_distributed(int(os.environ.get("WORLD_SIZE", "1")), timeout_s=120)
    peer = PeerComm(comm, 5120, m_cap=64, ar_rows=max(args.rows + [64]))
    results = []
    if "1" in args.ops:
        op1(peer, comm, args, results)
    if "2" in args.ops:
        op2(peer, comm, args, results)
    if comm.rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    dist.barrier()
    torch.cuda.synchronize()
    peer.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
