"""Attention micro-benchmark: correctness against torch SDPA plus a throughput sweep.

Counterpart of the reference's kernels/_bench_gqa.py:131-158 (flash kernel against torch SDPA, TFLOP/s as a
fraction of a hard-coded A100 peak).  Here:

* prefill: the tcgen05 varlen kernel (ops/csrc/attn_prefill.cu) on one causal sequence of 1k..32k tokens read
  straight from scattered KV pages; TFLOP/s = 4 * T^2/2 * D * heads / time against the MEASURED cuBLAS bf16
  throughput of this GPU (MEASURED_PEAKS.json, `bf16_tflops_sustained`);
* decode: the split-KV paged kernel (ops/csrc/attn_paged.cu) for a batch of single-token queries; GB/s of K/V
  bytes against the MEASURED copy bandwidth (`hbm_gbs`).

    python benchmarks/bench_attn.py [--out attn.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
BF16 = torch.bfloat16


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["bf16_tflops_sustained"], p["hbm_gbs"], "measured"
    except Exception:
        return 1400.0, 6650.0, "fallback"


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()                       # write a buffer larger than L2 between timed iterations
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def paged(T, hkv, D, extra=8):
    nb = (T + 15) // 16
    perm = torch.randperm(nb + extra)
    table = perm[:nb].int().cuda()
    K = torch.randn(nb * 16, hkv, D, device="cuda").to(BF16)
    V = torch.randn(nb * 16, hkv, D, device="cuda").to(BF16)
    kc = torch.zeros(nb + extra, hkv, 16, D, dtype=BF16, device="cuda")
    vc = torch.zeros(nb + extra, hkv, D, 16, dtype=BF16, device="cuda")
    kc[table.long()] = K.view(nb, 16, hkv, D).permute(0, 2, 1, 3)
    vc[table.long()] = V.view(nb, 16, hkv, D).permute(0, 2, 3, 1)
    return K[:T], V[:T], kc, vc, table, nb + extra


def prefill_case(F, T, hq, hkv, D, flush, check):
    K, V, kc, vc, table, nblocks = paged(T, hkv, D)
    q = (2.0 * torch.randn(T, hq, D, device="cuda")).to(BF16)
    proj = torch.randn(T, hq * 2 * D, device="cuda").to(BF16)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    tiles = [(min(T, a + 128), 0, a, min(128, T - a)) for a in range(0, T, 128)]
    tiles.sort(reverse=True)
    tl = torch.tensor([[t[1] for t in tiles], [t[2] for t in tiles], [t[3] for t in tiles]], dtype=torch.int32, device="cuda")
    out = torch.zeros(T, hq * D, dtype=BF16, device="cuda")
    bt = table.view(1, -1).contiguous()

    def run():
        F.attn_prefill(q, kc, vc, nblocks, bt, pos, tl, proj, out, hq=hq, hkv=hkv, D=D, max_blocks=bt.shape[1], ld=proj.shape[1])
    run()
    err = None
    if check:
        G = hq // hkv
        ref = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(0, 1).unsqueeze(0).float(), K.transpose(0, 1).repeat_interleave(G, 0).unsqueeze(0).float(),
            V.transpose(0, 1).repeat_interleave(G, 0).unsqueeze(0).float(), is_causal=True)[0].transpose(0, 1)
        gate = proj.view(T, hq, 2 * D)[..., D:].float()
        err = float((out.view(T, hq, D).float() - ref * torch.sigmoid(gate)).abs().max())
    ms = timed(run, 5, flush)
    flops = 4.0 * (T * (T + 1) / 2) * D * hq
    return ms, flops / ms / 1e9, err


def decode_case(F, B, ctx, hq, hkv, D, flush):
    nb_seq = (ctx + 15) // 16
    nblocks = B * nb_seq + 4
    kc = torch.randn(nblocks, hkv, 16, D, device="cuda").to(BF16)
    vc = torch.randn(nblocks, hkv, D, 16, device="cuda").to(BF16)
    bt = torch.randperm(nblocks)[:B * nb_seq].int().view(B, nb_seq).cuda()
    q = torch.randn(B, hq, D, device="cuda").to(BF16)
    proj = torch.randn(B, hq * 2 * D, device="cuda").to(BF16)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    nsplit = max(1, min(32, -(-1184 // (B * hkv))))
    qg = torch.stack([torch.arange(B), torch.arange(B), torch.ones(B, dtype=torch.long)]).int().cuda()
    items = B * hkv * nsplit
    o_part = torch.empty(items * 16 * D, device="cuda")
    ml = torch.empty(items * 32, device="cuda")
    out = torch.zeros(B, hq * D, dtype=BF16, device="cuda")
    a = F.AttnParams()
    a.q, a.kcache, a.vcache, a.block_tables, a.positions = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), pos.data_ptr()
    a.qg_seq, a.qg_tok0, a.qg_ntok = qg[0].data_ptr(), qg[1].data_ptr(), qg[2].data_ptr()
    a.o_part, a.ml_part, a.gate_src, a.out = o_part.data_ptr(), ml.data_ptr(), proj.data_ptr(), out.data_ptr()
    a.hq, a.hkv, a.max_blocks, a.nsplit, a.ld, a.num_qg = hq, hkv, nb_seq, nsplit, proj.shape[1], B
    a.scale_log2e = D ** -0.5 * 1.4426950408889634
    ms = timed(lambda: F.attn_paged(a, D), 5, flush)
    bytes_ = 2.0 * B * ctx * hkv * D * 2
    return ms, bytes_ / ms / 1e6


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--max-len", type=int, default=32768)
    args = ap.parse_args()
    from tileinfer_b200.ops import functional as F
    F.L()
    tflops_peak, hbm, how = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    hq, hkv, D = 24, 4, 256
    for T in (1024, 2048, 4096, 8192, 16384, 32768):
        if T > args.max_len:
            break
        ms, tf, err = prefill_case(F, T, hq, hkv, D, flush, check=T <= 4096)
        rows.append({"op": "prefill_tcgen05", "tokens": T, "heads": f"{hq}q/{hkv}kv", "D": D, "ms": round(ms, 3),
                     "tflops": round(tf, 1), f"fraction_of_{how}_bf16_sustained": round(tf / tflops_peak, 3),
                     "max_abs_err_vs_sdpa": err})
        print(json.dumps(rows[-1]), flush=True)
    for hq_, hkv_ in ((3, 1),):            # per-rank heads at TP = 8 (KV heads replicated)
        ms, tf, err = prefill_case(F, 8192, hq_, hkv_, D, flush, check=False)
        rows.append({"op": "prefill_tcgen05", "tokens": 8192, "heads": f"{hq_}q/{hkv_}kv", "D": D, "ms": round(ms, 3),
                     "tflops": round(tf, 1), f"fraction_of_{how}_bf16_sustained": round(tf / tflops_peak, 3)})
        print(json.dumps(rows[-1]), flush=True)
    for B, ctx in ((1, 256), (1, 1024), (1, 4096), (1, 32768), (16, 2048), (64, 2048), (64, 8192)):
        ms, gbs = decode_case(F, B, ctx, hq, hkv, D, flush)
        rows.append({"op": "decode_paged_splitkv", "batch": B, "context": ctx, "ms": round(ms, 4), "kv_gbs": round(gbs, 1),
                     f"fraction_of_{how}_hbm": round(gbs / hbm, 3)})
        print(json.dumps(rows[-1]), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
