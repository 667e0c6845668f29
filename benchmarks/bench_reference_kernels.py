"""Kernel-level anchors: the reference's OWN kernels, imported unchanged from baseline/_ref, timed on this GPU next
to this package's kernels at the 27B shapes.

The reference's engine cannot serve a request on sm_90+ (its prefill attention dispatch passes a keyword its kernel
factory does not take), so an end-to-end ratio on the same box does not exist; its decode kernels can still be
called one by one.  Entry points: kernels/splitk_gemv.py:220-229 (`gemv_int8`), kernels/gqa_decode_paged.py:374-437,
kernels/deltanet_fused.py:634-684, kernels/rms_norm.py, kernels/residual_rmsnorm.py.  A kernel that does not build or
run here is recorded with its one-line error; nothing of the reference is patched.  CUDA events, weights rotated over
copies larger than L2.

    python benchmarks/bench_reference_kernels.py [--out ref_kernels.json]
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

BF16 = torch.bfloat16


def timed(fn, iters=30, warm=5):
    """us per call and how it was launched: inside a CUDA graph of `iters` calls where the kernel can be captured
    (device time without host launch overhead: how a decode step runs it), else eagerly back to back."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    how, g = "graph", torch.cuda.CUDAGraph()
    try:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for i in range(iters):
                    fn(i)
        torch.cuda.current_stream().wait_stream(s)
        g.replay()
        torch.cuda.synchronize()
        run = g.replay
    except Exception:                              # noqa: BLE001  (not capturable: time it eagerly)
        how = "eager"
        torch.cuda.synchronize()

        def run():
            for i in range(iters):
                fn(i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters, how


def guarded(name, rows, build):
    """Runs build() -> (callable, note); records its time or the one-line error."""
    try:
        fn, note = build()
        us, how = timed(fn)
        rows.append({"kernel": name, "impl": "reference", "us": round(us, 2), "launch": how, "note": note})
    except Exception as e:                       # noqa: BLE001  (the record IS the result)
        rows.append({"kernel": name, "impl": "reference", "error": f"{type(e).__name__}: {str(e)[:160]}".replace("\n", " ")})
    print(json.dumps(rows[-1]), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    from tileinfer_b200.ops import functional as F
    F.L()
    rows = []
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    have_ref = os.path.isdir(os.path.join(ref_dir, "kernels"))
    if have_ref:
        sys.path.insert(0, ref_dir)
    shapes = {"in_proj": (16480, 5120), "gate_up": (34816, 5120), "down": (5120, 17408), "out_proj": (5120, 6144)}

    # ---- W8A16 GEMV, one row
    for name, (N, K) in shapes.items():
        ncopy = max(2, int(400e6 // (N * K)) + 1)
        ws = [torch.randn(N, K, device="cuda") * 0.05 for _ in range(ncopy)]
        x = torch.randn(1, K, device="cuda").to(BF16)
        ours = [F.LinearW(w, True) for w in ws]
        out = torch.zeros(1, N, dtype=BF16, device="cuda")
        ps = [F.make_gemv_params(W, x, out, 1) for W in ours]
        us, how = timed(lambda i: F.gemv_launch(ps[i % ncopy], F.W_INT8))
        rows.append({"kernel": f"gemv_w8a16 {name} N={N} K={K}", "impl": "tileinfer_b200", "us": round(us, 2), "launch": how,
                     "weight_gbs": round(N * K / us / 1e3, 1)})
        print(json.dumps(rows[-1]), flush=True)
        if have_ref:
            def build(ws=ws, x=x, N=N, K=K, ncopy=ncopy):
                from kernels.splitk_gemv import gemv_int8
                from model.qwen_36 import quantize_weight_int8
                qs = [quantize_weight_int8(w.to(BF16)) for w in ws]
                xv = x[0].contiguous()
                return (lambda i: gemv_int8(xv, qs[i % ncopy][0], qs[i % ncopy][1])), "kernels/splitk_gemv.py gemv_int8"
            guarded(f"gemv_int8 {name} N={N} K={K}", rows, build)
        del ws, ours
        torch.cuda.empty_cache()

    # ---- RMSNorm / residual + RMSNorm, one row of 5120
    h = torch.randn(1, 5120, device="cuda").to(BF16)
    w = torch.zeros(5120, dtype=BF16, device="cuda")
    o = torch.zeros_like(h)
    r = torch.zeros_like(h)
    us, how = timed(lambda i: F.rmsnorm(h, w, 1e-6, out=o))
    rows.append({"kernel": "rmsnorm 1x5120", "impl": "tileinfer_b200", "us": round(us, 2), "launch": how,
                 "note": "stand-alone form; in the decode step the norm is the prologue of the consuming GEMV (no launch)"})
    print(json.dumps(rows[-1]), flush=True)
    us, how = timed(lambda i: F.rmsnorm(h, w, 1e-6, add=h, out=o, r_out=r))
    rows.append({"kernel": "residual+rmsnorm 1x5120", "impl": "tileinfer_b200", "us": round(us, 2), "launch": how})
    print(json.dumps(rows[-1]), flush=True)
    if have_ref:
        def build_norm():
            from kernels.rms_norm import rmsnorm
            return (lambda i: rmsnorm(h, w, 1e-6, True)), "kernels/rms_norm.py rmsnorm"
        guarded("rms_norm 1x5120", rows, build_norm)

        def build_rnorm():
            from kernels.residual_rmsnorm import residual_rmsnorm
            return (lambda i: residual_rmsnorm(h, h, w, 1e-6, True)), "kernels/residual_rmsnorm.py residual_rmsnorm"
        guarded("residual_rmsnorm 1x5120", rows, build_rnorm)

    # ---- paged decode attention, batch 1 and 64, context 2048
    for B in (1, 64):
        ctx, hq, hkv, D = 2048, 24, 4, 256
        nb_seq = ctx // 16
        nblocks = B * nb_seq + 1
        kc = torch.randn(nblocks, hkv, 16, D, device="cuda").to(BF16)
        vc = torch.randn(nblocks, hkv, D, 16, device="cuda").to(BF16)
        bt = torch.arange(B * nb_seq, dtype=torch.int32, device="cuda").view(B, nb_seq)
        q = torch.randn(B, hq, D, device="cuda").to(BF16)
        proj = torch.randn(B, hq * 2 * D, device="cuda").to(BF16)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
        nsplit = max(1, min(32, -(-8 * F.NUM_SMS // (B * hkv))))
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
        us, how = timed(lambda i: F.attn_paged(a, D))
        rows.append({"kernel": f"paged decode attention B={B} ctx={ctx}", "impl": "tileinfer_b200", "us": round(us, 2),
                     "launch": how, "note": "split-KV + merge + sigmoid gate (2 launches)"})
        print(json.dumps(rows[-1]), flush=True)
        if have_ref:
            def build_attn(B=B, q=q, ctx=ctx, hq=hq, hkv=hkv, D=D, nb_seq=nb_seq, nblocks=nblocks, bt=bt):
                from kernels.gqa_decode_paged import gqa_decode_paged_fn
                kpages = torch.randn(nblocks, 16, hkv, D, device="cuda").to(BF16)
                vpages = torch.randn(nblocks, 16, hkv, D, device="cuda").to(BF16)
                lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
                return (lambda i: gqa_decode_paged_fn(q, kpages, vpages, bt, lens, 16)), \
                    "kernels/gqa_decode_paged.py gqa_decode_paged_fn (no split-KV, no output gate)"
            guarded(f"gqa_decode_paged B={B} ctx={ctx}", rows, build_attn)

    # ---- DeltaNet decode step, batch 1 (48 v-heads)
    hk, hv, dk, dv = 16, 48, 128, 128
    ld = 2 * hk * dk + 2 * hv * dv + 2 * hv
    proj = torch.randn(1, ld, device="cuda").to(BF16)
    p = F.GdnParams()
    conv_w = torch.randn(2 * hk * dk + hv * dv, 4, device="cuda")
    neg, dtb, nw = -torch.rand(hv, device="cuda"), torch.zeros(hv, device="cuda"), torch.ones(dv, device="cuda")
    state = torch.zeros(2, hv, dk, dv, device="cuda")
    cs = torch.zeros(2, hv, 3, 2 * dk + dv, dtype=BF16, device="cuda")
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    outg = torch.zeros(1, hv * dv, dtype=BF16, device="cuda")
    p.proj, p.conv_w, p.neg_a_exp, p.dt_bias, p.norm_w = proj.data_ptr(), conv_w.data_ptr(), neg.data_ptr(), dtb.data_ptr(), nw.data_ptr()
    p.state, p.conv_state, p.slots, p.cu, p.out = state.data_ptr(), cs.data_ptr(), slots.data_ptr(), cu.data_ptr(), outg.data_ptr()
    p.ld, p.hk, p.hv, p.eps = ld, hk, hv, 1e-6
    us, how = timed(lambda i: F.gdn_step(p, 1, dk, dv, False, single=True))
    rows.append({"kernel": "DeltaNet decode step B=1 (conv + delta rule + gated norm, in place, fp32 state)", "impl": "tileinfer_b200",
                 "us": round(us, 2), "launch": how})
    print(json.dumps(rows[-1]), flush=True)
    if have_ref:
        def build_gdn():
            from kernels.deltanet_fused import fused_postproj_recurrent
            qkv = torch.randn(1, 2 * hk * dk + hv * dv, device="cuda").to(BF16)
            al = torch.randn(1, hv, device="cuda").to(BF16)
            be = torch.randn(1, hv, device="cuda").to(BF16)
            z = torch.randn(1, hv, dv, device="cuda").to(BF16)
            st = torch.zeros(1, hv, dk, dv, dtype=BF16, device="cuda")
            return (lambda i: fused_postproj_recurrent(qkv, al, be, neg, dtb, st, hk, hv, dk, nw.to(BF16), z)), \
                "kernels/deltanet_fused.py fused_postproj_recurrent (no conv, bf16 state, state copied out)"
        guarded("fused_postproj_recurrent B=1", rows, build_gdn)
    if not have_ref:
        rows.append({"impl": "reference", "error": "baseline/_ref is not installed"})
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
