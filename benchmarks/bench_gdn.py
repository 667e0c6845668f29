"""Gated-DeltaNet micro-benchmark at the 27B head shapes (16 k-heads, 48 v-heads, 128 x 128 state per head).

* prefill: the chunk-parallel kernels (ops/csrc/gdn_chunk.cu) against the token-serial kernel (ops/csrc/gdn.cu)
  for one sequence of T tokens: time, microseconds per token, and how the time compares with streaming the
  projections in and the outputs out once (the floor of any prefill form);
* decode: one token for each of B sequences with the three decode kernels (one block per head and sequence, column-split
  blocks, staged blocks that walk several sequences): time and the recurrent-state bytes moved per second against the
  measured copy bandwidth (the state is read and written once per token: 2 * B * 48 * 128 * 128 * 4 bytes).

    python benchmarks/bench_gdn.py [--prefill 2048 8192] [--decode 1 16 64 256] [--bf16-state]
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

BF16 = torch.bfloat16
HK, HV, DK, DV = 16, 48, 128, 128


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def timed(fn, iters, flush):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / iters


def common(F, T, nslots, state_bf16):
    kd, vd = HK * DK, HV * DV
    ld = 2 * kd + 2 * vd + 2 * HV
    g = dict(ld=ld, vd=vd)
    g["proj"] = torch.randn(T, ld, device="cuda").to(BF16)
    g["conv_w"] = torch.randn(2 * kd + vd, 4, device="cuda") * 0.5
    g["neg"] = (-(torch.randn(HV, device="cuda") * 0.5).exp()).contiguous()
    g["dt_bias"] = torch.randn(HV, device="cuda") * 0.5
    g["norm_w"] = 1 + 0.1 * torch.randn(DV, device="cuda")
    sdt = BF16 if state_bf16 else torch.float32
    g["state"] = (torch.randn(nslots, HV, DK, DV, device="cuda") * 0.05).to(sdt)
    g["cs"] = torch.randn(nslots, HV, 3, 2 * DK + DV, device="cuda").to(BF16)
    g["out"] = torch.zeros(T, vd, dtype=BF16, device="cuda")
    return g


def fill(p, g, slots, cu=None):
    p.proj, p.conv_w, p.neg_a_exp = g["proj"].data_ptr(), g["conv_w"].data_ptr(), g["neg"].data_ptr()
    p.dt_bias, p.norm_w = g["dt_bias"].data_ptr(), g["norm_w"].data_ptr()
    p.state, p.conv_state, p.slots, p.out = g["state"].data_ptr(), g["cs"].data_ptr(), slots.data_ptr(), g["out"].data_ptr()
    if cu is not None:
        p.cu = cu.data_ptr()
    p.ld, p.hk, p.hv, p.eps = g["ld"], HK, HV, 1e-6


def prefill_case(F, T, state_bf16, flush):
    g = common(F, T, 1, state_bf16)
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    p = F.GdnParams()
    fill(p, g, slots, cu)
    ms_serial = timed(lambda: F.gdn_step(p, 1, DK, DV, state_bf16), 3, flush)
    ck, seq_ck = F.gdn_chunk_table([0, T])
    ck, seq_ck = ck.cuda(), seq_ck.cuda()
    c = F.GdnChunkParams()
    fill(c, g, slots, cu)
    c.ck_seq, c.ck_tok0, c.ck_ntok, c.ck_snap = ck[0].data_ptr(), ck[1].data_ptr(), ck[2].data_ptr(), ck[3].data_ptr()
    c.seq_ck, c.nc = seq_ck.data_ptr(), ck.shape[1]
    ws = F.GdnChunkWorkspace("cuda").get(ck.shape[1] * HV, DK, DV)
    c.wf, c.qf, c.mf, c.kf, c.u, c.gamma = (b.data_ptr() for b in ws)
    ms_chunk = timed(lambda: F.gdn_chunked(c, 1, T, DK, DV, state_bf16), 5, flush)
    return ms_serial, ms_chunk, T * (g["ld"] + g["vd"]) * 2.0


def decode_case(F, B, state_bf16, flush):
    g = common(F, B, B + 2, state_bf16)
    slots = torch.randperm(B + 2, device="cuda")[:B].to(torch.int32)
    p = F.GdnParams()
    fill(p, g, slots)
    res = {}
    res["tiled"] = timed(lambda: F.gdn_step(p, B, DK, DV, state_bf16), 5, flush)
    res["decode"] = timed(lambda: F.gdn_step(p, B, DK, DV, state_bf16, single=True), 5, flush)
    res["decode_staged"] = timed(lambda: F.gdn_step(p, B, DK, DV, state_bf16, single=True, staged=True), 5, flush)
    return res, 2.0 * B * HV * DK * DV * (2 if state_bf16 else 4)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prefill", type=int, nargs="*", default=[2048, 8192])
    ap.add_argument("--decode", type=int, nargs="*", default=[1, 16, 64, 256])
    ap.add_argument("--bf16-state", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    from tileinfer_b200.ops import functional as F
    F.L()
    hbm, how = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for T in args.prefill:
        ms_s, ms_c, io = prefill_case(F, T, args.bf16_state, flush)
        rows.append({"op": "gdn_prefill", "tokens": T, "serial_ms": round(ms_s, 3), "chunked_ms": round(ms_c, 3),
                     "chunked_us_per_token": round(ms_c * 1e3 / T, 3), "speedup": round(ms_s / ms_c, 2),
                     "io_floor_fraction": round(io / hbm / 1e6 / ms_c, 3)})
        print(json.dumps(rows[-1]), flush=True)
    for B in args.decode:
        res, state_bytes = decode_case(F, B, args.bf16_state, flush)
        row = {"op": "gdn_decode", "batch": B, "state": "bf16" if args.bf16_state else "fp32"}
        for k, ms in res.items():
            row[k + "_us"] = round(ms * 1e3, 1)
            row[k + f"_state_gbs"] = round(state_bytes / ms / 1e6, 1)
        row[f"best_fraction_of_{how}_hbm"] = round(state_bytes / min(res.values()) / 1e6 / hbm, 3)
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
