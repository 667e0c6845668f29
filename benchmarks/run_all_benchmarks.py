"""Runs the benchmark suite and aggregates the results into one JSON file.

Counterpart of the reference's tests/run_all_benchmarks.py and of the scaling table of
tests/bench_multi_gpu.py:235-275: for every tensor-parallel degree in --gpus the headline decode bench
(`bench.py`), the batched-decode sweep, the prefill bench and the fused-collective microbench are run as child
processes (torchrun for more than one GPU); the aggregate holds every JSON line they print plus a scaling table
(tok/s, speed-up over one GPU, efficiency = speed-up / GPUs) for decode and prefill.

    python benchmarks/run_all_benchmarks.py --gpus 1,2,4,8 --out all_benchmarks.json [--quick]
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(script, n, extra, port, timeout):
    path = os.path.join(ROOT, script)
    if n == 1:
        cmd = [sys.executable, path] + extra
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
               "127.0.0.1", "--master-port", str(port), path] + extra
    t0 = time.time()
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
        out, rc = r.stdout, r.returncode
        err = r.stderr[-800:] if rc else ""
    except subprocess.TimeoutExpired:
        out, rc, err = "", -9, "timeout"
    lines = []
    for l in out.splitlines():
        if l.startswith("{"):
            try:
                lines.append(json.loads(l))
            except ValueError:
                pass
    return {"script": script, "n_gpus": n, "rc": rc, "seconds": round(time.time() - t0, 1), "results": lines, "stderr_tail": err}


def scaling(rows, key="value"):
    base = next((r[key] for r in rows if r["n_gpus"] == 1), None)
    out = []
    for r in sorted(rows, key=lambda r: r["n_gpus"]):
        sp = r[key] / base if base else None
        out.append({"n_gpus": r["n_gpus"], key: r[key], "speedup": None if sp is None else round(sp, 3),
                    "efficiency": None if sp is None else round(sp / r["n_gpus"], 3)})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", default="1")
    ap.add_argument("--out", default="all_benchmarks.json")
    ap.add_argument("--quick", action="store_true", help="fewer steps, shorter prompts")
    ap.add_argument("--model", default="preset:qwen3.6-27b")
    args = ap.parse_args()
    ns = [int(n) for n in args.gpus.split(",")]
    steps = "20" if args.quick else "64"
    plen = "8192" if args.quick else "32768"
    runs = []
    for i, n in enumerate(ns):
        port = 29700 + 10 * i
        runs.append(run("bench.py", n, ["--gpus", str(n), "--steps", steps, "--warmup", "5", "--model", args.model], port, 1800))
        runs.append(run("benchmarks/bench_batched_decode.py", n, ["--model", args.model, "--steps", steps, "--batches",
                                                                  "1,8,64" if args.quick else "1,2,4,8,16,32,64"], port + 1, 1800))
        runs.append(run("benchmarks/bench_prefill.py", n, ["--model", args.model, "--prompts", "1", "--prompt-len", plen,
                                                           "--chunk", "8192"], port + 2, 1800))
        if n == 1:      # kernel micro-benchmarks (one GPU)
            for script, extra in (("benchmarks/bench_gemv.py", ["--chain"]), ("benchmarks/bench_gemm.py", ["--M", "64", "2048", "8192"]),
                                  ("benchmarks/bench_attn.py", ["--max-len", plen]), ("benchmarks/bench_gdn.py", [])):
                runs.append(run(script, 1, extra, port + 4, 1800))
        if n > 1:
            runs.append(run("benchmarks/bench_fused_collectives.py", n, ["--iters", "30" if args.quick else "100"], port + 3, 1800))
    decode = [r["results"][-1] for r in runs if r["script"] == "bench.py" and r["results"]]
    prefill = [r["results"][-1] for r in runs if r["script"].endswith("bench_prefill.py") and r["results"]]
    agg = {"model": args.model, "gpus": ns, "runs": runs,
           "decode_scaling": scaling(decode), "prefill_scaling": scaling(prefill),
           "decode_e2e_scaling": scaling([dict(n_gpus=d["n_gpus"], value=d["e2e"]["value"]) for d in decode if "e2e" in d])}
    with open(args.out, "w") as f:
        json.dump(agg, f, indent=1)
    print(json.dumps({"decode_scaling": agg["decode_scaling"], "prefill_scaling": agg["prefill_scaling"],
                      "failed": [(r["script"], r["n_gpus"]) for r in runs if r["rc"] != 0]}))


if __name__ == "__main__":
    main()
