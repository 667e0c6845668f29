"""Reference arm of bench.py: runs the UNMODIFIED reference package installed under baseline/_ref through
its own public API (engine.llm.LLM.generate) on a synthesised checkpoint of the named architecture."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}


def run(args) -> dict:
    if not os.path.isdir(os.path.join(REF, "engine")):
        return _unavailable("baseline/_ref is not installed")
    rank = int(os.environ.get("RANK", "0"))
    preset = args.model.split(":", 1)[1] if ":" in args.model else args.model
    ckpt = os.path.join(os.environ.get("TI_REF_CKPT_DIR", "/tmp"), f"ti_ref_ckpt_{preset}")
    done = os.path.join(ckpt, "DONE")
    if rank == 0 and not os.path.exists(done):
        r = subprocess.run([sys.executable, os.path.join(HERE, "make_checkpoint.py"), preset, ckpt],
                           capture_output=True, text=True)
        if r.returncode != 0:
            with open(os.path.join(os.environ.get("TI_REF_CKPT_DIR", "/tmp"), f"ti_ref_ckpt_{preset}.failed"), "w") as f:
                f.write(r.stderr[-2000:])
    t0 = time.time()
    while not os.path.exists(done):
        if os.path.exists(ckpt + ".failed") or time.time() - t0 > 3600:
            return _unavailable("could not synthesise the checkpoint the reference needs (see make_checkpoint.py)") if rank == 0 else None
        time.sleep(2)
    env = dict(os.environ)
    env["PYTHONPATH"] = REF
    env.setdefault("TILELANG_CACHE_DIR", os.path.join(os.environ.get("TI_REF_CKPT_DIR", "/tmp"), "ti_ref_tilelang_cache"))
    cmd = [sys.executable, os.path.join(HERE, "ref_worker.py"), "--ckpt", ckpt, "--gpus", str(args.gpus),
           "--steps", str(args.steps), "--warmup", str(args.warmup), "--model-name", preset]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=REF,
                           timeout=float(os.environ.get("TI_REF_TIMEOUT", "3000")))
    except subprocess.TimeoutExpired:
        return _unavailable("the reference did not finish within its time limit") if rank == 0 else None
    if rank != 0:
        return None
    for line in r.stdout.splitlines():
        if line.startswith("REF_RESULT "):
            return json.loads(line[len("REF_RESULT "):])
    tail = (r.stderr or r.stdout or "").strip().splitlines()[-3:]
    return _unavailable("reference run failed: " + " | ".join(tail))
