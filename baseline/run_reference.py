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


def _sm90_dispatch_defect() -> str | None:
    """The reference picks its warp-specialised prefill attention on compute capability >= 9.0 and calls
    it with a `num_stages` keyword that the kernel factory does not accept (kernels/gqa_varlen.py:193-196
    against :376-379), so every prefill raises TypeError there.  Seen on a B200 with the 8-layer
    configuration; the reference was developed on sm_80, where the other branch runs.  The check reads the
    installed source as text, so a reference without the defect is run normally."""
    import re
    try:
        import torch
        if not torch.cuda.is_available() or torch.cuda.get_device_capability(0) < (9, 0):
            return None
        src = open(os.path.join(REF, "kernels", "gqa_varlen.py")).read()
    except OSError:
        return None
    sig = re.search(r"def flashattn_ws\((.*?)\):", src, re.S)
    call = re.search(r"return flashattn_ws\((.*?)\)", src, re.S)
    if sig and call and "num_stages" in call.group(1) and "num_stages" not in sig.group(1):
        return ("the unmodified reference cannot prefill on sm_90+: kernels/gqa_varlen.py calls flashattn_ws(num_stages=3) "
                "but flashattn_ws takes no num_stages (TypeError, observed on B200)")
    return None


def run(args) -> dict:
    if not os.path.isdir(os.path.join(REF, "engine")):
        return _unavailable("baseline/_ref is not installed")
    import torch
    if not torch.cuda.is_available():
        return _unavailable("the reference needs a CUDA device")
    why = _sm90_dispatch_defect()
    if why is not None:
        return _unavailable(why) if int(os.environ.get("RANK", "0")) == 0 else None
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
