"""Tracing helpers: NVTX ranges behind an environment flag, and a torch.profiler wrapper that sorts kernel time
into categories.

The reference has no tracing inside the engine; its tests/profile_decode.py:71-114,188-191 wraps one `generate` in
torch.profiler, sums `key_averages()` into keyword buckets and can export a Chrome trace.  Here the same harness is
a library function (`profile_call`), and the model marks every layer and operator with an NVTX range when
`TI_NVTX=1`, so that external timeline tools show the structure of a step.  With the flag off the ranges cost one
attribute lookup.
"""
from __future__ import annotations

import contextlib
import os

_NVTX = os.environ.get("TI_NVTX", "0") == "1"


def nvtx_enabled() -> bool:
    return _NVTX


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _NVTX:
        yield
        return
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_mark(name: str):
    """Opens a range that the next nvtx_mark / nvtx_end closes: for straight-line code with many phases."""
    if _NVTX:
        import torch
        torch.cuda.nvtx.range_pop() if getattr(nvtx_mark, "_open", False) else None
        torch.cuda.nvtx.range_push(name)
        nvtx_mark._open = True


def nvtx_end():
    if _NVTX and getattr(nvtx_mark, "_open", False):
        import torch
        torch.cuda.nvtx.range_pop()
        nvtx_mark._open = False


# kernel-name keywords -> category; first match wins (names of this package's kernels first, then ATen / NCCL)
CATEGORIES = (
    ("GEMV (W8A16 / bf16, fused norm / SwiGLU / all-reduce)", ("gemv_kernel",)),
    ("GEMM (tcgen05)", ("gemm_w8a16_kernel", "quant_rows")),
    ("Fused all-reduce (many rows)", ("ar_rows_kernel",)),
    ("Attention", ("attn_kernel", "attn_merge", "attn_prefill", "qkv_prep")),
    ("DeltaNet", ("gdn_",)),
    ("Sampling", ("topk_", "sample_kernel", "logits_edit")),
    ("Embedding", ("embed_kernel",)),
    ("Norm / pointwise", ("rmsnorm_kernel", "act_mul", "swiglu")),
    ("Communication (NCCL)", ("nccl", "AllReduce", "AllGather", "Broadcast")),
    ("Memory", ("memcpy", "memset", "copy_kernel", "Memcpy", "Memset")),
    ("Elementwise (ATen)", ("elementwise", "vectorized", "unrolled")),
    ("Reduction (ATen)", ("reduce_kernel", "softmax", "sort", "scan", "topk")),
)


def categorize(kernel_name: str) -> str:
    for cat, keys in CATEGORIES:
        if any(k in kernel_name for k in keys):
            return cat
    return "Other"


def profile_call(fn, *, trace_path: str | None = None, top: int = 15, with_cpu: bool = True) -> dict:
    """Runs fn() under torch.profiler (CPU + CUDA activities, shapes recorded) and returns
    {"categories": {name: us}, "top_kernels": [(name, calls, us)], "total_cuda_us": ...}; writes a Chrome trace to
    `trace_path` when given."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    acts = [ProfilerActivity.CUDA] + ([ProfilerActivity.CPU] if with_cpu else [])
    with profile(activities=acts, record_shapes=True) as prof:
        fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    cats, kernels = {}, []
    for ev in prof.key_averages():
        us = float(getattr(ev, "self_device_time_total", 0.0) or getattr(ev, "self_cuda_time_total", 0.0) or 0.0)
        if us <= 0.0:
            continue
        cats[categorize(ev.key)] = cats.get(categorize(ev.key), 0.0) + us
        kernels.append((ev.key, int(ev.count), us))
    kernels.sort(key=lambda k: -k[2])
    if trace_path:
        prof.export_chrome_trace(trace_path)
    return {"categories": dict(sorted(cats.items(), key=lambda kv: -kv[1])), "top_kernels": kernels[:top],
            "total_cuda_us": sum(cats.values())}


def format_profile(res: dict) -> str:
    tot = max(res["total_cuda_us"], 1e-9)
    lines = ["category                                                     us      share"]
    for name, us in res["categories"].items():
        lines.append(f"{name:56s} {us:10.1f}  {100 * us / tot:5.1f} %")
    lines.append("")
    lines.append("top kernels                                                calls         us")
    for name, calls, us in res["top_kernels"]:
        lines.append(f"{name[:58]:58s} {calls:6d} {us:10.1f}")
    return "\n".join(lines)
