"""Tensor parallelism on real GPUs (2 or 4 ranks): the fused row-parallel all-reduce over peer memory, the
fused top-k candidate exchange, KV-head replication and CUDA-graph decode; checked against the CPU oracle
and against the NCCL baseline path."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tp, fused, port, nvls=False, **extra_env):
    # NVLS (NCCL's and this package's own multimem loads) stays off except in the tests that are about it
    env = dict(os.environ, TI_TEST_FUSED="1" if fused else "0", NCCL_NVLS_ENABLE="1" if nvls else "0",
               TI_NVLS="1" if nvls else "0", **extra_env)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(tp),
                        "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_gpu_worker.py")],
                       capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    line = [l for l in r.stdout.splitlines() if l.startswith("TP_RESULT ")][0]
    return json.loads(line[len("TP_RESULT "):])


def _near_greedy(tokens, prompt, slack=0.08, tp=2):
    from tileinfer_b200.models.config import TINY_HYBRID_TP, TINY_HYBRID_TP8
    from tileinfer_b200.models.reference_cpu import naive_logits
    from tileinfer_b200.models.weights import RandomWeights
    cfg = TINY_HYBRID_TP8 if tp == 8 else TINY_HYBRID_TP
    lg = naive_logits(cfg, RandomWeights(cfg, 0), list(prompt) + list(tokens), quant="w8a16")
    worst = max(float(lg[len(prompt) - 1 + i].max() - lg[len(prompt) - 1 + i][t]) for i, t in enumerate(tokens))
    assert worst <= slack, f"token off the oracle arg-max by {worst}"


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_fused_tp_matches_oracle_and_all_ranks_agree(tp):
    if torch.cuda.device_count() < tp:
        pytest.skip(f"needs {tp} GPUs")
    res = _run(tp, True, 29540 + tp)
    ranks = res["ranks"]
    assert all(r["status"] == 0 for r in ranks), "a peer wait timed out"
    assert all(r["greedy"] == ranks[0]["greedy"] and r["sampled"] == ranks[0]["sampled"] for r in ranks)
    assert ranks[0]["graph_launches"] > 0 and all(r["scrubs"] >= 2 for r in ranks)
    for p, o in zip(res["prompts"], ranks[0]["greedy"]):
        assert len(o) == 12
        _near_greedy(o, p, tp=tp)


def test_fused_tp_with_nvls_multimem_reduction():
    """The many-row all-reduce reading the partial sums through the NVLS multicast window (multimem.ld_reduce):
    same tokens as the oracle, all ranks agree.  Nobody leaves in this test."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(2, True, 29551, nvls=True)
    ranks = res["ranks"]
    if not all(r.get("nvls") for r in ranks):
        pytest.skip("no NVLS multicast binding on this machine (torch symmetric memory reported none)")
    assert all(r["status"] == 0 for r in ranks)
    assert all(r["greedy"] == ranks[0]["greedy"] and r["sampled"] == ranks[0]["sampled"] for r in ranks)
    for p, o in zip(res["prompts"], ranks[0]["greedy"]):
        _near_greedy(o, p)


@pytest.mark.parametrize("tp,nvls", [(2, True), (4, False), (8, True)])
def test_fused_tp_two_shot_allreduce(tp, nvls):
    """The two-shot form of the many-row all-reduce (every rank reduces 1/tp of the rows and writes the sums into all
    ranks' buffers: multimem.ld_reduce + multimem.st with NVLS, peer loads and stores without), forced for every
    prefill chunk of 8 rows or more: same tokens as the oracle, all ranks agree, no wait runs out."""
    if torch.cuda.device_count() < tp:
        pytest.skip(f"needs {tp} GPUs")
    res = _run(tp, True, 29560 + tp, nvls=nvls, TI_AR_TWO_SHOT_ROWS="8", TI_AR_TWO_SHOT_TP="2")
    ranks = res["ranks"]
    if nvls and not all(r.get("nvls") for r in ranks):
        pytest.skip("no NVLS multicast binding on this machine (torch symmetric memory reported none)")
    assert all(r["status"] == 0 for r in ranks)
    assert all(r["greedy"] == ranks[0]["greedy"] and r["sampled"] == ranks[0]["sampled"] for r in ranks)
    for p, o in zip(res["prompts"], ranks[0]["greedy"]):
        _near_greedy(o, p, tp=tp)


def test_nccl_baseline_path_tp2():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(2, False, 29549)
    ranks = res["ranks"]
    assert all(r["greedy"] == ranks[0]["greedy"] for r in ranks)
    for p, o in zip(res["prompts"], ranks[0]["greedy"]):
        _near_greedy(o, p)


def test_rank_leaving_between_steps_is_noticed_on_the_host():
    """2 GPUs, NVLS off, plain peer stores only: a rank exits between two requests; the survivor's heartbeat
    reports it before the next launch and its CUDA context stays usable."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, TI_TEST_MODE="leave", NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29547", os.path.join(ROOT, "tests", "tp_gpu_worker.py")],
                       capture_output=True, text=True, env=env, timeout=240)
    line = [l for l in r.stdout.splitlines() if l.startswith("LEAVE_RESULT")]
    assert line and "PEER_LOST [1]" in line[0] and "context_ok=True" in line[0], (r.stdout[-800:], r.stderr[-2000:])
