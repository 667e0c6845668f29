"""Tensor-parallel logic on CPU: sharded model + distributed sampling over a fake communicator,
the server's worker protocol, host-side failure detection, and real gloo ranks."""
import json
import os
import subprocess
import sys
import threading
import urllib.request

import pytest
import torch

from tileinfer_b200.engine.llm import LLM
from tileinfer_b200.engine.sampling_params import SamplingParams
from tileinfer_b200.models.config import TINY_HYBRID_TP
from tileinfer_b200.parallel.fake_comm import CommTimeout, run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _prompt(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 1023, (n,), generator=g).tolist()


def _mk(comm=None, tp=1, **kw):
    return LLM("preset:tiny-hybrid-tp", device="cpu", quantization="bf16", num_kvcache_blocks=64, max_num_seqs=4,
               max_model_len=512, tp_size=tp, comm=comm, **kw)


def test_kv_replication_config():
    from tileinfer_b200.models.config import QWEN36_27B
    QWEN36_27B.validate_tp(8)
    assert QWEN36_27B.kv_heads_per_rank(8) == 1
    assert [QWEN36_27B.kv_head_start(8, r) for r in range(8)] == [0, 0, 1, 1, 2, 2, 3, 3]
    assert [QWEN36_27B.kv_head_start(2, r) for r in range(2)] == [0, 2]
    with pytest.raises(ValueError):
        QWEN36_27B.validate_tp(5)


@pytest.mark.parametrize("tp", [2, 4])
def test_tp_ranks_agree_with_single_rank(tp):
    prompts = [_prompt(21, 1), _prompt(40, 2)]
    greedy = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    sampled = SamplingParams(temperature=0.9, top_k=8, max_tokens=8, ignore_eos=True)
    one = _mk()
    want_g = one.generate_token_ids(prompts, greedy)
    want_s = _mk().generate_token_ids(prompts, sampled)

    def rank_fn(comm):
        llm = _mk(comm, tp)
        return llm.generate_token_ids(prompts, greedy), llm.generate_token_ids(prompts, sampled)
    results, errors, _ = run_ranks(tp, rank_fn)
    assert errors == [None] * tp, errors
    for g, s in results:
        assert g == want_g
        assert s == results[0][1]                  # every rank samples the same tokens without a broadcast
    assert TINY_HYBRID_TP.num_kv_heads == 2          # tp=4 exercises KV-head replication


def test_missing_rank_is_detected_on_the_host():
    def rank_fn(comm):
        if comm.rank == 1:
            return "never joins"                      # the rank exits before its first collective
        return _mk(comm, 2)
    results, errors, _ = run_ranks(2, rank_fn, hub_timeout_s=1.0)
    assert isinstance(errors[0], CommTimeout) and "ranks [1]" in str(errors[0])


def test_server_http_and_tp_worker_protocol():
    from tileinfer_b200.server.api_server import Service, make_handler, make_sampling_params
    from http.server import ThreadingHTTPServer
    box = {}

    def rank_fn(comm):
        llm = _mk(comm, 2)
        svc = Service(llm, "tiny")
        if comm.rank != 0:
            svc.worker_loop()
            return "worker done"
        httpd = ThreadingHTTPServer(("127.0.0.1", 0), make_handler(svc))
        box["port"] = httpd.server_address[1]
        t = threading.Thread(target=httpd.serve_forever, daemon=True)
        t.start()
        base = f"http://127.0.0.1:{box['port']}"
        models = json.load(urllib.request.urlopen(base + "/v1/models"))
        req = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0,
               "guided_regex": "[ab]{3}", "stop": ["zz"]}
        r = urllib.request.Request(base + "/v1/chat/completions", json.dumps(req).encode(), {"Content-Type": "application/json"})
        full = json.load(urllib.request.urlopen(r))
        req["stream"] = True
        r = urllib.request.Request(base + "/v1/chat/completions", json.dumps(req).encode(), {"Content-Type": "application/json"})
        sse = urllib.request.urlopen(r).read().decode()
        bad = urllib.request.Request(base + "/v1/chat/completions", b'{"messages": []}', {"Content-Type": "application/json"})
        try:
            urllib.request.urlopen(bad)
            code = 200
        except urllib.error.HTTPError as e:
            code = e.code
        httpd.shutdown()
        svc.shutdown_workers()
        return models, full, sse, code
    results, errors, _ = run_ranks(2, rank_fn, timeout_s=120)
    assert errors == [None, None], errors
    models, full, sse, code = results[0]
    assert results[1] == "worker done"
    assert models["data"][0]["id"] == "tiny" and models["object"] == "list"
    text = full["choices"][0]["message"]["content"]
    assert len(text) == 3 and set(text) <= {"a", "b"} and full["choices"][0]["finish_reason"] == "stop"
    assert full["usage"]["completion_tokens"] == 3 and full["object"] == "chat.completion"
    events = [l[6:] for l in sse.splitlines() if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    streamed = "".join(json.loads(e)["choices"][0]["delta"].get("content", "") for e in events[:-1])
    assert streamed == text
    assert code == 400
    sp = make_sampling_params({"response_format": {"type": "json_object"}, "stop": "x", "top_k": 5})
    assert sp.guided_json is True and sp.stop == ["x"] and sp.top_k == 5
    assert SamplingParams.from_json(sp.to_json()) == sp


def test_gloo_ranks_end_to_end(tmp_path):
    """Two real torch.distributed (gloo) processes run the engine at tp=2 and must agree with tp=1."""
    script = r'''
import sys, json, torch
sys.path.insert(0, %r)
from tileinfer_b200.engine.llm import LLM
from tileinfer_b200.engine.sampling_params import SamplingParams
g = torch.Generator().manual_seed(1)
p = torch.randint(0, 1023, (21,), generator=g).tolist()
llm = LLM("preset:tiny-hybrid-tp", device="cpu", quantization="bf16", num_kvcache_blocks=64, max_num_seqs=4,
          max_model_len=512, tp_size=2, nccl_timeout=60)
out = llm.generate_token_ids([p], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
if llm.comm.rank == 0:
    print("RESULT", json.dumps(out))
import torch.distributed as dist
llm.close()                                  # the engine made the process group, so it also takes it down
assert not dist.is_initialized()
llm.close()
print("CLOSED", flush=True)
''' % ROOT
    path = tmp_path / "tp2_gloo.py"
    path.write_text(script)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(path)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")][0]
    assert r.stdout.count("CLOSED") == 2
    got = json.loads(line[7:])
    g = torch.Generator().manual_seed(1)
    p = torch.randint(0, 1023, (21,), generator=g).tolist()
    assert got == _mk().generate_token_ids([p], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))


def test_heartbeat_reports_silent_peer_with_fake_clock():
    """Three ranks share an in-process store; rank 2 stops beating; the others report it after the timeout,
    and only it."""
    import torch.distributed as dist
    from tileinfer_b200.parallel.watchdog import Heartbeat, PeerLostError
    store = dist.HashStore()
    now = [0.0]
    lost_cb = []
    hbs = [Heartbeat(store, r, 3, interval_s=0.1, timeout_s=1.0, clock=lambda: now[0], on_lost=lost_cb.append)
           for r in range(3)]
    for t in range(5):                       # everybody alive
        now[0] = 0.2 * t
        for h in hbs:
            h.tick()
    assert not any(h.lost for h in hbs)
    for t in range(5, 14):                   # rank 2 is gone from t = 1.0 on
        now[0] = 0.2 * t
        hbs[0].tick()
        hbs[1].tick()
    assert hbs[0].lost == {2} and hbs[1].lost == {2} and sorted(lost_cb) == [2, 2]
    with pytest.raises(PeerLostError) as e:
        hbs[0].check()
    assert e.value.ranks == [2]

    class Broken:                            # the store itself went away: the rank that hosted it is lost
        def set(self, *a):
            raise RuntimeError("connection reset")
    hb = Heartbeat(Broken(), 1, 2, store_owner=0)
    hb.tick()
    assert hb.lost == {0}


def test_engine_notices_rank_that_left_between_steps(tmp_path):
    """gloo, 2 processes: rank 1 leaves between two requests (nothing in flight); rank 0 learns of it from the
    heartbeat on the host and refuses to start the next step instead of blocking in a collective."""
    script = r'''
import os, sys, time, torch
sys.path.insert(0, %r)
import torch.distributed as dist
from tileinfer_b200.engine.llm import LLM
from tileinfer_b200.engine.sampling_params import SamplingParams
from tileinfer_b200.parallel.watchdog import PeerLostError
llm = LLM("preset:tiny-hybrid-tp", device="cpu", quantization="bf16", num_kvcache_blocks=64, max_num_seqs=4,
          max_model_len=512, tp_size=2, nccl_timeout=60, heartbeat_interval=0.1, heartbeat_timeout=1.0)
sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
llm.generate_token_ids([[5, 6, 7, 8]], sp)
dist.barrier()
if llm.comm.rank == 1:
    llm.watchdog.stop()
    os._exit(0)                               # leaves with nothing in flight
time.sleep(2.5)
try:
    llm.generate_token_ids([[9, 10, 11]], sp)
    print("NOT_DETECTED", flush=True)
except PeerLostError as e:
    print("PEER_LOST", e.ranks, flush=True)
os._exit(0)
''' % ROOT
    path = tmp_path / "hb_gloo.py"
    path.write_text(script)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29537")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29537", str(path)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert "PEER_LOST [1]" in r.stdout, (r.stdout[-500:], r.stderr[-1500:])


def test_full_vocab_gather_baseline_matches_candidate_exchange():
    """The measuring baseline (every rank gathers whole logit rows, top-k over the full vocabulary) must pick the
    same tokens as the default path (per-rank top-k, exchange of the k candidates)."""
    prompts = [_prompt(21, 1), _prompt(40, 2)]
    greedy = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    sampled = SamplingParams(temperature=0.9, top_k=8, max_tokens=6, ignore_eos=True)

    def rank_fn(comm):
        a = _mk(comm, 2)
        b = _mk(comm, 2, baseline_full_vocab_gather=True)
        assert b.model_runner.sampler.full_vocab_gather
        return (a.generate_token_ids(prompts, greedy), a.generate_token_ids(prompts, sampled),
                b.generate_token_ids(prompts, greedy), b.generate_token_ids(prompts, sampled))
    results, errors, _ = run_ranks(2, rank_fn, timeout_s=120)
    assert errors == [None] * 2, errors
    for g1, s1, g2, s2 in results:
        assert g1 == g2 and s1 == s2
