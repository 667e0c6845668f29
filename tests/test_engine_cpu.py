"""Tiny hybrid model on CPU: the paged, chunked, mixed-batch engine must reproduce the cache-free
oracle (logits and greedy tokens)."""
import torch

from tileinfer_b200.engine.llm import LLM
from tileinfer_b200.engine.sampling_params import SamplingParams
from tileinfer_b200.models.config import TINY_HYBRID
from tileinfer_b200.models.reference_cpu import Batch, TorchHybridModel, gdn_chunked, gdn_recurrent, naive_logits
from tileinfer_b200.models.weights import RandomWeights


def _prompts():
    g = torch.Generator().manual_seed(1)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (17, 33)]


def _oracle_greedy(prompt, n, quant="none"):
    src = RandomWeights(TINY_HYBRID, 0)
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(naive_logits(TINY_HYBRID, src, toks, quant=quant)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out


def test_chunked_delta_rule_equals_recurrent():
    torch.manual_seed(0)
    T, H, D = 100, 3, 16
    q, v = torch.randn(T, H, D), torch.randn(T, H, D)
    k = torch.nn.functional.normalize(torch.randn(T, H, D), dim=-1)
    g, b, S = -torch.rand(T, H), torch.rand(T, H), torch.randn(H, D, D) * 0.1
    o1, s1 = gdn_recurrent(q, k, v, g, b, S)
    o2, s2 = gdn_chunked(q, k, v, g, b, S, chunk=32)
    assert torch.allclose(o1, o2, atol=1e-4) and torch.allclose(s1, s2, atol=1e-4)


def test_engine_matches_oracle_tokens():
    llm = LLM("preset:tiny-hybrid", device="cpu", quantization="bf16", num_kvcache_blocks=64,
              max_num_seqs=4, max_prefill_chunk_tokens=16)
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    prompts = _prompts()
    got = llm.generate_token_ids(prompts, sp)
    for p, o in zip(prompts, got):
        assert o == _oracle_greedy(p, 16)


def test_paged_logits_match_oracle_logits():
    src = RandomWeights(TINY_HYBRID, 0)
    p = _prompts()[1]
    ref = naive_logits(TINY_HYBRID, src, p)
    m = TorchHybridModel(TINY_HYBRID, src)
    m.alloc_cache(8, 16, 2)
    # prefill in two chunks with scattered blocks, then check the last-token logits
    table = [5, 2, 7]
    slots = torch.tensor([table[i // 16] * 16 + i % 16 for i in range(len(p))])
    ids = torch.tensor(p)
    h = m.forward(Batch(ids[:16], torch.arange(16), [0, 16], [16], [table], slots[:16], [1]))
    assert torch.allclose(m.logits(h)[0], ref[15], atol=2e-4)
    h = m.forward(Batch(ids[16:], torch.arange(16, len(p)), [0, len(p) - 16], [len(p)], [table], slots[16:], [1]))
    assert torch.allclose(m.logits(h)[0], ref[-1], atol=2e-4)


def test_w8a16_engine_matches_quantised_oracle():
    llm = LLM("preset:tiny-hybrid", device="cpu", quantization="w8a16", num_kvcache_blocks=64, max_num_seqs=4)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    p = _prompts()[0]
    assert llm.generate_token_ids([p], sp)[0] == _oracle_greedy(p, 6, quant="w8a16")


def test_generate_and_stream_api():
    llm = LLM("preset:tiny-hybrid", device="cpu", num_kvcache_blocks=64, max_num_seqs=4)
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    out = llm.generate(["hello", "abc"], sp)
    assert [set(o) >= {"text", "prompt", "token_ids", "prompt_token_ids"} for o in out] == [True, True]
    assert out[0]["prompt"] == "hello" and len(out[0]["token_ids"]) == 5 and out[0]["finish_reason"] == "length"
    events = list(llm.generate_stream(["hello"], sp))
    assert [e[0] for e in events] == [0] * 5 and [e[2] for e in events] == [False] * 4 + [True]
    assert llm.stats()["finished_requests"] == 3


def test_close_is_idempotent_and_cli_runs_through_it(capsys):
    """`LLMEngine.close()` (graphs, peer buffers, own process group) is safe on the CPU executor and when called twice;
    the command-line entry point ends with it."""
    from tileinfer_b200.engine.llm import LLM
    llm = LLM("preset:tiny-hybrid", device="cpu", num_kvcache_blocks=32, max_num_seqs=2, max_model_len=128)
    llm.close()
    llm.close()
    import run_engine
    out = run_engine.main(["--model", "preset:tiny-hybrid", "--device", "cpu", "--prompt", "hi", "--max-tokens", "3",
                           "--temperature", "0"])
    assert isinstance(out["text"], str)


def test_optimisation_benchmark_runs_on_the_cpu_executor():
    """`benchmarks/bench_optimizations.py` (one process per variant, public API only) produces its JSON rows."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "benchmarks", "bench_optimizations.py"), "--model", "preset:tiny-hybrid",
                        "--device", "cpu", "--quick"], capture_output=True, text=True, timeout=600, cwd=root)
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0 and len(rows) == 2, (r.stdout[-500:], r.stderr[-1500:])
    assert all("error" not in x and x["decode_tok_s"] > 0 and x["prefill_tok_s"] > 0 for x in rows)
    assert rows[0]["variant"] == "default" and rows[0]["decode_vs_default"] == 1.0
