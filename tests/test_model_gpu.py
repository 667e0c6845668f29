"""Tiny hybrid model on the GPU path against the fp32 CPU oracle, plus the engine end to end."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _prompt(n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 1023, (n,), generator=g).tolist()


def _near_greedy(tokens, prompt, quant, slack=0.06):
    """Every generated token must be (nearly) the oracle's arg-max given the same history."""
    from tileinfer_b200.models.config import TINY_HYBRID
    from tileinfer_b200.models.reference_cpu import naive_logits
    from tileinfer_b200.models.weights import RandomWeights
    full = list(prompt) + list(tokens)
    lg = naive_logits(TINY_HYBRID, RandomWeights(TINY_HYBRID, 0), full, quant=quant)
    worst = 0.0
    for i, t in enumerate(tokens):
        row = lg[len(prompt) - 1 + i]
        worst = max(worst, float(row.max() - row[t]))
    assert worst <= slack, f"token off the oracle arg-max by {worst}"


@pytest.mark.parametrize("quant", ["bf16", "w8a16"])
def test_forward_logits_match_oracle(quant):
    from tileinfer_b200.models.config import TINY_HYBRID
    from tileinfer_b200.models.hybrid_b200 import B200HybridModel
    from tileinfer_b200.models.reference_cpu import Batch, naive_logits
    from tileinfer_b200.models.weights import RandomWeights
    src = RandomWeights(TINY_HYBRID, 0)
    p = _prompt(45)
    ref = naive_logits(TINY_HYBRID, src, p, quant="w8a16" if quant == "w8a16" else "none")
    m = B200HybridModel(TINY_HYBRID, src, quant=quant)
    m.alloc_cache(16, 16, 3)
    table = [9, 3, 12]
    slots = torch.tensor([table[i // 16] * 16 + i % 16 for i in range(len(p))])
    ids = torch.tensor(p)
    # chunk 1 (32 tokens), chunk 2 (12 tokens), then one decode token: three different code paths
    cuts = [(0, 32), (32, 44), (44, 45)]
    for a, b in cuts:
        h = m.forward(Batch(ids[a:b], torch.arange(a, b), [0, b - a], [b], [table], slots[a:b], [1]))
        lg = m.logits(h)[0].float().cpu()
        err = float((lg - ref[b - 1]).abs().max())
        assert err < 0.05, f"logits error {err} after tokens [{a},{b})"
    assert m.peer_status() == 0


@pytest.mark.parametrize("quant,eager", [("w8a16", False), ("w8a16", True), ("bf16", False)])
def test_engine_gpu_generate(quant, eager):
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    llm = LLM("preset:tiny-hybrid", quantization=quant, enforce_eager=eager, num_kvcache_blocks=128, max_num_seqs=8,
              max_model_len=512, max_prefill_chunk_tokens=32)
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    prompts = [_prompt(17, 1), _prompt(70, 2), _prompt(5, 3)]
    outs = llm.generate_token_ids(prompts, sp)
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        _near_greedy(o, p, quant="w8a16" if quant == "w8a16" else "none")
    if not eager:
        assert llm.model_runner.model.launches_per_decode_step > 0
    # sampling path (top-k candidates on the device, seeded draw on the host)
    sp2 = SamplingParams(temperature=0.8, top_k=20, max_tokens=8, ignore_eos=True)
    o2 = llm.generate_token_ids([prompts[0]], sp2)[0]
    assert len(o2) == 8 and all(0 <= t < 1024 for t in o2)
    # constrained path (full logits on the host)
    sp3 = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True, allowed_token_ids=[5, 6, 7])
    assert set(llm.generate_token_ids([prompts[0]], sp3)[0]) <= {5, 6, 7}


def test_prefix_reuse_and_swap_on_gpu():
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    llm = LLM("preset:tiny-hybrid", quantization="w8a16", num_kvcache_blocks=40, max_num_seqs=4, max_model_len=512,
              prefix_state_stride=16, swap_space_bytes=64 << 20)
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    shared = _prompt(48, 5)
    a = llm.generate_token_ids([shared + _prompt(9, 6)], sp)[0]
    b = llm.generate_token_ids([shared + _prompt(9, 6)], sp)[0]          # full prefix hit
    st = llm.stats()
    assert st["prefix_hits"] >= 1 and st["prefix_hit_tokens"] >= 48
    _near_greedy(b, shared + _prompt(9, 6), "w8a16")
    # memory pressure: 4 sequences x (up to 12 blocks) > 40 blocks -> preemption by swapping
    prompts = [_prompt(150, 10 + i) for i in range(4)]
    outs = llm.generate_token_ids(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    st = llm.stats()
    assert st["preemptions"] >= 1 and st["swaps_out"] >= 1 and st["swaps_in"] >= 1
    for p, o in zip(prompts, outs):
        _near_greedy(o, p, "w8a16")


def test_weight_shard_cache_round_trip(tmp_path):
    """First start writes the rank's weights in kernel layout; the second start loads them (no sharding, no
    quantisation) and generates the same tokens."""
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    kw = dict(quantization="w8a16", num_kvcache_blocks=64, max_num_seqs=4, max_model_len=256,
              weight_cache_dir=str(tmp_path))
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompts = [list(range(5, 40)), [7, 8, 9]]
    a = LLM("preset:tiny-hybrid", **kw).generate_token_ids(prompts, sp)
    files = list(tmp_path.iterdir())
    assert len(files) == 1 and files[0].stat().st_size > 1 << 20
    from tileinfer_b200.models.hybrid_b200 import B200HybridModel

    def boom(self, *args):
        raise AssertionError("the cached shards must be used")
    keep = B200HybridModel._build_shards
    B200HybridModel._build_shards = boom
    try:
        b = LLM("preset:tiny-hybrid", **kw).generate_token_ids(prompts, sp)
    finally:
        B200HybridModel._build_shards = keep
    assert a == b


def test_edited_requests_stay_on_the_device_path_and_match_the_host_sampler():
    """Repetition penalty, logit bias, allow-list and a regex grammar: the device path (logit-edit kernel + top-k +
    sample kernel inside the CUDA graph) must produce the tokens of the host path (full logits to the CPU)."""
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    llm = LLM("preset:tiny-hybrid", quantization="w8a16", num_kvcache_blocks=128, max_num_seqs=8, max_model_len=512)
    model = llm.model_runner.model
    prompts = [_prompt(20, 31), _prompt(33, 32), _prompt(9, 33)]
    params = [SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True, repetition_penalty=1.5),
              SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True, logit_bias={65: 2.0, 66: 1.5},
                             bad_token_ids=[67]),
              SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, guided_regex="[a-c]+")]
    steps0 = model.host_steps
    dev = llm.generate_token_ids(prompts, params)
    assert model.host_steps > steps0
    keep = model.EDIT_SLOTS
    model.EDIT_SLOTS = -1                      # no row qualifies: everything takes the host path
    try:
        host = llm.generate_token_ids(prompts, params)
    finally:
        model.EDIT_SLOTS = keep
    assert dev == host
    text = "".join(chr(t) for t in dev[2])
    assert text and set(text) <= set("abc")
    # sampled requests draw the same tokens on both paths (same seeded uniform numbers, same candidates)
    sp = SamplingParams(temperature=0.9, top_k=40, top_p=0.95, max_tokens=12, ignore_eos=True)
    a = LLM("preset:tiny-hybrid", quantization="w8a16", num_kvcache_blocks=128, max_num_seqs=8, max_model_len=512)
    b = LLM("preset:tiny-hybrid", quantization="w8a16", num_kvcache_blocks=128, max_num_seqs=8, max_model_len=512)
    b.model_runner.model.EDIT_SLOTS = -1
    assert a.generate_token_ids([prompts[0]], sp) == b.generate_token_ids([prompts[0]], sp)


def test_a_set_device_status_word_stops_the_engine():
    """The status word the kernels raise when a bounded wait runs out travels to the host with every step's tokens; a
    non-zero word must stop the step (its tokens are discarded) instead of letting wrong results through."""
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    from tileinfer_b200.parallel.watchdog import PeerLostError
    llm = LLM("preset:tiny-hybrid", quantization="w8a16", num_kvcache_blocks=64, max_num_seqs=4, max_model_len=256)
    prompt = [[5, 9, 200, 31, 77, 8]]
    ok = llm.generate_token_ids(prompt, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert len(ok[0]) == 4
    model = llm.model_runner.model
    model.ctrl[1] = 1                                   # what wait_flag_ge / mbar_wait do on expiry
    with pytest.raises(PeerLostError) as e:
        llm.generate_token_ids(prompt, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert "status word" in str(e.value)
    model.ctrl[1] = 0
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
