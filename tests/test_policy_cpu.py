"""Scheduling, paged-KV accounting, swapping, prefix reuse, fault injection: no GPU involved."""
import pytest
import torch

from tileinfer_b200.engine.block_manager import BlockManager
from tileinfer_b200.engine.llm import LLM
from tileinfer_b200.engine.model_runner import SimulatedOOM
from tileinfer_b200.engine.prefix_cache import PrefixCache
from tileinfer_b200.engine.sampling_params import SamplingParams
from tileinfer_b200.engine.sequence import Sequence, SequenceStatus


def _prompt(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 1023, (n,), generator=g).tolist()


def _llm(**kw):
    base = dict(device="cpu", quantization="bf16", num_kvcache_blocks=64, max_num_seqs=4, max_model_len=512)
    base.update(kw)
    return LLM("preset:tiny-hybrid", **base)


def test_block_manager_refcounts_and_swap():
    bm = BlockManager(8, 16, num_cpu_blocks=4)
    Sequence.block_size = 16
    a = Sequence(list(range(40)))
    bm.allocate(a)
    assert len(a.block_table) == 3 and bm.num_free_blocks == 5
    b = Sequence(list(range(40)))
    bm.share_blocks(b, a.block_table[:2])
    bm.allocate_extra(b)
    assert bm.ref_count[a.block_table[0]] == 2 and bm.num_free_blocks == 4
    assert bm.can_swap_out(a)
    dev, host = bm.swap_out(a)
    assert len(host) == 3 and a.block_table == [] and len(bm.free_cpu_block_ids) == 1
    assert bm.ref_count[dev[0]] == 1 and bm.ref_count[dev[2]] == 0          # shared blocks survive
    assert bm.can_swap_in(a)
    host2, dev2 = bm.swap_in(a)
    assert host2 == host and len(dev2) == 3 and len(bm.free_cpu_block_ids) == 4
    bm.deallocate(a)
    bm.deallocate(b)
    assert bm.num_free_blocks == 8 and all(r == 0 for r in bm.ref_count)


def test_prefix_cache_needs_state_and_evicts_lru():
    bm = BlockManager(8, 4)
    pc = PrefixCache(4, bm)
    toks = list(range(20))
    blocks = [bm._take() for _ in range(4)]
    chain = pc.insert(toks, blocks, 4)
    assert [n.depth for n in chain] == [1, 2, 3, 4] and all(bm.ref_count[b] == 2 for b in blocks)
    assert pc.find_longest_prefix(toks) == ([], 0)                 # KV alone is not reusable
    pc.mark_state(chain[1].node_id)
    nodes, n = pc.find_longest_prefix(toks)
    assert n == 8 and [x.block_id for x in nodes] == blocks[:2]
    nodes, n = pc.find_longest_prefix(toks[:8])                    # never the whole prompt
    assert n == 4 or n == 0
    for b in blocks:
        bm.decref(b)                                               # the producing sequence is gone
    assert pc.num_evictable() == 4
    dropped = []
    pc.on_node_evicted = dropped.append
    assert pc.evict(2) == 2 and len(pc) == 2 and bm.num_free_blocks == 6
    assert dropped == [chain[3].node_id, chain[2].node_id]          # leaves first


def test_chunked_mixed_batches_match_unchunked():
    prompts = [_prompt(70, 1), _prompt(9, 2), _prompt(33, 3)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    ref = _llm(max_prefill_chunk_tokens=4096).generate_token_ids(prompts, sp)
    llm = _llm(max_prefill_chunk_tokens=16, max_num_batched_tokens=24)
    got = llm.generate_token_ids(prompts, sp)
    assert got == ref
    assert llm.stats()["steps"] > 10          # really ran in many mixed steps


def test_prefix_reuse_gives_identical_tokens_and_skips_compute():
    shared = _prompt(64, 7)
    p1, p2 = shared + _prompt(10, 8), shared + _prompt(12, 9)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    cold = _llm(enable_prefix_caching=False)
    want = cold.generate_token_ids([p1], sp) + cold.generate_token_ids([p2], sp)
    llm = _llm(prefix_state_stride=32)
    got1 = llm.generate_token_ids([p1], sp)
    before = llm.stats()["prefill_tokens"]
    got2 = llm.generate_token_ids([p2], sp)
    st = llm.stats()
    assert got1 + got2 == want
    assert st["prefix_hits"] == 1 and st["prefix_hit_tokens"] == 64
    assert st["prefill_tokens"] - before == len(p2) - 64
    # same prompt again: everything but the tail is reused, and at least one token is computed
    got3 = llm.generate_token_ids([p2], sp)
    assert got3 == got2 and llm.stats()["prefix_hit_tokens"] >= 64 + 64


def test_prefix_state_survives_until_the_hit_sequence_runs():
    """A sequence that was admitted with a prefix hit may run its first chunk steps later; the snapshot it
    needs must not be evicted by the snapshots other sequences save in between (tiny snapshot LRU)."""
    shared = _prompt(64, 70)
    prompts = [shared + _prompt(40 + 3 * i, 71 + i) for i in range(10)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = _llm(enable_prefix_caching=False, num_kvcache_blocks=256, max_num_seqs=8).generate_token_ids(prompts, sp)
    llm = _llm(prefix_state_stride=16, max_prefix_states=2, num_kvcache_blocks=256, max_num_seqs=8,
               max_prefill_chunk_tokens=32, max_num_batched_tokens=40)
    first = llm.generate_token_ids(prompts[:1], sp)
    rest = llm.generate_token_ids(prompts[1:], sp)
    assert first + rest == want
    assert llm.stats()["prefix_hits"] >= 1 and not llm.model_runner.pinned_prefix_states


def test_swap_preemption_preserves_outputs():
    prompts = [_prompt(60, 20 + i) for i in range(4)]
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    want = _llm(num_kvcache_blocks=64, enable_prefix_caching=False).generate_token_ids(prompts, sp)
    llm = _llm(num_kvcache_blocks=20, swap_space_bytes=1 << 24, enable_prefix_caching=False)
    got = llm.generate_token_ids(prompts, sp)
    st = llm.stats()
    assert got == want
    assert st["swaps_out"] >= 1 and st["swaps_in"] == st["swaps_out"] and st["recomputes"] == 0


def test_recompute_preemption_when_no_swap_space():
    prompts = [_prompt(60, 30 + i) for i in range(4)]
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    want = _llm(num_kvcache_blocks=64, enable_prefix_caching=False).generate_token_ids(prompts, sp)
    llm = _llm(num_kvcache_blocks=20, swap_space_bytes=0, enable_prefix_caching=False)
    got = llm.generate_token_ids(prompts, sp)
    assert got == want and llm.stats()["recomputes"] >= 1


def test_multi_step_scheduling_same_tokens():
    prompts = [_prompt(20, 40), _prompt(7, 41)]
    sp = SamplingParams(temperature=0.0, max_tokens=13, ignore_eos=True)
    assert _llm(num_scheduler_steps=4).generate_token_ids(prompts, sp) == _llm().generate_token_ids(prompts, sp)


def test_oom_injection_drops_last_sequence_and_recovers():
    llm = _llm(enable_prefix_caching=False)
    prompts = [_prompt(20, 50 + i) for i in range(3)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = _llm(enable_prefix_caching=False).generate_token_ids(prompts, sp)
    calls = {"n": 0}

    def hook(seqs):
        calls["n"] += 1
        if calls["n"] == 3 and len(seqs) > 1:
            raise SimulatedOOM("injected")
    llm.model_runner.fault_hook = hook
    got = llm.generate_token_ids(prompts, sp)
    assert got == want and llm.stats()["oom_retries"] == 1

    def always(seqs):
        raise SimulatedOOM("injected")
    llm.model_runner.fault_hook = always
    with pytest.raises(RuntimeError, match="out of memory"):
        llm.generate_token_ids([prompts[0]], sp)
    llm.model_runner.fault_hook = None
    assert llm.scheduler.is_finished() and llm.scheduler.block_manager.num_free_blocks == 64   # nothing leaked
    assert llm.generate_token_ids([prompts[0]], sp) == [want[0]]


def test_finish_reasons_stop_strings_and_validation():
    llm = _llm()
    out = llm.generate(["ab"], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))[0]
    assert out["finish_reason"] == "length" and len(out["token_ids"]) == 3
    # force EOS through the bias: finishes with "stop" after one token
    eos = llm.tokenizer.eos_token_id
    out = llm.generate(["ab"], SamplingParams(temperature=0.0, max_tokens=9, logit_bias={eos: 1e4}))[0]
    assert out["finish_reason"] == "stop" and out["token_ids"] == [eos]
    # stop string: bias towards 'x' then stop on "xx"
    out = llm.generate(["ab"], SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True,
                                              logit_bias={ord("x"): 1e4}, stop=["xx"]))[0]
    assert out["text"] == "xx" and out["finish_reason"] == "stop"
    with pytest.raises(ValueError):
        llm.add_request([5] * 600)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    assert llm.scheduler.is_finished()


def test_sampling_is_seeded_and_respects_top_k():
    sp = SamplingParams(temperature=1.0, top_k=3, max_tokens=12, ignore_eos=True)
    a = _llm().generate_token_ids([_prompt(9, 60)], sp)
    b = _llm().generate_token_ids([_prompt(9, 60)], sp)
    assert a == b
    greedy = _llm().generate_token_ids([_prompt(9, 60)], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    assert a != greedy or True      # usually differs; never an error
    seq_status = SequenceStatus.FINISHED
    assert seq_status.name == "FINISHED"


def test_gemv_planner_choices():
    """Host-side planning of the decode GEMV (pure Python): ring depth that fits beside the staged activations,
    team size for products with few row tiles, rows per launch."""
    from tileinfer_b200.ops import functional as F
    # 27B layer shapes, one row: (row tiles, k tiles)
    assert F.plan_team(4352, 80, 1) == 1          # gate_up: more units than warps -> warp-owned units
    assert F.plan_team(2060, 80, 1) == 1          # in_proj: 0.87 units per warp is enough
    assert F.plan_team(640, 272, 1) == 3          # down: few row tiles -> three warps share a unit (five teams per CTA)
    assert F.plan_team(640, 96, 1) == 3           # out_proj
    assert F.plan_team(544, 80, 1) == 4 and F.plan_team(258, 80, 1) == 8      # 1/8 tensor-parallel shards
    assert F.plan_team(640, 12, 1) == 1           # k too short to share
    assert F.plan_team(640, 272, 1, team=1) == 1
    R, tps, stages = F.plan_gemv(F.W_INT8, F.XNORM, 1, 4352, 80)
    assert (R, tps) == (1, 8) and stages == 3
    assert F.plan_gemv(F.W_INT8, F.XGLOBAL, 1, 640, 272)[2] == 2              # K = 17408: x takes 37 KB
    assert F.plan_gemv(F.W_INT8, F.XNORM, 16, 4352, 80) is None               # 16 rows of K = 5120 do not fit
    assert F.max_rows(F.W_INT8, F.XNORM, 5120) == 12 and F.max_rows(F.W_INT8, F.XGLOBAL, 17408) == 4
    for m in (1, 4, 12):
        xb = F.x_smem_bytes(F.W_INT8, F.XNORM, m, 5120, 5120)
        _, tps, st = F.plan_gemv(F.W_INT8, F.XNORM, m, 4352, 80)
        assert xb + F.GEMV_WARPS * (st * (tps * 512 + 8) + 64) <= F.SMEM_LIMIT


def test_prefix_hit_under_memory_pressure_does_not_crash():
    """6 KV blocks: 4 hold a cached prefix (cache-only references), 2 belong to a running sequence.  A new request
    that matches the cached prefix needs one more block than exist once the prefix blocks are pinned by the hit:
    the request must stay in the waiting queue (or fall back to eviction), never raise from the allocator."""
    from tileinfer_b200.engine.config import Config
    from tileinfer_b200.engine.scheduler import Scheduler
    cfg = Config("preset:tiny-hybrid", device="cpu", num_kvcache_blocks=6, max_num_seqs=4, max_model_len=512)
    Sequence.block_size = 16
    sch = Scheduler(cfg)
    bm, pc = sch.block_manager, sch.prefix_cache
    shared = _prompt(64, 90)
    blocks = [bm._take() for _ in range(4)]
    chain = pc.insert(shared, blocks, 4)
    pc.mark_state(chain[-1].node_id)
    for b in blocks:
        bm.decref(b)                                   # the producer is gone: cache-only references
    running = Sequence(_prompt(30, 91))
    bm.allocate(running)                               # the two remaining free blocks
    assert bm.num_free_blocks == 0 and pc.num_evictable() == 4
    new = Sequence(shared + _prompt(40, 92))           # 104 tokens = 7 blocks: 4 shared + 3 more, none free
    ok = sch._allocate_blocks_for_new_seq(new)         # used to raise RuntimeError('out of KV blocks')
    assert ok is False and new.block_table == []
    assert all(bm.ref_count[b] == 1 for b in blocks)   # references given back, cache entries intact
    assert pc.num_evictable() == 4
    # a request that fits after evicting part of the cached prefix still gets blocks
    small = Sequence(shared[:32] + _prompt(8, 93))     # 40 tokens = 3 blocks
    assert sch._allocate_blocks_for_new_seq(small) and len(small.block_table) == 3


def test_gdn_chunk_table_cuts_at_64_tokens_and_at_snapshot_points():
    """Host side of the chunk-parallel DeltaNet prefill: chunks of at most 64 tokens that never straddle a snapshot
    point; the snapshot entry rides on the chunk that ends there."""
    from tileinfer_b200.ops import functional as F
    ck, seq_ck = F.gdn_chunk_table([0, 1, 8, 208, 272])                       # lengths 1, 7, 200, 64; no snapshots
    assert seq_ck.tolist() == [0, 1, 2, 6, 7]
    assert ck[2].tolist() == [1, 7, 64, 64, 64, 8, 64] and ck[1].tolist() == [0, 1, 8, 72, 136, 200, 208]
    assert ck[0].tolist() == [0, 1, 2, 2, 2, 2, 3] and set(ck[3].tolist()) == {-1}
    # snapshots after 48 and 192 tokens of a 200-token sequence (entries 5 and 9), after 64 of a 64-token one (entry 2)
    ck, seq_ck = F.gdn_chunk_table([0, 200, 264], [[48, 192], [64]], [[5, 9], [2]])
    lens, snaps = ck[2].tolist(), ck[3].tolist()
    assert sum(lens[:seq_ck[1]]) == 200 and max(lens) <= 64
    ends = [int(ck[1][i]) + lens[i] for i in range(seq_ck[1])]
    assert 48 in ends and 192 in ends
    assert snaps[ends.index(48)] == 5 and snaps[ends.index(192)] == 9 and snaps[-1] == 2
    assert [s for s in snaps if s >= 0] == [5, 9, 2]
    # a point past the end of the step's tokens is ignored
    ck, _ = F.gdn_chunk_table([0, 30], [[16, 40]], [[1, 7]])
    assert ck[2].tolist() == [16, 14] and ck[3].tolist() == [1, -1]


def test_device_sampling_spec_draws_like_the_host_sampler():
    """What the device sampler is fed is built on the host: the uniform numbers come from the shared generator in row
    order and only for rows that sample; an edited row carries the additive row its constraint makes of zeros and the
    sorted ids that get the repetition penalty (rank-local)."""
    from tileinfer_b200.engine.constraints import make_constraint
    from tileinfer_b200.engine.sampler import Sampler
    from tileinfer_b200.parallel.comm import SingleComm

    def seqs():
        out = []
        for sp, toks in ((SamplingParams(temperature=0.0), [3, 4]), (SamplingParams(temperature=0.7, top_k=20), [9, 9, 5]),
                         (SamplingParams(temperature=0.8, top_k=1), [1]),
                         (SamplingParams(temperature=0.5, repetition_penalty=1.3, bad_token_ids=[7]), [40, 2, 40, 130])):
            s = Sequence(list(toks), sp)
            s.constraint = make_constraint(sp, None)                 # what LLMEngine.add_request does
            out.append(s)
        return out
    a, b = Sampler(SingleComm(), 32, (127,), seed=11), Sampler(SingleComm(), 32, (127,), seed=11)
    a._v_local = b._v_local = 96                                     # this rank owns token ids 32..127
    ss = seqs()
    spec = a.device_spec(ss, edit_rows=[3])
    want = torch.rand(2, 1, generator=b.gen)                         # rows 1 and 3 sample; rows 0 (greedy) and 2 (top-k 1) do not
    assert spec["u"][0] == 0.0 and spec["u"][2] == 0.0
    assert spec["u"][1] == float(want[0, 0]) and spec["u"][3] == float(want[1, 0])
    assert spec["temperature"] == [0.0, 0.7, 0.8, 0.5] and spec["top_k"][1] == 20
    (row, add, pen, rp), = spec["edits"]
    assert row == 3 and rp == 1.3
    assert pen.tolist() == [8]                                       # ids 40 -> local 8; 2 belongs to another rank, 130 - 32 = 98 is past this shard
    assert add is not None and add.shape == (96,) and float(add.max()) == 0.0 and int(torch.isinf(add).sum()) == 0    # bad id 7 is another rank's
    # the same request on the rank that owns token 7: its additive row masks it
    c = Sampler(SingleComm(), 0, (127,), seed=11)
    c._v_local = 32
    (_, add0, pen0, _), = c.device_spec(seqs(), edit_rows=[3])["edits"]
    assert float(add0[7]) == float("-inf") and int(torch.isinf(add0).sum()) == 1 and pen0.tolist() == [2]


def test_all_reduce_flags_are_rebased_behind_the_next_tags():
    """The many-row all-reduce waits for 'flag >= tag' modulo 2^32.  A flag left by a collective long ago would look ahead
    of the next tags once the step counter has advanced by more than 2^15; the periodic scrub therefore rewrites every
    flag to step * 65536, which no tag of this or a later step counts as reached, across the 32-bit wrap too."""
    from tileinfer_b200.parallel.symm_mem import flag_rebase_value

    def ready(flag, want):                                  # wait_flag_ge in ops/csrc/common.cuh
        d = (flag - want) & 0xFFFFFFFF
        return d < (1 << 31)

    def tag(step, order):
        return (step * 65536 + order + 1) & 0xFFFFFFFF

    stale = tag(10, 3)
    assert ready(stale, tag(10, 3)) and not ready(stale, tag(11, 0))
    assert ready(stale, tag(10 + 40000, 0))                 # the hazard: 40000 steps later the old flag passes for a fresh one
    for step in (0, 7, 32767, 32768, 40010, 65535, 65536, 65537, 2 ** 20 + 5):
        base = flag_rebase_value(step) & 0xFFFFFFFF
        assert -(1 << 31) <= flag_rebase_value(step) < (1 << 31)
        for later in (0, 1, 100, 32767):                    # until the next scrub, at most 2^15 steps away
            for order in (0, 1, 200, 65534):
                assert not ready(base, tag(step + later, order)), (step, later, order)
        assert ready(tag(step, 5), tag(step, 5)) and ready(tag(step + 1, 0), tag(step, 5))
