"""Rank 0's share of a tensor-parallel model on ONE GPU with collectives that do nothing: every kernel of the prefill and
decode paths runs with the per-rank shapes of TP = 4 and TP = 8 (27B architecture, 8 layers: 2060-column DeltaNet
projections whose rows are not 16-byte multiples, 3 query heads on one replicated KV head, 6 DeltaNet heads, k = 768 / 2176
products) and of the tiny test model.  The numbers mean nothing (the partial sums are never added up); what is checked is
that every launch accepts the shapes, nothing faults and the activations stay finite."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(preset, tp, prefill_lens, batches):
    from tileinfer_b200.models.config import get_preset
    from tileinfer_b200.models.hybrid_b200 import B200HybridModel
    from tileinfer_b200.models.reference_cpu import Batch
    from tileinfer_b200.models.weights import RandomWeights
    from tileinfer_b200.parallel.comm import SingleComm

    class NoopComm(SingleComm):
        world_size = tp

    cfg = get_preset(preset)
    conf = types.SimpleNamespace(gdn_state_dtype="fp32", fused_collectives=False, max_num_batched_tokens=4096, max_num_seqs=64)
    m = B200HybridModel(cfg, RandomWeights(cfg, 0, device="cuda"), quant="w8a16", tp=tp, rank=0, comm=NoopComm(), config=conf)
    for T in prefill_lens:
        nblk = T // 16 + 2
        m.alloc_cache(nblk + 1, 16, 2)
        batch = Batch(torch.randint(0, cfg.vocab_size - 1, (T,)), torch.arange(T), [0, T], [T], [list(range(nblk))],
                      torch.arange(T), [0])
        h = m.forward(batch)
        torch.cuda.synchronize()
        assert bool(torch.isfinite(h.float()).all()), (preset, tp, T)
    for B in batches:
        ctx = 256
        nb = ctx // 16 + 2
        m.alloc_cache(B * nb + 1, 16, B + 1)
        m.release_graphs()
        m.capture_decode_graphs(B, B, ctx + 16, B)
        tables = [list(range(s * nb, (s + 1) * nb)) for s in range(B)]
        pos = ctx - 1
        batch = Batch(torch.randint(0, cfg.vocab_size - 1, (B,)), torch.full((B,), pos), list(range(B + 1)), [pos + 1] * B,
                      tables, torch.tensor([t[pos // 16] * 16 + pos % 16 for t in tables]), list(range(B)))
        m._decode_graph_step(batch, 1)
        torch.cuda.synchronize()
    m.release_graphs()
    assert float(torch.ones(4, device="cuda").sum()) == 4.0          # the context is alive


@pytest.mark.parametrize("tp", [4, 8])
def test_27b_shard_shapes(tp):
    _run("preset:qwen3.6-27b-8l", tp, (128, 2048, 40, 7), (1, 8, 64))


@pytest.mark.parametrize("preset,tp", [("preset:tiny-hybrid-tp", 4), ("preset:tiny-hybrid-tp", 2), ("preset:tiny-hybrid-tp8", 8)])
def test_tiny_shard_shapes(preset, tp):
    _run(preset, tp, (70, 21, 5), (1, 8))
