"""The fp32 oracle and the checkpoint reader against the upstream HuggingFace model.

`naive_logits` is the oracle every kernel and engine test is measured against, and `HFWeights` is how a real
checkpoint reaches the engine; neither is exercised against upstream anywhere else.  A random-init
`Qwen3_5ForCausalLM` of the tiny hybrid architecture is written to disk, read back through `HFWeights`, and the
oracle's logits must agree with the HuggingFace forward on the same tokens; then the engine itself generates from
that directory (`weights="hf"`, tokenizer from disk)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

qwen = pytest.importorskip("transformers.models.qwen3_5")


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    from baseline.make_checkpoint import make
    return make("tiny-hybrid", str(tmp_path_factory.mktemp("hf") / "tiny"))


def test_oracle_logits_match_huggingface(ckpt):
    from transformers import AutoConfig
    from tileinfer_b200.models.config import from_hf_config
    from tileinfer_b200.models.reference_cpu import naive_logits
    from tileinfer_b200.models.weights import HFWeights
    cfg = from_hf_config(AutoConfig.from_pretrained(ckpt))
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size - 1, (45,), generator=g).tolist()
    ours = naive_logits(cfg, HFWeights(cfg, ckpt), ids, quant="none")
    hf = qwen.Qwen3_5ForCausalLM.from_pretrained(ckpt, torch_dtype=torch.float32).eval()
    with torch.no_grad():
        ref = hf(torch.tensor([ids])).logits[0].float()
    assert ours.shape == ref.shape
    assert float((ours - ref).abs().max()) < 1e-4
    assert torch.equal(ours.argmax(-1), ref.argmax(-1))


def test_engine_generates_from_hf_directory(ckpt):
    from tileinfer_b200.engine.llm import LLM
    from tileinfer_b200.engine.sampling_params import SamplingParams
    from tileinfer_b200.models.reference_cpu import naive_logits
    from tileinfer_b200.models.weights import HFWeights
    llm = LLM(ckpt, device="cpu", quantization="bf16", num_kvcache_blocks=32, max_num_seqs=2, max_model_len=128)
    assert llm.config.weights == "hf"
    prompt = [3, 14, 15, 92, 65, 35, 89, 79]
    out = llm.generate_token_ids([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0]
    lg = naive_logits(llm.config.model_config, HFWeights(llm.config.model_config, ckpt), prompt + out, quant="none")
    for i, t in enumerate(out):
        row = lg[len(prompt) - 1 + i]
        assert float(row.max() - row[t]) < 1e-3
    text = llm.generate(["t5 t6 t7"], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))[0]
    assert len(text["token_ids"]) == 3 and text["prompt_token_ids"] == [5, 6, 7]
