"""Writes a random-init HuggingFace Qwen3.5/3.6 text checkpoint + a word-level tokenizer to a directory,
so that the reference engine (which insists on a checkpoint and a tokenizer on disk) can be run offline
on the architecture named by a tileinfer_b200 preset.  Weights are N(0, 0.02) like the presets'."""
from __future__ import annotations

import json
import os
import sys
import time


def make(preset_name: str, out_dir: str, seed: int = 0) -> str:
    import torch
    from transformers.models.qwen3_5 import Qwen3_5ForCausalLM, Qwen3_5TextConfig
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from tileinfer_b200.models.config import get_preset

    done = os.path.join(out_dir, "DONE")
    if os.path.exists(done):
        return out_dir
    os.makedirs(out_dir, exist_ok=True)
    c = get_preset(preset_name)
    cfg = Qwen3_5TextConfig(
        vocab_size=c.vocab_size, hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
        num_hidden_layers=c.num_layers, num_attention_heads=c.num_q_heads, num_key_value_heads=c.num_kv_heads,
        head_dim=c.head_dim, max_position_embeddings=32768, tie_word_embeddings=c.tie_embeddings,
        rms_norm_eps=c.rms_eps, linear_conv_kernel_dim=c.gdn_conv_kernel, linear_key_head_dim=c.gdn_head_k_dim,
        linear_value_head_dim=c.gdn_head_v_dim, linear_num_key_heads=c.gdn_num_k_heads,
        linear_num_value_heads=c.gdn_num_v_heads, layer_types=list(c.layer_types),
        rope_parameters={"rope_theta": c.rope_theta, "partial_rotary_factor": c.rotary_dim / c.head_dim,
                         "rope_type": "default"},
        eos_token_id=c.vocab_size - 1, pad_token_id=c.vocab_size - 1, initializer_range=0.02,
    )
    cfg.architectures = ["Qwen3_5ForCausalLM"]
    torch.manual_seed(seed)
    t0 = time.time()
    with torch.device("cpu"):
        model = Qwen3_5ForCausalLM(cfg).to(torch.bfloat16)
    model.save_pretrained(out_dir, safe_serialization=True, max_shard_size="4GB")
    # word-level tokenizer: token i is the word "t<i>"
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {f"t{i}": i for i in range(c.vocab_size - 1)}
    vocab["<eos>"] = c.vocab_size - 1
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(out_dir, "tokenizer.json"))
    with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "pad_token": "<eos>",
                   "unk_token": "t0"}, f)
    with open(done, "w") as f:
        f.write(f"{preset_name} {time.time() - t0:.1f}s\n")
    return out_dir


if __name__ == "__main__":
    print(make(sys.argv[1], sys.argv[2]))
