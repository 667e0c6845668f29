"""Engine configuration.

Field names and defaults follow the reference's Config dataclass (engine/config.py:11-41).
`model` may be a preset ("preset:tiny-hybrid", "preset:qwen3.6-27b") or a local HuggingFace
directory; presets need neither a checkpoint nor a tokenizer on disk.  Additional fields are new
and all have defaults.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

from ..models.config import ModelConfig, from_hf_config, get_preset, PRESETS


@dataclass
class Config:
    model: str
    # scheduling
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 64
    max_model_len: int = 32768
    # memory
    gpu_memory_utilization: float = 0.9
    kvcache_block_size: int = 16
    num_kvcache_blocks: int = -1
    swap_space_bytes: int = 0
    # execution
    enforce_eager: bool = False
    cuda_graph_max_batch_size: int = 256
    hf_config: object = None
    eos: list = None
    max_prefill_chunk_tokens: int = 4096
    enable_prefix_caching: bool = True
    max_prefix_states: int = 64
    num_scheduler_steps: int = 1
    tp_size: int = 1
    nccl_timeout: float = 600.0
    # ---- additions -------------------------------------------------------
    weights: str = "random:0"          # "random:<seed>" or "hf"
    quantization: str = "w8a16"        # "w8a16" or "bf16"
    device: str = "auto"               # "auto" | "cuda" | "cpu"
    prefix_state_stride: int = 256     # DeltaNet state snapshots at stride * 2^j prompt tokens
    gdn_state_dtype: str = "fp32"      # recurrent-state pool dtype on the GPU: "fp32" | "bf16"
    fused_collectives: bool = True     # peer-memory fused TP kernels (False: NCCL baseline path)
    baseline_full_vocab_gather: bool = False   # sampling baseline: all-gather the whole logit rows (measurement only)
    heartbeat_interval: float = 0.0    # seconds between peer heartbeats under tensor parallelism (0: watchdog off)
    heartbeat_timeout: float = 10.0    # a peer silent for this long is reported lost before the next step
    weight_cache_dir: str = None       # on-disk cache of per-rank quantised shards
    model_config: ModelConfig = None
    tokenizer: str = "auto"            # "auto" | "byte" | local path

    def __post_init__(self):
        if self.model_config is None:
            name = self.model
            if name.startswith("preset:") or name in PRESETS:
                self.model_config = get_preset(name)
            elif os.path.isdir(name):
                from transformers import AutoConfig
                self.hf_config = AutoConfig.from_pretrained(name, trust_remote_code=False)
                self.model_config = from_hf_config(self.hf_config)
                if self.weights.startswith("random") and os.path.exists(os.path.join(name, "config.json")) \
                        and any(f.endswith(".safetensors") for f in os.listdir(name)):
                    self.weights = "hf"
            else:
                raise ValueError(f"model {name!r} is neither a preset ({sorted(PRESETS)}) nor a local directory")
        mc = self.model_config
        self.max_model_len = min(self.max_model_len, mc.max_position_embeddings)
        if self.eos is None:
            self.eos = list(mc.eos_token_ids)
        if self.device == "auto":
            import torch
            self.device = "cuda" if torch.cuda.is_available() else "cpu"
        if self.kvcache_block_size != 16 and self.device == "cuda":
            raise ValueError("the sm_100a attention kernels use 16-token KV pages")
        if self.max_prefill_chunk_tokens % self.kvcache_block_size:
            raise ValueError("max_prefill_chunk_tokens must be a multiple of kvcache_block_size")
        if self.prefix_state_stride % self.kvcache_block_size:
            raise ValueError("prefix_state_stride must be a multiple of kvcache_block_size")
        if self.quantization not in ("w8a16", "bf16"):
            raise ValueError(f"quantization must be w8a16 or bf16, got {self.quantization}")
        mc.validate_tp(self.tp_size)
