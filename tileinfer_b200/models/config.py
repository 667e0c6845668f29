"""Architecture description of the hybrid (gated-DeltaNet + GQA) decoder and its presets.

The reference reads these numbers from a HuggingFace config at start-up and keeps
27B fallbacks in code (reference: engine/model_runner.py:57-100, model/qwen_36.py:23-49).
Here they are explicit presets, so no checkpoint or hub access is needed to build a
model of the named architecture.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace


@dataclass(frozen=True)
class ModelConfig:
    name: str
    vocab_size: int
    hidden_size: int
    num_layers: int
    # "linear_attention" (gated DeltaNet) or "full_attention" (GQA) per layer
    layer_types: tuple
    intermediate_size: int
    # GQA attention
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    rotary_dim: int
    rope_theta: float
    # gated DeltaNet
    gdn_num_k_heads: int
    gdn_num_v_heads: int
    gdn_head_k_dim: int
    gdn_head_v_dim: int
    gdn_conv_kernel: int = 4
    rms_eps: float = 1e-6
    tie_embeddings: bool = False
    eos_token_ids: tuple = ()
    max_position_embeddings: int = 262144

    # ---- derived sizes -------------------------------------------------
    @property
    def gdn_key_dim(self) -> int:
        return self.gdn_num_k_heads * self.gdn_head_k_dim

    @property
    def gdn_value_dim(self) -> int:
        return self.gdn_num_v_heads * self.gdn_head_v_dim

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_key_dim + self.gdn_value_dim

    @property
    def num_gdn_layers(self) -> int:
        return sum(t == "linear_attention" for t in self.layer_types)

    @property
    def num_attn_layers(self) -> int:
        return self.num_layers - self.num_gdn_layers

    def is_gdn(self, layer: int) -> bool:
        return self.layer_types[layer] == "linear_attention"

    def validate_tp(self, tp: int) -> None:
        """TP must divide every sharded dimension except the KV heads.

        The reference rejects tp_size > num_kv_heads (engine/config.py:60-82). Here
        KV heads are replicated instead, so tp=8 works with 4 KV heads as long as
        num_kv_heads divides tp or tp divides num_kv_heads.
        """
        if tp <= 1:
            return
        dims = {
            "num_q_heads": self.num_q_heads,
            "gdn_num_k_heads": self.gdn_num_k_heads,
            "gdn_num_v_heads": self.gdn_num_v_heads,
            "intermediate_size": self.intermediate_size,
        }
        for k, v in dims.items():
            if v % tp:
                raise ValueError(f"tp_size={tp} does not divide {k}={v} ({dims})")
        kv = self.num_kv_heads
        if kv % tp and tp % kv:
            raise ValueError(f"tp_size={tp} and num_kv_heads={kv}: neither divides the other")
        if (self.num_q_heads // tp) > 0 and kv < tp:
            # replicated KV: every rank's q heads must map to ONE kv head
            group = self.num_q_heads // kv
            if group % (self.num_q_heads // tp):
                raise ValueError("q heads of one rank would span two kv heads")

    def kv_heads_per_rank(self, tp: int) -> int:
        return max(1, self.num_kv_heads // tp)

    def kv_head_start(self, tp: int, rank: int) -> int:
        """First (global) KV head served by `rank`; replicated when tp > num_kv_heads."""
        if tp <= self.num_kv_heads:
            return rank * (self.num_kv_heads // tp)
        return rank * self.num_kv_heads // tp


def _pattern(n: int) -> tuple:
    return tuple("full_attention" if (i % 4) == 3 else "linear_attention" for i in range(n))


TINY_HYBRID = ModelConfig(
    name="tiny-hybrid",
    vocab_size=1024,
    hidden_size=384,
    num_layers=4,
    layer_types=_pattern(4),
    intermediate_size=1024,
    num_q_heads=6,
    num_kv_heads=1,
    head_dim=64,
    rotary_dim=16,
    rope_theta=1e7,
    gdn_num_k_heads=4,
    gdn_num_v_heads=8,
    gdn_head_k_dim=64,
    gdn_head_v_dim=64,
    tie_embeddings=True,
    eos_token_ids=(1023,),
    max_position_embeddings=32768,
)

# A TP-friendly small model (2 KV heads, 4/8 DeltaNet heads) used by multi-rank tests.
TINY_HYBRID_TP = replace(
    TINY_HYBRID,
    name="tiny-hybrid-tp",
    num_q_heads=8,
    num_kv_heads=2,
    hidden_size=512,
)

# every head count divisible by 8 (except the 2 KV heads, which are then replicated): the 8-rank tests
TINY_HYBRID_TP8 = replace(
    TINY_HYBRID_TP,
    name="tiny-hybrid-tp8",
    gdn_num_k_heads=8,
    gdn_num_v_heads=16,
)

QWEN36_27B = ModelConfig(
    name="qwen3.6-27b",
    vocab_size=248320,
    hidden_size=5120,
    num_layers=64,
    layer_types=_pattern(64),
    intermediate_size=17408,
    num_q_heads=24,
    num_kv_heads=4,
    head_dim=256,
    rotary_dim=64,
    rope_theta=1e7,
    gdn_num_k_heads=16,
    gdn_num_v_heads=48,
    gdn_head_k_dim=128,
    gdn_head_v_dim=128,
    tie_embeddings=False,
    eos_token_ids=(248046, 248044),
    max_position_embeddings=262144,
)

# The 27B layer shapes with only 8 layers: used to test full-size kernels quickly.
QWEN36_27B_8L = replace(QWEN36_27B, name="qwen3.6-27b-8l", num_layers=8, layer_types=_pattern(8))

PRESETS = {c.name: c for c in (TINY_HYBRID, TINY_HYBRID_TP, TINY_HYBRID_TP8, QWEN36_27B, QWEN36_27B_8L)}


def get_preset(name: str) -> ModelConfig:
    key = name.split(":", 1)[1] if name.startswith("preset:") else name
    if key not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return PRESETS[key]


def from_hf_config(hf) -> ModelConfig:
    """Build a ModelConfig from a HuggingFace Qwen3.5/3.6 text config object."""
    hf = getattr(hf, "text_config", hf)
    n = hf.num_hidden_layers
    lt = tuple(getattr(hf, "layer_types", None) or _pattern(n))
    head_dim = getattr(hf, "head_dim", hf.hidden_size // hf.num_attention_heads)
    rope = getattr(hf, "rope_parameters", None) or {}
    theta = rope.get("rope_theta", getattr(hf, "rope_theta", 1e7))
    prf = rope.get("partial_rotary_factor", getattr(hf, "partial_rotary_factor", 0.25))
    eos = getattr(hf, "eos_token_id", None)
    eos = tuple(eos) if isinstance(eos, (list, tuple)) else ((eos,) if eos is not None else ())
    return ModelConfig(
        name=getattr(hf, "name_or_path", "hf-model") or "hf-model",
        vocab_size=hf.vocab_size,
        hidden_size=hf.hidden_size,
        num_layers=n,
        layer_types=lt,
        intermediate_size=hf.intermediate_size,
        num_q_heads=hf.num_attention_heads,
        num_kv_heads=hf.num_key_value_heads,
        head_dim=head_dim,
        rotary_dim=int(head_dim * prf),
        rope_theta=float(theta),
        gdn_num_k_heads=getattr(hf, "linear_num_key_heads", 16),
        gdn_num_v_heads=getattr(hf, "linear_num_value_heads", 48),
        gdn_head_k_dim=getattr(hf, "linear_key_head_dim", 128),
        gdn_head_v_dim=getattr(hf, "linear_value_head_dim", 128),
        gdn_conv_kernel=getattr(hf, "linear_conv_kernel_dim", 4),
        rms_eps=getattr(hf, "rms_norm_eps", 1e-6),
        tie_embeddings=bool(getattr(hf, "tie_word_embeddings", False)),
        eos_token_ids=eos,
        max_position_embeddings=getattr(hf, "max_position_embeddings", 32768),
    )
