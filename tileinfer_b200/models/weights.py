"""Weight sources (random-init or HuggingFace checkpoint), INT8 quantisation and TP sharding.

Reference behaviour kept: symmetric per-output-row INT8 with scale = amax/127, rows padded
to a multiple of 64 with scale 1.0 (reference: model/qwen_36.py:172-184); Megatron-style
column/row sharding with Q/K/V segments sharded separately (model/qwen_36.py:445-459,
engine/parallel.py:98-125). New here: bf16 scales, KV-head replication for tp > num_kv_heads,
the tiled int8 layout the sm_100a GEMV/GEMM kernels stream, and an optional on-disk cache of
the per-rank quantised shards so a restart skips quantisation.
"""
from __future__ import annotations

import hashlib
import math
import os
from dataclasses import dataclass

import torch

from .config import ModelConfig

GDN = "linear_attention"


# --------------------------------------------------------------------------- sources
class RandomWeights:
    """Deterministic N(0, std) weights; every tensor has its own generator stream.

    Matrices are rounded to bf16 so the fp32 oracle and the bf16/int8 device path see the
    same values.  RMSNorm weights use the (1+w) convention and are stored as 0 (effective
    scale 1); the DeltaNet gated-norm weight is a plain multiplier and is stored as 1.
    """

    def __init__(self, cfg: ModelConfig, seed: int = 0, std: float = 0.02, device="cpu"):
        self.cfg, self.seed, self.std = cfg, seed, std
        self.device = torch.device(device)
        self.cpu_numel_limit = 1 << 24

    def _gen(self, name: str) -> torch.Generator:
        h = hashlib.sha256(f"{self.seed}:{name}".encode()).digest()
        g = torch.Generator(device=self.device)
        g.manual_seed(int.from_bytes(h[:7], "little"))
        return g

    def shape(self, name: str):
        c = self.cfg
        leaf = name.split(".")[-1]
        kind = name.split(".")[-2] if "." in name else ""
        if name == "embed" or name == "lm_head":
            return (c.vocab_size, c.hidden_size)
        if leaf in ("input_norm", "post_norm") or name == "final_norm":
            return (c.hidden_size,)
        if kind == "mlp":
            return (c.hidden_size, c.intermediate_size) if leaf == "down" else (c.intermediate_size, c.hidden_size)
        if kind == "gdn":
            return {
                "in_qkv": (c.gdn_conv_dim, c.hidden_size),
                "in_z": (c.gdn_value_dim, c.hidden_size),
                "in_b": (c.gdn_num_v_heads, c.hidden_size),
                "in_a": (c.gdn_num_v_heads, c.hidden_size),
                "conv_w": (c.gdn_conv_dim, c.gdn_conv_kernel),
                "A_log": (c.gdn_num_v_heads,),
                "dt_bias": (c.gdn_num_v_heads,),
                "norm_w": (c.gdn_head_v_dim,),
                "out": (c.hidden_size, c.gdn_value_dim),
            }[leaf]
        if kind == "attn":
            return {
                "q": (c.num_q_heads * c.head_dim * 2, c.hidden_size),
                "k": (c.num_kv_heads * c.head_dim, c.hidden_size),
                "v": (c.num_kv_heads * c.head_dim, c.hidden_size),
                "q_norm": (c.head_dim,),
                "k_norm": (c.head_dim,),
                "o": (c.hidden_size, c.num_q_heads * c.head_dim),
            }[leaf]
        raise KeyError(name)

    def get(self, name: str) -> torch.Tensor:
        """Full (unsharded) tensor in fp32 on `self.device`."""
        if name == "lm_head" and self.cfg.tie_embeddings:
            name = "embed"
        shape = self.shape(name)
        leaf = name.split(".")[-1]
        if leaf in ("input_norm", "post_norm", "q_norm", "k_norm") or name == "final_norm":
            return torch.zeros(shape, dtype=torch.float32, device=self.device)
        if leaf == "norm_w":
            return torch.ones(shape, dtype=torch.float32, device=self.device)
        numel = 1
        for d in shape:
            numel *= d
        if self.device.type != "cpu" and numel <= self.cpu_numel_limit:
            # small tensors come from the CPU generator so CPU and GPU runs see identical weights
            cpu = RandomWeights(self.cfg, self.seed, self.std, "cpu")
            return cpu.get(name).to(self.device)
        w = torch.empty(shape, dtype=torch.float32, device=self.device)
        w.normal_(0.0, self.std, generator=self._gen(name))
        return w.to(torch.bfloat16).float()


class HFWeights:
    """Reads a local HuggingFace Qwen3.5/3.6 checkpoint (safetensors) tensor by tensor."""

    _MAP = {
        "input_norm": "input_layernorm.weight",
        "post_norm": "post_attention_layernorm.weight",
        "mlp.gate": "mlp.gate_proj.weight",
        "mlp.up": "mlp.up_proj.weight",
        "mlp.down": "mlp.down_proj.weight",
        "gdn.in_qkv": "linear_attn.in_proj_qkv.weight",
        "gdn.in_z": "linear_attn.in_proj_z.weight",
        "gdn.in_b": "linear_attn.in_proj_b.weight",
        "gdn.in_a": "linear_attn.in_proj_a.weight",
        "gdn.conv_w": "linear_attn.conv1d.weight",
        "gdn.A_log": "linear_attn.A_log",
        "gdn.dt_bias": "linear_attn.dt_bias",
        "gdn.norm_w": "linear_attn.norm.weight",
        "gdn.out": "linear_attn.out_proj.weight",
        "attn.q": "self_attn.q_proj.weight",
        "attn.k": "self_attn.k_proj.weight",
        "attn.v": "self_attn.v_proj.weight",
        "attn.q_norm": "self_attn.q_norm.weight",
        "attn.k_norm": "self_attn.k_norm.weight",
        "attn.o": "self_attn.o_proj.weight",
    }

    def __init__(self, cfg: ModelConfig, model_dir: str, device="cpu"):
        import glob
        import json

        from safetensors import safe_open  # noqa: F401  (fail early when missing)

        self.cfg, self.device = cfg, torch.device(device)
        self.dir = model_dir
        self.index = {}
        idx = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.index = json.load(f)["weight_map"]
        else:
            for fn in glob.glob(os.path.join(model_dir, "*.safetensors")):
                with safe_open(fn, "pt") as f:
                    for k in f.keys():
                        self.index[k] = os.path.basename(fn)
        self._prefix = None
        for cand in ("model.language_model.", "model.", "language_model.model.", ""):
            if f"{cand}embed_tokens.weight" in self.index:
                self._prefix = cand
                break
        if self._prefix is None:
            raise ValueError(f"no embed_tokens.weight under {model_dir}")

    def _load(self, key: str) -> torch.Tensor:
        from safetensors import safe_open

        with safe_open(os.path.join(self.dir, self.index[key]), "pt") as f:
            return f.get_tensor(key)

    def get(self, name: str) -> torch.Tensor:
        p = self._prefix
        if name == "embed":
            key = f"{p}embed_tokens.weight"
        elif name == "final_norm":
            key = f"{p}norm.weight"
        elif name == "lm_head":
            key = "lm_head.weight" if "lm_head.weight" in self.index else f"{p}embed_tokens.weight"
        else:
            _, i, rest = name.split(".", 2)
            key = f"{p}layers.{i}.{self._MAP[rest]}"
        t = self._load(key).to(self.device).float()
        if name.endswith("conv_w"):
            t = t.reshape(t.shape[0], -1)
        return t


def make_weight_source(cfg: ModelConfig, spec: str, model_dir: str | None, device="cpu"):
    """`spec` is "random:<seed>" or "hf"."""
    if spec.startswith("random"):
        seed = int(spec.split(":", 1)[1]) if ":" in spec else 0
        return RandomWeights(cfg, seed=seed, device=device)
    if spec == "hf":
        return HFWeights(cfg, model_dir, device=device)
    raise ValueError(f"unknown weights spec {spec!r}")


# --------------------------------------------------------------------------- quantisation
def quantize_int8_rowwise(w: torch.Tensor):
    """Symmetric per-output-row INT8.  Returns (q int8 [N,K], scale bf16 [N]).

    The scale is rounded to bf16 *before* quantising so that q*scale reproduces the stored
    format exactly.
    """
    w = w.float()
    amax = w.abs().amax(dim=1).clamp_min(1e-8)
    scale = (amax / 127.0).to(torch.bfloat16)
    q = torch.round(w / scale.float()[:, None]).clamp_(-128, 127).to(torch.int8)
    return q, scale


def dequantize_int8_rowwise(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.float() * scale.float()[:, None]


def fake_quant(w: torch.Tensor) -> torch.Tensor:
    q, s = quantize_int8_rowwise(w)
    return dequantize_int8_rowwise(q, s)


def pad_rows(w: torch.Tensor, mult: int) -> torch.Tensor:
    n = w.shape[0]
    pad = (-n) % mult
    if pad == 0:
        return w
    return torch.cat([w, w.new_zeros((pad,) + tuple(w.shape[1:]))], dim=0)


def tile_int8(q: torch.Tensor) -> torch.Tensor:
    """[N,K] int8 row-major -> [N/8, K/64, 8, 64] contiguous (one 512-byte tile per 8 rows x 64 k).

    A warp of the GEMV kernel reads one tile with a single fully coalesced 16-byte-per-lane load;
    the same tile is one 8-row x 128-byte bf16 swizzle atom after dequantisation in the GEMM.
    """
    n, k = q.shape
    assert n % 8 == 0 and k % 64 == 0, (n, k)
    return q.view(n // 8, 8, k // 64, 64).permute(0, 2, 1, 3).contiguous()


def untile_int8(t: torch.Tensor) -> torch.Tensor:
    nt, kt, _, _ = t.shape
    return t.permute(0, 2, 1, 3).reshape(nt * 8, kt * 64)


def tile_bf16(w: torch.Tensor) -> torch.Tensor:
    """[N,K] bf16 row-major -> [N/8, K/32, 8, 32] (same 512-byte tiles, 32 bf16 per row)."""
    n, k = w.shape
    assert n % 8 == 0 and k % 32 == 0, (n, k)
    return w.view(n // 8, 8, k // 32, 32).permute(0, 2, 1, 3).contiguous()


# --------------------------------------------------------------------------- TP sharding
@dataclass
class ShardSpec:
    tp: int
    rank: int

    def rows(self, w: torch.Tensor, groups: int = 1) -> torch.Tensor:
        """Column-parallel: shard dim 0; `groups` keeps group boundaries (e.g. per-head blocks)."""
        if self.tp == 1:
            return w
        n = w.shape[0]
        assert n % self.tp == 0, (n, self.tp)
        s = n // self.tp
        return w[self.rank * s:(self.rank + 1) * s]

    def cols(self, w: torch.Tensor) -> torch.Tensor:
        """Row-parallel: shard dim 1 (input features)."""
        if self.tp == 1:
            return w
        k = w.shape[1]
        assert k % self.tp == 0, (k, self.tp)
        s = k // self.tp
        return w[:, self.rank * s:(self.rank + 1) * s]


def shard_layer(cfg: ModelConfig, src, layer: int, sh: ShardSpec) -> dict:
    """Per-rank fp32 tensors of one decoder layer, already concatenated the way the kernels want.

    Returns (GDN layer):  in_proj [q|k|v|z|b|a rows], conv_w [q|k|v channels, 4], A_log, dt_bias,
                          norm_w, out [H, Vdim/tp]
            (attention):  qkv [per-head (q|gate) ... | k | v], q_norm, k_norm, o [H, Hq*D/tp]
            (both):       input_norm, post_norm, gate_up (gate,up rows interleaved), down [H, I/tp]
    """
    c, p = cfg, f"layers.{layer}"
    out = {
        "input_norm": src.get(f"{p}.input_norm"),
        "post_norm": src.get(f"{p}.post_norm"),
    }
    gate = sh.rows(src.get(f"{p}.mlp.gate"))
    up = sh.rows(src.get(f"{p}.mlp.up"))
    out["gate_up"] = torch.stack([gate, up], dim=1).reshape(-1, gate.shape[1])  # g0,u0,g1,u1,...
    out["down"] = sh.cols(src.get(f"{p}.mlp.down"))
    if c.is_gdn(layer):
        kd, vd = c.gdn_key_dim, c.gdn_value_dim
        qkv = src.get(f"{p}.gdn.in_qkv")
        q, k, v = qkv[:kd], qkv[kd:2 * kd], qkv[2 * kd:]
        parts = [sh.rows(q), sh.rows(k), sh.rows(v), sh.rows(src.get(f"{p}.gdn.in_z")),
                 sh.rows(src.get(f"{p}.gdn.in_b")), sh.rows(src.get(f"{p}.gdn.in_a"))]
        out["in_proj"] = torch.cat(parts, dim=0)
        cw = src.get(f"{p}.gdn.conv_w")
        out["conv_w"] = torch.cat([sh.rows(cw[:kd]), sh.rows(cw[kd:2 * kd]), sh.rows(cw[2 * kd:])], dim=0)
        out["A_log"] = sh.rows(src.get(f"{p}.gdn.A_log"))
        out["dt_bias"] = sh.rows(src.get(f"{p}.gdn.dt_bias"))
        out["norm_w"] = src.get(f"{p}.gdn.norm_w")
        out["out"] = sh.cols(src.get(f"{p}.gdn.out"))
    else:
        d = c.head_dim
        hq = c.num_q_heads // sh.tp
        q = src.get(f"{p}.attn.q")[sh.rank * hq * 2 * d:(sh.rank + 1) * hq * 2 * d]
        kvh = c.kv_heads_per_rank(sh.tp)
        k0 = c.kv_head_start(sh.tp, sh.rank)
        k = src.get(f"{p}.attn.k")[k0 * d:(k0 + kvh) * d]
        v = src.get(f"{p}.attn.v")[k0 * d:(k0 + kvh) * d]
        out["qkv"] = torch.cat([q, k, v], dim=0)
        out["q_norm"] = src.get(f"{p}.attn.q_norm")
        out["k_norm"] = src.get(f"{p}.attn.k_norm")
        out["o"] = sh.cols(src.get(f"{p}.attn.o"))
    return out


QUANTIZED_KEYS = ("in_proj", "out", "qkv", "o", "gate_up", "down")


def shard_cache_path(cache_dir: str, cfg: ModelConfig, spec: str, quant: str, tp: int, rank: int) -> str:
    tag = hashlib.sha1(f"{cfg.name}|{spec}|{quant}|{tp}".encode()).hexdigest()[:12]
    return os.path.join(cache_dir, f"{cfg.name}-{tag}-tp{tp}-rank{rank}.pt")


def weight_bytes_per_rank(cfg: ModelConfig, tp: int, quant: str = "w8a16") -> int:
    """Bytes of layer weights + lm_head a decode step streams on one rank."""
    c = cfg
    b = 1 if quant == "w8a16" else 2
    kvh = c.kv_heads_per_rank(tp)
    gdn = (c.gdn_conv_dim + c.gdn_value_dim + 2 * c.gdn_num_v_heads) // tp * c.hidden_size \
        + c.hidden_size * c.gdn_value_dim // tp
    att = (c.num_q_heads * 2 * c.head_dim // tp + 2 * kvh * c.head_dim) * c.hidden_size \
        + c.hidden_size * c.num_q_heads * c.head_dim // tp
    mlp = 3 * c.hidden_size * c.intermediate_size // tp
    total = c.num_gdn_layers * (gdn + mlp) + c.num_attn_layers * (att + mlp)
    return total * b + c.vocab_size // tp * c.hidden_size * 2


def align_up(x: int, m: int) -> int:
    return int(math.ceil(x / m) * m)
