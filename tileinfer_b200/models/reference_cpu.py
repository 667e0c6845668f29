"""Pure-PyTorch executor of the hybrid model: the numerical oracle and the CPU execution path.

Maths follow what the reference executes (model/qwen_36.py:575-708 and 939-1133, with
kernels/deltanet_fused.py:686-757 for the recurrent step and the upstream HuggingFace
qwen3_5 functions for the delta rule, gated norm and causal conv):

* block:  h += Mixer(RMSNorm_{1+w}(h));  h += down(silu(gate(x)) * up(x)),  x = RMSNorm_{1+w}(h)
* gated DeltaNet: [q|k|v] = silu(causal_conv1d(in_proj_qkv(x))), q,k L2-normalised,
  q *= Dk^-1/2, g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b),
  S <- exp(g) S;  delta = beta (v - S^T k);  S <- S + k delta^T;  o = S^T q,
  out = RMSNorm_w(o) * silu(z) per v-head, then out_proj.
* attention: q_proj yields [q|gate] per head, per-head RMSNorm_{1+w} on q and k, partial RoPE
  (rotate-half over the first rotary_dim dims), causal softmax, out * sigmoid(gate), o_proj.

The executor works on a flattened variable-length batch with a paged KV cache and per-sequence
DeltaNet state slots, so the engine's scheduling, chunked prefill, prefix reuse and swapping can be
tested without a GPU.  `naive_logits` recomputes a whole sequence without any cache and is the
ground truth the paged path is tested against.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .config import ModelConfig
from .weights import ShardSpec, fake_quant, shard_layer, QUANTIZED_KEYS


@dataclass
class Batch:
    """One forward step over `num_seqs` sequences flattened to T tokens."""
    input_ids: torch.Tensor          # [T] int64
    positions: torch.Tensor          # [T] int64
    cu_seqlens: list                 # [S+1] token offsets of each sequence in the flat batch
    context_lens: list               # [S] tokens in the KV cache after this step
    block_tables: list               # [S] list[int] physical KV blocks
    slot_mapping: torch.Tensor       # [T] int64 flat KV slot (block*block_size+offset)
    state_slots: list                # [S] DeltaNet state slot per sequence
    # absolute token counts at which a DeltaNet state snapshot must be taken: [S] list[int]
    snapshot_at: list = field(default_factory=list)

    @property
    def num_seqs(self) -> int:
        return len(self.cu_seqlens) - 1


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, one_plus: bool = True) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y * ((1.0 + w.float()) if one_plus else w.float())


def softplus20(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20.0, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def rope_partial(x: torch.Tensor, pos: torch.Tensor, rotary_dim: int, theta: float) -> torch.Tensor:
    """x: [T, H, D]; rotate-half over the first `rotary_dim` dims, pairs (i, i+rotary_dim/2)."""
    half = rotary_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=x.device) * 2.0 / rotary_dim))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:rotary_dim] = x2 * cos + x1 * sin
    return out


def gdn_recurrent(q, k, v, g, beta, state):
    """Token-serial gated delta rule.  q,k: [T,Hv,Dk] (already normalised/scaled), v: [T,Hv,Dv],
    g, beta: [T,Hv], state: [Hv,Dk,Dv] fp32 (updated copy returned).  Returns (o [T,Hv,Dv], state)."""
    T = q.shape[0]
    S = state.clone()
    out = torch.empty_like(v)
    for t in range(T):
        S = S * g[t].exp()[:, None, None]
        kv = torch.einsum("hkv,hk->hv", S, k[t])
        delta = (v[t] - kv) * beta[t][:, None]
        S = S + k[t][:, :, None] * delta[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out, S


def gdn_chunked(q, k, v, g, beta, state, chunk: int = 64):
    """Chunk-parallel form of the same rule (WY / UT transform), used to cross-check kernels.
    Same signature as `gdn_recurrent`."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    pad = (-T) % chunk
    if pad:
        z = lambda x: F.pad(x, (0, 0) * (x.dim() - 1) + (0, pad))
        q, k, v = z(q), z(k), z(v)
        g, beta = F.pad(g, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    n = (T + pad) // chunk
    # -> [H, n, C, *]
    rs = lambda x: x.transpose(0, 1).reshape(H, n, chunk, -1)
    q, k, v = rs(q), rs(k), rs(v)
    g = g.transpose(0, 1).reshape(H, n, chunk).cumsum(-1)
    beta = beta.transpose(0, 1).reshape(H, n, chunk)
    kb, vb = k * beta[..., None], v * beta[..., None]
    decay = (g[..., :, None] - g[..., None, :]).tril().exp().tril()
    upper = torch.triu(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), 0)
    A = -((kb @ k.transpose(-1, -2)) * decay).masked_fill(upper, 0)
    for i in range(1, chunk):
        row = A[..., i, :i].clone()
        sub = A[..., :i, :i].clone()
        A[..., i, :i] = row + (row[..., None] * sub).sum(-2)
    A = A + torch.eye(chunk, device=q.device)
    u = A @ vb
    w = A @ (kb * g.exp()[..., None])
    S = state.clone()
    out = torch.zeros(H, n, chunk, Dv, device=q.device)
    strict = torch.triu(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), 1)
    for i in range(n):
        attn = (q[:, i] @ k[:, i].transpose(-1, -2) * decay[:, i]).masked_fill(strict, 0)
        v_new = u[:, i] - w[:, i] @ S
        out[:, i] = (q[:, i] * g[:, i, :, None].exp()) @ S + attn @ v_new
        S = S * g[:, i, -1, None, None].exp() + \
            (k[:, i] * (g[:, i, -1, None] - g[:, i]).exp()[..., None]).transpose(-1, -2) @ v_new
    out = out.reshape(H, n * chunk, Dv).transpose(0, 1)[:T]
    return out, S


class TorchHybridModel:
    """Functional executor.  `comm` (optional) provides all_reduce(tensor) for TP on CPU ranks."""

    def __init__(self, cfg: ModelConfig, src, *, quant: str = "none", dtype=torch.float32,
                 device="cpu", tp: int = 1, rank: int = 0, comm=None):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.tp, self.rank, self.comm = tp, rank, comm
        cfg.validate_tp(tp)
        sh = ShardSpec(tp, rank)
        self.layers = []
        for i in range(cfg.num_layers):
            lw = shard_layer(cfg, src, i, sh)
            if quant == "w8a16":
                for kname in QUANTIZED_KEYS:
                    if kname in lw:
                        lw[kname] = fake_quant(lw[kname])
            self.layers.append({k: v.to(self.device, dtype) for k, v in lw.items()})
        self.embed = src.get("embed").to(self.device, dtype)
        self.final_norm = src.get("final_norm").to(self.device, dtype)
        head = src.get("lm_head")
        vs = cfg.vocab_size // tp if cfg.vocab_size % tp == 0 else None
        if tp > 1:
            assert vs is not None, "vocab must divide tp"
            head = head[rank * vs:(rank + 1) * vs]
        self.lm_head = head.to(self.device, dtype)
        self.vocab_start = 0 if tp == 1 else rank * vs
        self.hq = cfg.num_q_heads // tp
        self.hkv = cfg.kv_heads_per_rank(tp)
        self.hk = cfg.gdn_num_k_heads // tp
        self.hv = cfg.gdn_num_v_heads // tp
        self.kv_cache = None
        self.rec_state = None
        self.conv_state = None
        self.block_size = 16
        self.snapshots = {}          # (seq index in batch, abs token count) -> (rec, conv) per layer

    # ---- cache management --------------------------------------------------
    def alloc_cache(self, num_blocks: int, block_size: int, num_slots: int):
        c = self.cfg
        self.block_size = block_size
        na, ng = c.num_attn_layers, c.num_gdn_layers
        self.kv_cache = torch.zeros(na, 2, num_blocks * block_size, self.hkv, c.head_dim,
                                    dtype=self.dtype, device=self.device)
        self.rec_state = torch.zeros(ng, num_slots, self.hv, c.gdn_head_k_dim, c.gdn_head_v_dim,
                                     dtype=torch.float32, device=self.device)
        conv_dim = 2 * self.hk * c.gdn_head_k_dim + self.hv * c.gdn_head_v_dim
        self.conv_state = torch.zeros(ng, num_slots, conv_dim, c.gdn_conv_kernel - 1,
                                      dtype=torch.float32, device=self.device)

    def cache_bytes_per_block(self) -> int:
        c = self.cfg
        return c.num_attn_layers * 2 * self.block_size * self.hkv * c.head_dim * self.kv_cache.element_size()

    def zero_state(self, slot: int):
        self.rec_state[:, slot].zero_()
        self.conv_state[:, slot].zero_()

    def state_out(self, slot: int):
        return self.rec_state[:, slot].clone().cpu(), self.conv_state[:, slot].clone().cpu()

    def state_in(self, slot: int, st):
        self.rec_state[:, slot].copy_(st[0])
        self.conv_state[:, slot].copy_(st[1])

    def blocks_out(self, block_ids: list):
        bs = self.block_size
        idx = torch.tensor([b * bs + j for b in block_ids for j in range(bs)], dtype=torch.long)
        return self.kv_cache[:, :, idx].clone().cpu()

    def blocks_in(self, block_ids: list, data):
        bs = self.block_size
        idx = torch.tensor([b * bs + j for b in block_ids for j in range(bs)], dtype=torch.long)
        self.kv_cache[:, :, idx] = data.to(self.device)

    def all_reduce(self, x):
        if self.tp > 1:
            return self.comm.all_reduce(x)
        return x

    # ---- layers ---------------------------------------------------------------
    def _mlp(self, lw, x):
        gu = x @ lw["gate_up"].t()
        act = F.silu(gu[:, 0::2]) * gu[:, 1::2]
        return act @ lw["down"].t()

    def _gdn(self, lw, li_g, x, batch: Batch, snaps):
        c = self.cfg
        dk, dv, hk, hv = c.gdn_head_k_dim, c.gdn_head_v_dim, self.hk, self.hv
        kd, vd = hk * dk, hv * dv
        proj = x @ lw["in_proj"].t()
        qkv_raw = proj[:, :2 * kd + vd]
        z = proj[:, 2 * kd + vd:2 * kd + 2 * vd]
        b = proj[:, 2 * kd + 2 * vd:2 * kd + 2 * vd + hv]
        a = proj[:, 2 * kd + 2 * vd + hv:2 * kd + 2 * vd + 2 * hv]
        K = c.gdn_conv_kernel
        out = torch.empty(x.shape[0], vd, dtype=x.dtype, device=x.device)
        for s in range(batch.num_seqs):
            t0, t1 = batch.cu_seqlens[s], batch.cu_seqlens[s + 1]
            slot = batch.state_slots[s]
            T = t1 - t0
            hist = self.conv_state[li_g, slot].t().to(x.dtype)              # [K-1, conv_dim]
            seq = torch.cat([hist, qkv_raw[t0:t1]], dim=0)                   # [T+K-1, conv_dim]
            win = seq.unfold(0, K, 1)                                        # [T, conv_dim, K]
            conv = F.silu((win * lw["conv_w"][None]).sum(-1))
            q = conv[:, :kd].reshape(T, hk, dk)
            k = conv[:, kd:2 * kd].reshape(T, hk, dk)
            v = conv[:, 2 * kd:].reshape(T, hv, dv)
            rep = hv // hk
            q = l2norm(q.float()).repeat_interleave(rep, dim=1) * dk ** -0.5
            k = l2norm(k.float()).repeat_interleave(rep, dim=1)
            g = -torch.exp(lw["A_log"].float())[None] * softplus20(a[t0:t1].float() + lw["dt_bias"].float()[None])
            beta = torch.sigmoid(b[t0:t1].float())
            start_abs = batch.context_lens[s] - T
            cuts = [n - start_abs for n in (batch.snapshot_at[s] if batch.snapshot_at else []) if 0 < n - start_abs <= T]
            S = self.rec_state[li_g, slot]
            o = torch.empty(T, hv, dv, dtype=torch.float32, device=x.device)
            prev = 0
            for cut in sorted(set(cuts + [T])):
                if cut > prev:
                    o[prev:cut], S = gdn_recurrent(q[prev:cut], k[prev:cut], v[prev:cut].float(),
                                                   g[prev:cut], beta[prev:cut], S)
                if cut in cuts:
                    conv_hist = seq[cut:cut + K - 1].t().float()
                    snaps.setdefault((s, start_abs + cut), []).append((S.clone(), conv_hist.clone()))
                prev = cut
            self.rec_state[li_g, slot] = S
            self.conv_state[li_g, slot] = seq[T:].t().float()
            on = rmsnorm(o, lw["norm_w"], c.rms_eps, one_plus=False)
            zz = z[t0:t1].reshape(T, hv, dv).float()
            out[t0:t1] = (on * F.silu(zz)).reshape(T, vd).to(x.dtype)
        return out @ lw["out"].t()

    def _attn(self, lw, li_a, x, batch: Batch):
        c = self.cfg
        d, hq, hkv = c.head_dim, self.hq, self.hkv
        T = x.shape[0]
        proj = x @ lw["qkv"].t()
        qg = proj[:, :hq * 2 * d].reshape(T, hq, 2 * d)
        q, gate = qg[..., :d], qg[..., d:].reshape(T, hq * d)
        k = proj[:, hq * 2 * d:hq * 2 * d + hkv * d].reshape(T, hkv, d)
        v = proj[:, hq * 2 * d + hkv * d:].reshape(T, hkv, d)
        q = rmsnorm(q, lw["q_norm"], c.rms_eps).to(x.dtype)
        k = rmsnorm(k, lw["k_norm"], c.rms_eps).to(x.dtype)
        q = rope_partial(q, batch.positions, c.rotary_dim, c.rope_theta)
        k = rope_partial(k, batch.positions, c.rotary_dim, c.rope_theta)
        valid = batch.slot_mapping >= 0
        self.kv_cache[li_a, 0, batch.slot_mapping[valid]] = k[valid]
        self.kv_cache[li_a, 1, batch.slot_mapping[valid]] = v[valid]
        out = torch.empty(T, hq * d, dtype=x.dtype, device=x.device)
        bs = self.block_size
        grp = hq // hkv
        for s in range(batch.num_seqs):
            t0, t1 = batch.cu_seqlens[s], batch.cu_seqlens[s + 1]
            L = batch.context_lens[s]
            bt = batch.block_tables[s]
            idx = torch.tensor([bt[p // bs] * bs + p % bs for p in range(L)], dtype=torch.long, device=x.device)
            kk = self.kv_cache[li_a, 0, idx].float()            # [L, hkv, d]
            vv = self.kv_cache[li_a, 1, idx].float()
            qq = q[t0:t1].float().reshape(t1 - t0, hkv, grp, d)
            sc = torch.einsum("tkgd,lkd->tkgl", qq, kk) * d ** -0.5
            qpos = batch.positions[t0:t1]
            mask = torch.arange(L, device=x.device)[None, :] > qpos[:, None]
            sc = sc.masked_fill(mask[:, None, None, :], float("-inf"))
            pr = torch.softmax(sc, dim=-1)
            o = torch.einsum("tkgl,lkd->tkgd", pr, vv).reshape(t1 - t0, hq * d)
            out[t0:t1] = o.to(x.dtype)
        out = out * torch.sigmoid(gate.float()).to(x.dtype)
        return out @ lw["o"].t()

    # ---- forward --------------------------------------------------------------
    @torch.no_grad()
    def forward(self, batch: Batch) -> torch.Tensor:
        """Returns the hidden state (after the final norm) of the LAST token of every sequence [S, H]."""
        c = self.cfg
        h = self.embed[batch.input_ids]
        ig = ia = 0
        snaps = {}
        for i, lw in enumerate(self.layers):
            x = rmsnorm(h, lw["input_norm"], c.rms_eps).to(self.dtype)
            if c.is_gdn(i):
                mix = self._gdn(lw, ig, x, batch, snaps)
                ig += 1
            else:
                mix = self._attn(lw, ia, x, batch)
                ia += 1
            h = h + self.all_reduce(mix)
            x = rmsnorm(h, lw["post_norm"], c.rms_eps).to(self.dtype)
            h = h + self.all_reduce(self._mlp(lw, x))
        self.snapshots = snaps
        last = [batch.cu_seqlens[s + 1] - 1 for s in range(batch.num_seqs)]
        return rmsnorm(h[last], self.final_norm, c.rms_eps).to(self.dtype)

    @torch.no_grad()
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """[S, H] -> this rank's vocabulary shard of the logits [S, V/tp] (fp32)."""
        return (hidden @ self.lm_head.t()).float()

    def take_snapshots(self):
        """{(seq index, abs tokens): (rec [ng,hv,dk,dv], conv [ng,conv_dim,K-1])} from the last forward."""
        out = {}
        for key, per_layer in self.snapshots.items():
            out[key] = (torch.stack([p[0] for p in per_layer]).cpu(), torch.stack([p[1] for p in per_layer]).cpu())
        self.snapshots = {}
        return out


@torch.no_grad()
def naive_logits(cfg: ModelConfig, src, tokens: list, quant: str = "none") -> torch.Tensor:
    """Logits of every position of one sequence, computed without caches (ground truth) [T, V]."""
    m = TorchHybridModel(cfg, src, quant=quant)
    T = len(tokens)
    bs = 16
    nb = (T + bs - 1) // bs
    m.alloc_cache(nb, bs, 1)
    ids = torch.tensor(tokens, dtype=torch.long)
    h = m.embed[ids]
    pos = torch.arange(T)
    batch = Batch(ids, pos, [0, T], [T], [list(range(nb))], torch.arange(T), [0])
    ig = ia = 0
    for i, lw in enumerate(m.layers):
        x = rmsnorm(h, lw["input_norm"], cfg.rms_eps)
        if cfg.is_gdn(i):
            mix = m._gdn(lw, ig, x, batch, {})
            ig += 1
        else:
            mix = m._attn(lw, ia, x, batch)
            ia += 1
        h = h + mix
        h = h + m._mlp(lw, rmsnorm(h, lw["post_norm"], cfg.rms_eps))
    return m.logits(rmsnorm(h, m.final_norm, cfg.rms_eps))
