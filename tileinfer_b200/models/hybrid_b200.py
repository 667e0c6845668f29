"""The hybrid model on one B200 (one tensor-parallel rank): weights in kernel layout, KV / DeltaNet
pools, the fused decode step (CUDA-graph captured) and the variable-length prefill / mixed step.

Replaces the reference's patched HuggingFace layers (model/qwen_36.py:242-1147) and the device half of
its ModelRunner (engine/model_runner.py:135-498).  Per decoder layer the decode step launches

  DeltaNet:   in_proj GEMV [RMSNorm fused in]  ->  gdn step (conv + delta rule + gated norm, in place)
              -> out_proj GEMV [all-reduce + residual fused in]
  attention:  qkv GEMV [RMSNorm fused in] -> qk-norm + RoPE + KV store -> paged attention (+ merge, gate)
              -> o_proj GEMV [all-reduce + residual fused in]
  MLP:        gate_up GEMV [RMSNorm in, SwiGLU out] -> down GEMV [all-reduce + residual fused in]

i.e. 5-7 launches and no separate collective, against 12-14 launches plus two NCCL all-reduces in the
reference (model/qwen_36.py:710-809, 939-1133).
"""
from __future__ import annotations

import gc
import math
import os

import torch

from ..ops import functional as F
from ..ops.functional import (EPI_ARGMAX, EPI_F32, EPI_ROWPAR, EPI_STORE, EPI_SWIGLU, XGLOBAL, XNORM, AttnParams, EditParams,
                              GdnChunkParams, GdnParams, GemvWorkspace, LinearW, QkvPrepParams, SampleParams, TopkParams, ptr)
from ..utils.trace import nvtx_end, nvtx_mark
from .config import ModelConfig
from .weights import ShardSpec, shard_layer

BF16 = torch.bfloat16


class _Layer:
    pass


class _ModelBase:
    def __init__(self, cfg: ModelConfig, src, *, quant="w8a16", tp=1, rank=0, comm=None, config=None):
        assert torch.cuda.is_available(), "B200HybridModel needs a CUDA device"
        F.L()   # load (or build) the kernel library now: fail loudly if it is missing
        self.cfg, self.tp, self.rank, self.comm = cfg, tp, rank, comm
        self.dev = torch.device("cuda", torch.cuda.current_device())
        cfg.validate_tp(tp)
        self.quant = quant
        self.state_bf16 = bool(config is not None and config.gdn_state_dtype == "bf16")
        self.fused = True if config is None else bool(config.fused_collectives)
        q8 = quant == "w8a16"
        c = cfg
        self.hq = c.num_q_heads // tp
        self.hkv = c.kv_heads_per_rank(tp)
        self.hk = c.gdn_num_k_heads // tp
        self.hv = c.gdn_num_v_heads // tp
        self.D, self.dk, self.dv = c.head_dim, c.gdn_head_k_dim, c.gdn_head_v_dim
        self.H = c.hidden_size
        self.I = c.intermediate_size // tp
        self.nch = 2 * self.dk + self.dv
        assert (self.dk, self.dv) in ((128, 128), (64, 64)), "gdn kernel instances: 128x128 and 64x64"
        assert self.D in (64, 128, 256)
        dev = self.dev
        cache = None
        if config is not None and getattr(config, "weight_cache_dir", None):
            from .weights import shard_cache_path
            spec = f"{getattr(config, 'model', cfg.name)}|{getattr(config, 'weights', '')}|seed{getattr(config, 'seed', 0)}"
            cache = shard_cache_path(config.weight_cache_dir, cfg, spec, quant, tp, rank)
        if cache is not None and os.path.exists(cache):
            self._load_shards(cache)
        else:
            self._build_shards(src, q8)
            if cache is not None:
                self._save_shards(cache)
        torch.cuda.empty_cache()

        self.ws = GemvWorkspace(dev)
        self.peer = None
        if tp > 1 and self.fused:
            from ..parallel.symm_mem import PeerComm
            rows = 0
            if config is not None:
                rows = max(int(config.max_num_batched_tokens), int(config.max_num_seqs), 64)
            self.peer = PeerComm(comm, self.H, m_cap=64, ar_rows=rows)
        self._ar_pending = None            # a many-row all-reduce whose result nobody has consumed yet
        self.ar_min_rows = int(os.environ.get("TI_AR_MIN_ROWS", "3"))   # more rows than this: GEMM + fused all-reduce
        # (measured at TP = 2, tok/s, packet GEMV -> GEMM + ar_rows: batch 2 331 -> 323, batch 4 590 -> 617, batch 8
        # 964 -> 1167, batch 16 1400 -> 2181)
        # two-shot all-reduce (reduce 1/tp of the rows, broadcast the sums, then read locally) from this many rows on this
        # many ranks: the one-shot form moves tp times more bytes per GPU, which only matters once the rows are many
        self.ar_two_shot_rows = int(os.environ.get("TI_AR_TWO_SHOT_ROWS", "256"))
        self.ar_two_shot_tp = int(os.environ.get("TI_AR_TWO_SHOT_TP", "4"))
        self.ctrl = self.peer.ctrl if self.peer is not None else torch.zeros(4, dtype=torch.int32, device=dev)
        self.step_ptr = self.ctrl.data_ptr()
        self.block_size = 16
        self.kv = None
        self.graphs = {}
        self.snapshots = {}
        self._order = 0
        self.host_steps = 0
        # one projection buffer serves both layer kinds; its row pitch is a multiple of 8 elements so that every row starts
        # on a 16-byte boundary (the attention kernels read the output gate with 16-byte loads; a DeltaNet projection
        # of 2 * hv extra columns is not a multiple of 8 for every tensor-parallel size, e.g. 2060 at TP = 8)
        self.proj_cols = (max([L.in_proj.N for L in self.layers if L.is_gdn] + [L.qkv.N for L in self.layers if not L.is_gdn]) + 7) // 8 * 8
        self.mix_cols = max(self.hv * self.dv, self.hq * self.D)
        self.launches_per_decode_step = 0
        self._launches = 0
        self._pending, self._pending_wt = [], 0
        self.chain = os.environ.get("TI_GEMV_CHAIN", "1") != "0"
        self.ll_handoff = os.environ.get("TI_LL_HANDOFF", "1") == "1"
        # every CTA then reads the packets of all ranks (tp x 40 KB per row): worth it for two ranks (measured +2 %),
        # more L2 traffic than the grid-wide collect + barrier it replaces for more
        self.ll_handoff_max_tp = int(os.environ.get("TI_LL_HANDOFF_MAX_TP", "2"))
        self.gdn_split = os.environ.get("TI_GDN_SPLIT", "0") == "1"   # prefill: a head's columns over a 4-block cluster
        # steps in which some sequence has at least this many tokens use the chunk-parallel DeltaNet kernels
        self.gdn_chunk_min_tokens = int(os.environ.get("TI_GDN_CHUNK_MIN", "32"))
        self.gdn_ws = F.GdnChunkWorkspace(dev)
        # more rows than this: tcgen05 GEMM; the persistent GEMV chain serves single rows.  (Measured on the 27B model,
        # one GPU, ms per decode step: 1 row 6.6 on the GEMV chain; 2 / 3 / 4 rows 8.2 / - / 10.5 on the GEMV against
        # 6.9 / 7.4 / 7.4 on the GEMM; 8 rows 16.0 on the GEMV, whose long-k products then need two passes over the
        # weights, 7.7 on the GEMM.)
        self.gemm_min_rows = int(os.environ.get("TI_GEMM_MIN_ROWS", "1"))

    # ------------------------------------------------------------------ weights: build / on-disk shard cache
    _LINEAR = ("gate_up", "down", "in_proj", "out", "qkv", "o")
    _PLAIN = ("input_norm", "post_norm", "conv_w", "neg_a_exp", "dt_bias", "norm_w", "q_norm", "k_norm")

    def _build_shards(self, src, q8: bool):
        """Shards, quantises and tiles this rank's weights from the source (replaces the per-layer CPU slicing and
        GPU quantisation of model/qwen_36.py:445-521, 861-898)."""
        c, tp, rank, dev = self.cfg, self.tp, self.rank, self.dev
        sh = ShardSpec(tp, rank)
        self.layers = []
        for i in range(c.num_layers):
            lw = shard_layer(c, src, i, sh)
            L = _Layer()
            L.is_gdn = c.is_gdn(i)
            L.input_norm = lw["input_norm"].to(dev, BF16).contiguous()
            L.post_norm = lw["post_norm"].to(dev, BF16).contiguous()
            L.gate_up = LinearW(lw["gate_up"], q8, dev)
            L.down = LinearW(lw["down"], q8, dev)
            if L.is_gdn:
                L.in_proj = LinearW(lw["in_proj"], q8, dev)
                L.out = LinearW(lw["out"], q8, dev)
                L.conv_w = lw["conv_w"].to(dev, torch.float32).contiguous()
                L.neg_a_exp = (-torch.exp(lw["A_log"].float())).to(dev).contiguous()
                L.dt_bias = lw["dt_bias"].to(dev, torch.float32).contiguous()
                L.norm_w = lw["norm_w"].to(dev, torch.float32).contiguous()
            else:
                L.qkv = LinearW(lw["qkv"], q8, dev)
                L.o = LinearW(lw["o"], q8, dev)
                L.q_norm = lw["q_norm"].to(dev, BF16).contiguous()
                L.k_norm = lw["k_norm"].to(dev, BF16).contiguous()
            self.layers.append(L)
            del lw
        self.embed = src.get("embed").to(dev, BF16).contiguous()
        self.final_norm = src.get("final_norm").to(dev, BF16).contiguous()
        head = src.get("lm_head")
        if tp > 1:
            assert c.vocab_size % tp == 0
            vs = c.vocab_size // tp
            head = head[rank * vs:(rank + 1) * vs]
            self.vocab_start = rank * vs
        else:
            self.vocab_start = 0
        self.lm_head = LinearW(head, False, dev)
        self.v_local = self.lm_head.N
        del head

    def _save_shards(self, path: str):
        """Writes this rank's weights in kernel layout (int8 tiles + bf16 scales, bf16 tiles) so that the next start
        skips sharding and quantisation.  Written to a temporary name first: a reader never sees half a file."""
        layers = []
        for L in self.layers:
            d = {"is_gdn": L.is_gdn}
            for k in self._LINEAR:
                if hasattr(L, k):
                    d[k] = {n: (v.cpu() if torch.is_tensor(v) else v) for n, v in getattr(L, k).state().items()}
            for k in self._PLAIN:
                if hasattr(L, k):
                    d[k] = getattr(L, k).cpu()
            layers.append(d)
        blob = {"format": 1, "layers": layers, "embed": self.embed.cpu(), "final_norm": self.final_norm.cpu(),
                "lm_head": {n: (v.cpu() if torch.is_tensor(v) else v) for n, v in self.lm_head.state().items()},
                "vocab_start": self.vocab_start}
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        tmp = f"{path}.tmp{os.getpid()}"
        torch.save(blob, tmp)
        os.replace(tmp, path)

    def _load_shards(self, path: str):
        blob = torch.load(path, map_location="cpu", weights_only=True)
        if blob.get("format") != 1 or len(blob["layers"]) != self.cfg.num_layers:
            raise RuntimeError(f"{path}: not a shard cache of this model")
        dev = self.dev
        self.layers = []
        for d in blob["layers"]:
            L = _Layer()
            L.is_gdn = d["is_gdn"]
            for k in self._LINEAR:
                if k in d:
                    setattr(L, k, LinearW.from_state(d[k], dev))
            for k in self._PLAIN:
                if k in d:
                    setattr(L, k, d[k].to(dev))
            self.layers.append(L)
        self.embed = blob["embed"].to(dev)
        self.final_norm = blob["final_norm"].to(dev)
        self.lm_head = LinearW.from_state(blob["lm_head"], dev)
        self.vocab_start = blob["vocab_start"]
        self.v_local = self.lm_head.N

    # ------------------------------------------------------------------ caches
    def weight_bytes(self) -> int:
        n = self.lm_head.nbytes()
        for L in self.layers:
            for name in ("gate_up", "down", "in_proj", "out", "qkv", "o"):
                w = getattr(L, name, None)
                if w is not None:
                    n += w.nbytes()
        return n

    def _state_bytes_per_slot(self) -> int:
        ng = self.cfg.num_gdn_layers
        return ng * self.hv * (self.dk * self.dv * (2 if self.state_bf16 else 4) + 3 * self.nch * 2)

    def cache_bytes_per_block(self) -> int:
        return self.cfg.num_attn_layers * 2 * 16 * self.hkv * self.D * 2

    def auto_num_blocks(self, util, block_size, num_slots, max_num_seqs, max_model_len) -> int:
        free, total = torch.cuda.mem_get_info()
        budget = free - (1.0 - util) * total - num_slots * self._state_bytes_per_slot() - (2 << 30)
        n = int(budget // self.cache_bytes_per_block())
        cap = max_num_seqs * (max_model_len // block_size + 2) + 64
        n = min(n, cap)
        if n < max_model_len // block_size + 2:
            raise RuntimeError(f"not enough GPU memory for one sequence of {max_model_len} tokens ({n} KV blocks)")
        return n

    def alloc_cache(self, num_blocks: int, block_size: int, num_slots: int):
        assert block_size == 16
        c, dev = self.cfg, self.dev
        na, ng = c.num_attn_layers, c.num_gdn_layers
        self.num_blocks, self.num_slots = num_blocks, num_slots
        self.kv = torch.zeros(max(na, 1), 2, num_blocks, self.hkv * 16 * self.D, dtype=BF16, device=dev)
        sdt = BF16 if self.state_bf16 else torch.float32
        self.rec = torch.zeros(max(ng, 1), num_slots, self.hv, self.dk, self.dv, dtype=sdt, device=dev)
        self.conv = torch.zeros(max(ng, 1), num_slots, self.hv, 3, self.nch, dtype=BF16, device=dev)

    def zero_state(self, slot: int):
        self.rec[:, slot].zero_()
        self.conv[:, slot].zero_()

    # ---- swap: pinned host buffers (recycled by shape), asynchronous copies ordered by the compute stream
    def _pinned(self, shape, dtype):
        pool = getattr(self, "_pin_pool", None)
        if pool is None:
            pool = self._pin_pool = {}
        free = pool.setdefault((tuple(shape), dtype), [])
        return free.pop() if free else torch.empty(tuple(shape), dtype=dtype, pin_memory=True)

    def _unpin(self, t):
        self._pin_pool.setdefault((tuple(t.shape), t.dtype), []).append(t)

    def state_out(self, slot: int):
        """Recurrent state + conv history of a slot -> pinned host memory (asynchronous; the copy back is ordered
        after it on the same stream).  The buffers are recycled when `state_in` consumes them."""
        rec, conv = self.rec[:, slot], self.conv[:, slot]
        hr, hc = self._pinned(rec.shape, rec.dtype), self._pinned(conv.shape, conv.dtype)
        hr.copy_(rec, non_blocking=True)
        hc.copy_(conv, non_blocking=True)
        live = getattr(self, "_swap_live", None)
        if live is None:
            live = self._swap_live = []
        live.extend((hr, hc))
        return hr, hc

    def state_in(self, slot: int, st):
        """Restores a slot from a swapped-out state (pinned host tensors from `state_out`) or from a prefix
        snapshot (device tensors, which stay owned by the snapshot cache)."""
        self.rec[:, slot].copy_(st[0], non_blocking=True)
        self.conv[:, slot].copy_(st[1], non_blocking=True)
        live = getattr(self, "_swap_live", [])
        for t in st:
            if any(t is x for x in live):
                self._swap_live = live = [x for x in live if x is not t]
                self._unpin(t)               # later writers of this buffer are ordered after the copy above

    def blocks_out(self, block_ids: list):
        idx = torch.tensor(block_ids, dtype=torch.long, device=self.dev)
        dev = self.kv[:, :, idx]
        host = self._pinned(dev.shape, dev.dtype)
        host.copy_(dev, non_blocking=True)
        return host

    def blocks_in(self, block_ids: list, data):
        idx = torch.tensor(block_ids, dtype=torch.long, device=self.dev)
        self.kv[:, :, idx] = data.to(self.dev, non_blocking=True)
        if data.device.type == "cpu" and data.is_pinned():
            self._unpin(data)

    def take_snapshots(self):
        out, self.snapshots = self.snapshots, {}
        return out


class _Ctx:
    """Device tensors of one step (static for CUDA-graph buckets, fresh for eager steps)."""
    snap_rel = None
    snap_idx = None
    snap_state = None
    snap_conv = None
    num_snap = 0
    cu = None
    tiles = None            # [3, n] query tiles of the tcgen05 prefill attention (sequence, first token, tokens)
    ck = None               # [4, nc] chunk table of the chunked DeltaNet prefill (None: token-serial kernel)
    seq_ck = None


class _StepMixin:
    # ------------------------------------------------------------------ buffers
    def _alloc_ctx(self, T: int, S: int, max_blocks: int, num_qg: int, nsplit: int) -> _Ctx:
        dev, x = self.dev, _Ctx()
        x.T, x.S, x.max_blocks, x.num_qg, x.nsplit = T, S, max_blocks, num_qg, nsplit
        x.ids = torch.zeros(T, dtype=torch.long, device=dev)
        x.positions = torch.zeros(T, dtype=torch.int32, device=dev)
        x.slot_mapping = torch.full((T,), -1, dtype=torch.long, device=dev)
        x.slots = torch.zeros(S, dtype=torch.int32, device=dev)
        x.block_tables = torch.zeros(S, max_blocks, dtype=torch.int32, device=dev)
        x.qg = torch.zeros(3, max(num_qg, 1), dtype=torch.int32, device=dev)      # seq, tok0, ntok
        x.h = [torch.zeros(T, self.H, dtype=BF16, device=dev) for _ in range(2)]
        x.proj = torch.zeros(T, self.proj_cols, dtype=BF16, device=dev)
        x.mix = torch.zeros(T, self.mix_cols, dtype=BF16, device=dev)
        x.act = torch.zeros(T, self.I, dtype=BF16, device=dev)
        if self.cfg.num_attn_layers:
            x.qbuf = torch.zeros(T, self.hq * self.D, dtype=BF16, device=dev)
            items = max(num_qg, 1) * self.hkv * nsplit
            x.o_part = torch.empty(items * 16 * self.D, dtype=torch.float32, device=dev)
            x.ml_part = torch.empty(items * 32, dtype=torch.float32, device=dev)
        return x

    # ------------------------------------------------------------------ launches
    def _gemm(self, W: LinearW, x, out, M, *, epi, norm_w=None, resid=None):
        """Many rows (prefill, batched decode): the tcgen05 GEMM.  int8 weights: limb planes of x first
        (RMSNorm fused); bf16 weights: RMSNorm kernel first when the product wants normalised input."""
        self._flush()
        gepi = {EPI_STORE: F.GEPI_STORE, EPI_SWIGLU: F.GEPI_SWIGLU, EPI_ROWPAR: F.GEPI_ROWPAR, EPI_F32: F.GEPI_F32}[epi]
        r = None if resid is None else resid[:M]
        if W.wt == F.W_INT8:
            limbs = F.quant_rows(x[:M], norm_w=norm_w, eps=self.cfg.rms_eps)
            F.gemm_w8a16(W, limbs, out=out[:M], epi=gepi, resid=r)
            self._launches += 2
            return
        xs = x[:M]
        if norm_w is not None:
            xs = F.rmsnorm(xs, norm_w, self.cfg.rms_eps)
            self._launches += 1
        elif xs.stride(0) != W.K:
            xs = xs.contiguous()
            self._launches += 1
        F.gemm_bf16(W, xs, out=out[:M], epi=gepi, resid=r)
        self._launches += 1

    def _gemv(self, W: LinearW, x, out, M, *, xmode, epi, norm_w=None, resid=None, ldo=None, out_idx=None):
        """y = x W^T in row chunks of 16; counts launches; assigns collective order numbers."""
        pend = self._ar_pending
        if pend is not None:
            if (pend["out"].data_ptr() == x.data_ptr() and pend["M"] == M and xmode == XNORM and M > self.gemm_min_rows
                    and (W.wt == F.W_BF16 or epi != EPI_F32) and x.stride(0) == W.K):
                return self._gemm_after_ar(W, x, out, M, epi=epi, norm_w=norm_w, resid=resid)
            self._ar_flush()
        if M > self.gemm_min_rows and (W.wt == F.W_BF16 or epi != EPI_F32) and not (epi == EPI_ROWPAR and self.tp > 1):
            return self._gemm(W, x, out, M, epi=epi, norm_w=norm_w if xmode == XNORM else None, resid=resid)
        step = F.max_rows(W.wt, xmode, W.K)
        for m0 in range(0, M, step):
            m = min(step, M - m0)
            order = 0
            if epi == EPI_ROWPAR:
                order = self._order
                self._order += 1
            # the product that consumes an all-reduced row-parallel output collects the packets itself (same launch)
            prev = self._pending[-1] if self._pending else None
            xll = (self.ll_handoff and prev is not None and M <= step and self.chain and prev.epi == EPI_ROWPAR
                   and 1 < prev.tp <= self.ll_handoff_max_tp and prev.M == m and prev.out == x.data_ptr() and prev.N == W.K
                   and x.stride(0) == W.K and xmode == XNORM and self._pending_wt == W.wt
                   and len(self._pending) < F.MAX_CHAIN)
            p = F.make_gemv_params(
                W, x[m0:m0 + m], out[m0:m0 + m], m, xmode=xmode, epi=epi, norm_w=norm_w,
                resid=None if resid is None else resid[m0:m0 + m], ws=self.ws, eps=self.cfg.rms_eps,
                ldx=x.stride(0), ldo=out.stride(0) if ldo is None else ldo,
                comm=self.peer if epi == EPI_ROWPAR else None, order=order, xll=xll,
                out_idx=None if out_idx is None else out_idx[m0:m0 + m])
            if M <= step and self.chain:
                # dependent products are collected and launched together (up to four per launch)
                if self._pending and (self._pending_wt != W.wt or len(self._pending) >= F.MAX_CHAIN):
                    self._flush()
                self._pending.append(p)
                self._pending_wt = W.wt
            else:
                F.gemv_launch(p, W.wt, xmode, epi)
                self._launches += 1

    def _gemm_after_ar(self, W: LinearW, x, out, M, *, epi, norm_w, resid):
        """The product that consumes an all-reduced row-parallel output: ONE kernel sums the ranks' partials over
        NVLink, adds the residual, writes the new residual stream `x`, and runs this product's prologue (RMSNorm,
        then int8 limb planes or bf16) on the rows while they are still in registers; then the tcgen05 GEMM."""
        pend, self._ar_pending = self._ar_pending, None
        self._flush()
        gepi = {EPI_STORE: F.GEPI_STORE, EPI_SWIGLU: F.GEPI_SWIGLU, EPI_ROWPAR: F.GEPI_ROWPAR, EPI_F32: F.GEPI_F32}[epi]
        r = None if resid is None else resid[:M]
        if W.wt == F.W_INT8:
            limbs = F.Limbs(M, W.K, self.dev)
            F.ar_rows(self.peer, pend["parity"], M, W.K, pend["resid"], x, order=pend["order"], mode=F.AR_LIMBS,
                      norm_w=norm_w, limbs=limbs, eps=self.cfg.rms_eps, two_shot=self._two_shot(M))
            F.gemm_w8a16(W, limbs, out=out[:M], epi=gepi, resid=r)
        else:
            xn = torch.empty(M, W.K, dtype=BF16, device=self.dev)
            F.ar_rows(self.peer, pend["parity"], M, W.K, pend["resid"], x, order=pend["order"], mode=F.AR_BF16,
                      norm_w=norm_w, xn=xn, eps=self.cfg.rms_eps, two_shot=self._two_shot(M))
            F.gemm_bf16(W, xn, out=out[:M], epi=gepi, resid=r)
        self._launches += 2

    def _ar_flush(self):
        """Completes a pending many-row all-reduce whose consumer is not a normalising GEMM (end of the step)."""
        pend, self._ar_pending = self._ar_pending, None
        if pend is not None:
            F.ar_rows(self.peer, pend["parity"], pend["M"], self.H, pend["resid"], pend["out"], order=pend["order"],
                      two_shot=self._two_shot(pend["M"]))
            self._launches += 1

    def _two_shot(self, M: int) -> int:
        return int(self.tp >= self.ar_two_shot_tp and M >= self.ar_two_shot_rows)

    def _flush(self):
        if self._pending:
            F.gemv_chain_launch(self._pending, self._pending_wt)
            self._launches += 1
            self._pending = []

    def _rowpar(self, W: LinearW, x, resid, out, M):
        """Row-parallel projection + all-reduce + residual add -> out."""
        # Under tensor parallelism, steps of up to m_cap rows (every decode bucket, so everything a CUDA graph
        # captures) keep the fused peer-memory all-reduce of the GEMV; only larger (eager prefill) steps take the
        # tcgen05 GEMM followed by an NCCL all-reduce.
        if self.tp > 1 and self.peer is not None and M > max(self.ar_min_rows, self.gemm_min_rows):
            # many rows under tensor parallelism: the tcgen05 GEMM stores this rank's partial sums (bf16) straight
            # into its symmetric buffer; the all-reduce, the residual add and the consumer's prologue are one kernel
            # launched by whoever consumes `out` (see _gemm_after_ar)
            self._ar_flush()
            order = self._order
            self._order += 1
            part = self.peer.part_view(order & 1, M)
            self._gemm(W, x, part, M, epi=EPI_STORE)
            self._ar_pending = {"parity": order & 1, "resid": resid[:M], "out": out, "M": M, "order": order}
            return
        fused_cap = self.peer.m_cap if self.peer is not None else self.gemm_min_rows
        if self.tp > 1 and M > max(fused_cap, self.gemm_min_rows):
            # prefill under tensor parallelism: tcgen05 GEMM to a bf16 partial, NCCL all-reduce, residual add
            part = torch.empty(M, W.N, dtype=BF16, device=self.dev)
            self._gemm(W, x, part, M, epi=EPI_STORE)
            self.comm.all_reduce(part)
            torch.add(resid[:M], part, out=out[:M])
            self._launches += 2
            return
        if self.tp == 1 or self.peer is not None:
            self._gemv(W, x, out, M, xmode=XGLOBAL, epi=EPI_ROWPAR, resid=resid)
            return
        # baseline: partial sums in bf16, NCCL all-reduce, separate residual add (the reference's structure)
        part = torch.empty(M, W.N, dtype=BF16, device=self.dev)
        self._gemv(W, x, part, M, xmode=XGLOBAL, epi=EPI_STORE)
        self._flush()
        self.comm.all_reduce(part)
        torch.add(resid[:M], part, out=out[:M])
        self._launches += 2

    def _run_layers(self, x: _Ctx):
        c, T, S = self.cfg, x.T, x.S
        eps = c.rms_eps
        if self.peer is not None and not torch.cuda.is_current_stream_capturing():
            self.peer.tick()
        F.embed(x.ids, self.embed, x.h[0], self.step_ptr)
        self._launches += 1
        self._order = 0
        cur, nxt = x.h[0], x.h[1]
        ig = ia = 0
        for li, L in enumerate(self.layers):
            nvtx_mark(f"layer {li} {'deltanet' if L.is_gdn else 'attention'} mixer")     # ranges only with TI_NVTX=1
            if L.is_gdn:
                self._gemv(L.in_proj, cur, x.proj, T, xmode=XNORM, epi=EPI_STORE, norm_w=L.input_norm)
                p = GdnParams()
                p.proj, p.conv_w, p.neg_a_exp, p.dt_bias, p.norm_w = ptr(x.proj), ptr(L.conv_w), ptr(L.neg_a_exp), ptr(L.dt_bias), ptr(L.norm_w)
                p.state, p.conv_state = ptr(self.rec[ig]), ptr(self.conv[ig])
                p.slots, p.cu, p.out = ptr(x.slots), ptr(x.cu), ptr(x.mix)
                p.ld, p.hk, p.hv, p.eps = x.proj.stride(0), self.hk, self.hv, eps
                if x.snap_rel is not None:
                    p.snap_rel, p.snap_idx, p.num_snap = ptr(x.snap_rel), ptr(x.snap_idx), x.num_snap
                    p.snap_state, p.snap_conv = ptr(x.snap_state[ig]), ptr(x.snap_conv[ig])
                self._flush()
                if x.ck is not None:
                    # prefill: chunk-parallel gated delta rule on the tensor cores
                    cp = GdnChunkParams()
                    for f in ("proj", "conv_w", "neg_a_exp", "dt_bias", "norm_w", "state", "conv_state", "slots", "cu",
                              "out", "snap_rel", "snap_idx", "snap_state", "snap_conv", "ld", "hk", "hv", "num_snap", "eps"):
                        setattr(cp, f, getattr(p, f))
                    cp.ck_seq, cp.ck_tok0, cp.ck_ntok, cp.ck_snap = ptr(x.ck[0]), ptr(x.ck[1]), ptr(x.ck[2]), ptr(x.ck[3])
                    cp.seq_ck, cp.nc = ptr(x.seq_ck), x.ck.shape[1]
                    ws = self.gdn_ws.get(cp.nc * self.hv, self.dk, self.dv)
                    cp.wf, cp.qf, cp.mf, cp.kf, cp.u, cp.gamma = (ptr(b) for b in ws)
                    F.gdn_chunked(cp, S, T, self.dk, self.dv, self.state_bf16)
                    self._launches += 4
                else:
                    F.gdn_step(p, S, self.dk, self.dv, self.state_bf16, split=self.gdn_split and T > S, single=T == S)
                    self._launches += 1
                # the kernel writes [T, hv*dv] densely
                mix = x.mix.view(-1)[:T * self.hv * self.dv].view(T, self.hv * self.dv)
                self._rowpar(L.out, mix, cur, nxt, T)
                ig += 1
            else:
                self._gemv(L.qkv, cur, x.proj, T, xmode=XNORM, epi=EPI_STORE, norm_w=L.input_norm)
                q = QkvPrepParams()
                q.proj, q.q_norm, q.k_norm = ptr(x.proj), ptr(L.q_norm), ptr(L.k_norm)
                q.positions, q.slot_mapping, q.q_out = ptr(x.positions), ptr(x.slot_mapping), ptr(x.qbuf)
                q.kcache, q.vcache = ptr(self.kv[ia, 0]), ptr(self.kv[ia, 1])
                q.ld, q.hq, q.hkv, q.rotary_dim = x.proj.stride(0), self.hq, self.hkv, c.rotary_dim
                q.eps, q.log2_theta, q.num_blocks = eps, math.log2(c.rope_theta), self.num_blocks
                self._flush()
                F.qkv_prep(q, T, self.D)
                a = AttnParams()
                a.q, a.kcache, a.vcache = ptr(x.qbuf), ptr(self.kv[ia, 0]), ptr(self.kv[ia, 1])
                a.block_tables, a.positions = ptr(x.block_tables), ptr(x.positions)
                a.qg_seq, a.qg_tok0, a.qg_ntok = ptr(x.qg[0]), ptr(x.qg[1]), ptr(x.qg[2])
                a.o_part, a.ml_part, a.gate_src = ptr(x.o_part), ptr(x.ml_part), ptr(x.proj)
                mix = x.mix.view(-1)[:T * self.hq * self.D].view(T, self.hq * self.D)
                a.out = ptr(mix)
                a.hq, a.hkv, a.max_blocks, a.nsplit = self.hq, self.hkv, x.max_blocks, x.nsplit
                a.ld, a.num_qg = x.proj.stride(0), x.num_qg
                a.scale_log2e, a.num_blocks = self.D ** -0.5 * 1.4426950408889634, self.num_blocks
                F.attn_paged(a, self.D)
                self._launches += 3 if x.num_qg else 1
                if x.tiles is not None:
                    # sequences with many tokens in this step: 128-row query tiles on the tcgen05 tensor cores
                    F.attn_prefill(x.qbuf, self.kv[ia, 0], self.kv[ia, 1], self.num_blocks, x.block_tables, x.positions,
                                   x.tiles, x.proj, mix, hq=self.hq, hkv=self.hkv, D=self.D, max_blocks=x.max_blocks,
                                   ld=x.proj.stride(0))
                    self._launches += 1
                self._rowpar(L.o, mix, cur, nxt, T)
                ia += 1
            cur, nxt = nxt, cur
            nvtx_mark(f"layer {li} mlp")
            self._gemv(L.gate_up, cur, x.act, T, xmode=XNORM, epi=EPI_SWIGLU, norm_w=L.post_norm)
            self._rowpar(L.down, x.act, cur, nxt, T)
            cur, nxt = nxt, cur
        self._flush()
        self._ar_flush()
        nvtx_end()
        return cur


class _RunMixin:
    # ------------------------------------------------------------------ helpers
    def _tokens_per_group(self) -> int:
        return 2 if (self.hq // self.hkv) * 2 <= 16 else 1

    def _topk_geometry(self, k: int):
        V = self.v_local
        max_chunks = min(128, 8192 // k)
        cs = -(-V // max_chunks)
        cs = max(256, -(-cs // 256) * 256)
        assert cs <= 4096, "vocabulary shard too large for the top-k kernel"
        return -(-V // cs), cs

    def _make_topk(self, logits, n, k, order=65000, per_cta=False):
        chunks, cs = self._topk_geometry(k)
        if per_cta:                      # candidates come from the arg-max epilogue of the GEMV: one per row and CTA
            chunks, cs = F.NUM_SMS, 0
        dev = self.dev
        t = _Ctx()
        t.ws_val = torch.empty(n * chunks * k, dtype=torch.float32, device=dev)
        t.ws_idx = torch.empty(n * chunks * k, dtype=torch.int32, device=dev)
        t.out_val = torch.empty(n, self.tp * k if self.peer is not None else k, dtype=torch.float32, device=dev)
        t.out_idx = torch.empty_like(t.out_val, dtype=torch.int32)
        p = TopkParams()
        p.logits, p.ws_val, p.ws_idx, p.out_val, p.out_idx = ptr(logits), ptr(t.ws_val), ptr(t.ws_idx), ptr(t.out_val), ptr(t.out_idx)
        p.M, p.V, p.ld, p.k, p.chunks, p.chunk_size = n, self.v_local, 0 if logits is None else logits.stride(0), k, chunks, cs
        p.vocab_start = self.vocab_start
        p.tp, p.rank, p.order, p.m_cap = 1, 0, order, 0
        if self.peer is not None:
            p.tp, p.rank, p.m_cap = self.tp, self.rank, self.peer.m_cap
            for r in range(self.tp):
                p.peer_buf[r] = self.peer.cand_ptrs[r]
            p.step_ptr, p.status, p.timeout_ns = self.peer.step_ptr, self.peer.status_ptr, self.peer.timeout_ns
        t.params = p
        return t

    def _lm_head(self, hidden, logits, n):
        self._gemv(self.lm_head, hidden, logits, n, xmode=XNORM, epi=EPI_F32, norm_w=self.final_norm)
        self._flush()

    def _lm_head_argmax(self, hidden, t, n):
        """Greedy rows, no logit edits: the lm_head GEMV keeps the best column of every row per CTA in its epilogue
        (no [n, V] logits in memory, no first selection pass); the merge kernel picks the winner and exchanges it."""
        self._gemv(self.lm_head, hidden, t.ws_val.view(n, -1), n, xmode=XNORM, epi=EPI_ARGMAX, norm_w=self.final_norm,
                   out_idx=t.ws_idx.view(n, -1))
        self._flush()
        F.topk_merge(t.params)
        self._launches += 1

    def fused_argmax_ok(self, n: int, k: int) -> bool:
        return k == 1 and n <= min(self.gemm_min_rows, F.max_rows(self.lm_head.wt, XNORM, self.lm_head.K)) \
            and os.environ.get("TI_FUSED_ARGMAX", "1") != "0"

    def _topk_rows(self, logits, n, k):
        """Per-rank top-k (+ fused candidate exchange); rows in chunks of the peer buffer capacity."""
        cap = self.peer.m_cap if self.peer is not None else n
        outs = []
        for ci, m0 in enumerate(range(0, n, cap)):
            m = min(cap, n - m0)
            t = self._make_topk(logits[m0:m0 + m], m, k, order=65000 + ci)
            F.topk(t.params)
            self._launches += 2
            outs.append(t)
        return torch.cat([t.out_val for t in outs]), torch.cat([t.out_idx for t in outs])

    # ------------------------------------------------------------------ eager variable-length step
    PREFILL_ATTN_MIN_TOKENS = 16      # sequences with at least this many tokens in a step use the tcgen05 attention

    def _fill_ctx(self, x: _Ctx, batch, host=None):
        """Work lists of the two attention kernels: query groups of one or two tokens for the split-KV kernel
        (decode tokens, short chunks) and 128-token query tiles, longest context first, for the tcgen05 kernel."""
        S, T = batch.num_seqs, batch.cu_seqlens[-1]
        gt = self._tokens_per_group()
        qg_seq, qg_tok0, qg_ntok, tiles = [], [], [], []
        for s in range(S):
            t0, t1 = batch.cu_seqlens[s], batch.cu_seqlens[s + 1]
            if t1 - t0 >= self.PREFILL_ATTN_MIN_TOKENS:
                start = batch.context_lens[s] - (t1 - t0)
                for a in range(t0, t1, 128):
                    n = min(128, t1 - a)
                    tiles.append((start + (a - t0) + n, s, a, n))
                continue
            for a in range(t0, t1, gt):
                qg_seq.append(s); qg_tok0.append(a); qg_ntok.append(min(gt, t1 - a))
        tiles.sort(reverse=True)
        return qg_seq, qg_tok0, qg_ntok, tiles

    @torch.no_grad()
    def forward(self, batch):
        """Eager step over a flattened batch (prefill chunks and/or decode tokens).  Returns the
        residual-stream rows of the last token of every sequence [S, H] (the final norm is fused
        into the lm_head kernel)."""
        dev = self.dev
        S, T = batch.num_seqs, batch.cu_seqlens[-1]
        qg_seq, qg_tok0, qg_ntok, tiles = self._fill_ctx(None, batch)
        nq = len(qg_seq)
        max_blocks = max(len(b) for b in batch.block_tables)
        nsplit = 1 if nq * self.hkv >= F.NUM_SMS else max(1, min(32, -(-8 * F.NUM_SMS // (max(nq, 1) * self.hkv))))
        x = self._alloc_ctx(T, S, max_blocks, nq, nsplit)
        x.ids.copy_(batch.input_ids, non_blocking=True)
        x.positions.copy_(batch.positions.to(torch.int32), non_blocking=True)
        x.slot_mapping.copy_(batch.slot_mapping, non_blocking=True)
        x.slots.copy_(torch.tensor(batch.state_slots, dtype=torch.int32), non_blocking=True)
        x.cu = torch.tensor(batch.cu_seqlens, dtype=torch.int32, device=dev)
        bt = torch.zeros(S, max_blocks, dtype=torch.int32)
        for s, b in enumerate(batch.block_tables):
            bt[s, :len(b)] = torch.tensor(b, dtype=torch.int32)
        x.block_tables.copy_(bt, non_blocking=True)
        if nq:
            x.qg.copy_(torch.tensor([qg_seq, qg_tok0, qg_ntok], dtype=torch.int32), non_blocking=True)
        if tiles and self.cfg.num_attn_layers:
            x.tiles = torch.tensor([[t[1] for t in tiles], [t[2] for t in tiles], [t[3] for t in tiles]],
                                   dtype=torch.int32).to(dev, non_blocking=True)
        snaps = []
        if batch.snapshot_at and any(batch.snapshot_at):
            ns = max(len(p) for p in batch.snapshot_at)
            rel = torch.zeros(S, ns, dtype=torch.int32)
            idx = torch.zeros(S, ns, dtype=torch.int32)
            for s, pts in enumerate(batch.snapshot_at):
                start = batch.context_lens[s] - (batch.cu_seqlens[s + 1] - batch.cu_seqlens[s])
                for j, a in enumerate(pts):
                    rel[s, j] = a - start
                    idx[s, j] = len(snaps)               # entry of the (compact) snapshot buffers
                    snaps.append((s, j, a))
            ng = max(self.cfg.num_gdn_layers, 1)
            x.snap_rel, x.snap_idx, x.num_snap = rel.to(dev), idx.to(dev), ns
            x.snap_state = torch.empty(ng, len(snaps), self.hv, self.dk, self.dv, dtype=torch.float32, device=dev)
            x.snap_conv = torch.empty(ng, len(snaps), self.hv, 3, self.nch, dtype=BF16, device=dev)
        lens = [b - a for a, b in zip(batch.cu_seqlens[:-1], batch.cu_seqlens[1:])]
        if self.cfg.num_gdn_layers and self.gdn_chunk_min_tokens > 0 and max(lens) >= self.gdn_chunk_min_tokens:
            rel_l = ent_l = None
            if snaps:
                rel_l, ent_l = rel.tolist(), idx.tolist()
            ck, seq_ck = F.gdn_chunk_table(batch.cu_seqlens, rel_l, ent_l)
            x.ck, x.seq_ck = ck.to(dev, non_blocking=True), seq_ck.to(dev, non_blocking=True)
        cur = self._run_layers(x)
        last = torch.tensor([c - 1 for c in batch.cu_seqlens[1:]], dtype=torch.long, device=dev)
        hidden = cur[last]
        # snapshots stay on the device (a 27B snapshot is 151 MB; 64 of them are 5 % of a B200's memory)
        for k, (s, j, a) in enumerate(snaps):
            self.snapshots[(s, a)] = (x.snap_state[:, k].clone(), x.snap_conv[:, k].clone())
        self.host_steps += 1
        return hidden

    @torch.no_grad()
    def logits(self, hidden) -> torch.Tensor:
        n = hidden.shape[0]
        hidden = hidden.contiguous()
        out = torch.empty(n, self.v_local, dtype=torch.float32, device=self.dev)
        self._lm_head(hidden, out, n)
        return out

    # ------------------------------------------------------------------ CUDA-graph decode
    def capture_decode_graphs(self, max_num_seqs, max_graph_bs, max_model_len, padding_slot):
        self.padding_slot = padding_slot
        self.graph_max_blocks = max_model_len // 16 + 2
        top = min(max_num_seqs, max_graph_bs)
        if self.peer is not None:
            top = min(top, self.peer.m_cap)      # one candidate exchange per step covers m_cap rows
        self.buckets = []
        b = 1
        while b < top:
            self.buckets.append(b)
            b *= 2
        self.buckets.append(top)
        self.graph_pool = None
        for b in self.buckets:
            self._get_graph(b, 1, self.fused_argmax_ok(b, 1))

    def release_graphs(self):
        """Drop every captured decode graph (and the reference to the one replayed last).  Graphs that captured NCCL
        collectives (the non-fused tensor-parallel path) must be gone before the process group is destroyed: NCCL
        waits for them."""
        self.graphs.clear()
        self._last_graph = None
        gc.collect()

    def decode_graph(self, n: int, k: int = 1, edits: bool = False):
        """The captured decode step that serves `n` sequences with `k` candidates (captured on first use)."""
        B = next(b for b in self.buckets if b >= n)
        k = 1 if k <= 1 else 64
        return self._get_graph(B, k, not edits and self.fused_argmax_ok(B, k))

    def _get_graph(self, B: int, k: int, fa: bool = False):
        """fa: the lm_head product keeps only each CTA's arg-max (greedy rows without logit edits)."""
        key = (B, k, fa)
        g = self.graphs.get(key)
        if g is not None:
            return g
        dev = self.dev
        nsplit = max(1, min(32, -(-8 * F.NUM_SMS // (B * self.hkv))))
        base = next((v for kk, v in self.graphs.items() if kk[0] == B), None)
        g = _Ctx()
        if base is not None:      # same bucket, other k: share the input tensors
            g.x = base.x
            g.host = base.host
        else:
            g.x = self._alloc_ctx(B, B, self.graph_max_blocks, B, nsplit)
            x = g.x
            g.host = {
                "ids": torch.zeros(B, dtype=torch.long).pin_memory(),
                "positions": torch.zeros(B, dtype=torch.int32).pin_memory(),
                "slot_mapping": torch.full((B,), -1, dtype=torch.long).pin_memory(),
                "slots": torch.full((B,), self.padding_slot, dtype=torch.int32).pin_memory(),
                "block_tables": torch.zeros(B, self.graph_max_blocks, dtype=torch.int32).pin_memory(),
                "qg": torch.zeros(3, B, dtype=torch.int32).pin_memory(),
            }
            x.slots.fill_(self.padding_slot)
        x = g.x
        g.logits = None if fa else torch.zeros(B, self.v_local, dtype=torch.float32, device=dev)
        g.topk = self._make_topk(g.logits, B, k, per_cta=fa)
        g.k = k
        g.samp = self._make_sampler_state(g.logits if not fa else g.topk.out_val, B, g.topk)
        fused_sample = self.tp == 1 or self.peer is not None

        def body():
            cur = self._run_layers(x)
            if fa:
                self._lm_head_argmax(cur, g.topk, B)
            else:
                self._lm_head(cur, g.logits, B)
                F.logits_edit(g.samp.edit)             # rows without an edit slot leave at once
                F.topk(g.topk.params)
                self._launches += 3
            if fused_sample:
                F.sample(g.samp.sample)
                self._launches += 1

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            body()                                   # warm-up (padding inputs touch only the padding slot)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self.comm is not None:
            self.comm.barrier()
        self._launches = 0
        g.graph = torch.cuda.CUDAGraph()
        # objects of an earlier engine (old graphs, tensors) must not be finalised while the stream
        # captures: collect them now and keep the collector off until the capture ends
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g.graph, pool=self.graph_pool):
                body()
        finally:
            if gc_was_on:
                gc.enable()
        g.launches = self._launches
        self.launches_per_decode_step = g.launches
        if self.graph_pool is None:
            self.graph_pool = g.graph.pool()
        self.graphs[key] = g
        return g

    # ------------------------------------------------------------------ sampling on the device
    EDIT_SLOTS = 8          # rows of a step that may carry logit edits (penalty, bias, masks, grammar)
    PEN_CAP = 8192          # penalised token ids per row

    def _edit_buffers(self):
        """Device buffers of the logit-edit kernel, shared by all graphs and eager steps (stable addresses)."""
        e = getattr(self, "_edit", None)
        if e is None:
            dev, R = self.dev, self.EDIT_SLOTS
            e = self._edit = _Ctx()
            e.add_rows = torch.zeros(R, self.v_local, dtype=torch.float32, device=dev)
            e.meta = torch.zeros(3, R, dtype=torch.int32, device=dev)          # add_valid | pen_cnt | pen_rp (float bits)
            e.pen_ids = torch.zeros(R, self.PEN_CAP, dtype=torch.int32, device=dev)
            e.h_meta = torch.zeros(3, R, dtype=torch.int32).pin_memory()
            e.h_pen = torch.zeros(R, self.PEN_CAP, dtype=torch.int32).pin_memory()
            e.h_add = torch.zeros(R, self.v_local, dtype=torch.float32).pin_memory()
        return e

    def _make_sampler_state(self, logits, n, topk_state):
        """Parameter blocks of the edit and sample kernels for `n` rows whose candidates `topk_state` produces."""
        dev, e = self.dev, self._edit_buffers()
        t = _Ctx()
        t.fpar = torch.zeros(3, n, dtype=torch.float32, device=dev)            # temperature | top_p | u
        t.ipar = torch.full((2, n), -1, dtype=torch.int32, device=dev)         # top_k | edit slot
        t.h_fpar = torch.zeros(3, n, dtype=torch.float32).pin_memory()
        t.h_ipar = torch.full((2, n), -1, dtype=torch.int32).pin_memory()
        t.tok = torch.zeros(n + 1, dtype=torch.int32, device=dev)
        t.h_tok = torch.zeros(n + 1, dtype=torch.int32).pin_memory()
        ep = EditParams()
        ep.logits, ep.row_slot, ep.add_rows = ptr(logits), ptr(t.ipar[1]), ptr(e.add_rows)
        ep.add_valid, ep.pen_cnt, ep.pen_rp, ep.pen_ids = ptr(e.meta[0]), ptr(e.meta[1]), ptr(e.meta[2]), ptr(e.pen_ids)
        ep.M, ep.V, ep.ld, ep.pen_cap, ep.chunk = n, self.v_local, logits.stride(0), self.PEN_CAP, 8192
        t.edit = ep
        sp = SampleParams()
        sp.cand_val, sp.cand_idx = ptr(topk_state.out_val), ptr(topk_state.out_idx)
        sp.temperature, sp.top_p, sp.u, sp.top_k = ptr(t.fpar[0]), ptr(t.fpar[1]), ptr(t.fpar[2]), ptr(t.ipar[0])
        sp.out_tok, sp.status_src = ptr(t.tok), self.ctrl.data_ptr() + 4
        sp.M, sp.n_cand = n, topk_state.out_val.shape[1]
        t.sample = sp
        return t

    def _upload_sampling(self, t, n, spec):
        """Host -> device copies of a step's sampling parameters and logit edits (pinned staging, asynchronous)."""
        hf, hi = t.h_fpar, t.h_ipar
        hf[0].zero_()                                   # padding rows: greedy
        hi[1].fill_(-1)
        hf[0, :n] = torch.tensor(spec["temperature"], dtype=torch.float32)
        hf[1, :n] = torch.tensor(spec["top_p"], dtype=torch.float32)
        hf[2, :n] = torch.tensor(spec["u"], dtype=torch.float32)
        hi[0, :n] = torch.tensor(spec["top_k"], dtype=torch.int32)
        edits = spec.get("edits") or []
        if edits:
            e = self._edit_buffers()
            assert len(edits) <= self.EDIT_SLOTS
            for slot, (row, add, pen, rp) in enumerate(edits):
                hi[1, row] = slot
                e.h_meta[0, slot] = 0 if add is None else 1
                if add is not None:
                    e.h_add[slot].copy_(add)
                    e.add_rows[slot].copy_(e.h_add[slot], non_blocking=True)
                cnt = 0 if pen is None else min(len(pen), self.PEN_CAP)
                e.h_meta[1, slot] = cnt
                e.h_meta[2, slot] = torch.tensor([float(rp)], dtype=torch.float32).view(torch.int32)[0]
                if cnt:
                    e.h_pen[slot, :cnt] = pen[:cnt]
                    e.pen_ids[slot, :cnt].copy_(e.h_pen[slot, :cnt], non_blocking=True)
            e.meta.copy_(e.h_meta, non_blocking=True)
        t.fpar.copy_(hf, non_blocking=True)
        t.ipar.copy_(hi, non_blocking=True)

    def _read_tokens(self, t, n) -> list:
        """The step's only device -> host copy: n token ids and the communicator's status word."""
        t.h_tok.copy_(t.tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        status = int(t.h_tok[t.tok.shape[0] - 1])
        if status != 0:
            # a bounded device wait ran out (a peer's flag or packet, an mbarrier) or a checked index was out of range:
            # whatever the kernels computed after that is not to be trusted, on one GPU as on eight
            from ..parallel.watchdog import PeerLostError
            err = PeerLostError([])
            err.args = (f"device status word {status:#x}: a bounded wait ran out"
                        f"{' on a tensor-parallel peer' if self.peer is not None else ''} or an index check failed; "
                        "the tokens of this step are discarded",)
            raise err
        return t.h_tok[:n].tolist()

    def _decode_graph_step(self, batch, k: int, spec=None):
        n = batch.num_seqs
        g = self.decode_graph(n, k, edits=bool(spec and spec.get("edits")))
        self._last_graph = g
        h, x = g.host, g.x
        h["ids"][:n] = batch.input_ids
        h["positions"][:n] = batch.positions
        h["slot_mapping"][:n] = batch.slot_mapping
        h["slot_mapping"][n:] = -1
        h["slots"][:n] = torch.tensor(batch.state_slots, dtype=torch.int32)
        h["slots"][n:] = self.padding_slot
        bt = h["block_tables"]
        for s, b in enumerate(batch.block_tables):
            bt[s, :len(b)] = torch.tensor(b, dtype=torch.int32)
        qg = h["qg"]
        qg[0, :n] = torch.arange(n, dtype=torch.int32)
        qg[1, :n] = torch.arange(n, dtype=torch.int32)
        qg[2, :n] = 1
        qg[2, n:] = 0
        x.ids.copy_(h["ids"], non_blocking=True)
        x.positions.copy_(h["positions"], non_blocking=True)
        x.slot_mapping.copy_(h["slot_mapping"], non_blocking=True)
        x.slots.copy_(h["slots"], non_blocking=True)
        x.block_tables.copy_(bt, non_blocking=True)
        x.qg.copy_(qg, non_blocking=True)
        if spec is not None:
            self._upload_sampling(g.samp, n, spec)
        if self.peer is not None:
            self.peer.tick()
        g.graph.replay()
        self.host_steps += 1
        return g.topk.out_val[:n], g.topk.out_idx[:n]

    def _default_spec(self, n):
        return {"temperature": [0.0] * n, "top_k": [1] * n, "top_p": [1.0] * n, "u": [0.0] * n, "edits": []}

    @torch.no_grad()
    def forward_and_sample(self, batch, sample_rows, k: int, spec=None):
        """Runs the step and samples on the device.  Returns one token id per sampling row (a list of ints; the
        same on every tensor-parallel rank).  `spec`: per-row temperature / top_k / top_p / u lists and `edits`,
        a list of (row, additive logit row or None, sorted penalised local ids or None, penalty).  The step's only
        device -> host copy is the token ids plus the peer status word; a non-zero status raises PeerLostError."""
        assert k <= 64, "more than 64 candidates: use forward() + logits() + the host sampler"
        k = 1 if k <= 1 else 64
        n = len(sample_rows)
        if spec is None:
            spec = self._default_spec(n)
        fused = self.tp == 1 or self.peer is not None        # candidates of all ranks are on this device after top-k
        decode_only = batch.cu_seqlens[-1] == batch.num_seqs and n == batch.num_seqs
        if decode_only and self.graphs and batch.num_seqs <= self.buckets[-1] \
                and max(len(b) for b in batch.block_tables) <= self.graph_max_blocks:
            vals, idx = self._decode_graph_step(batch, k, spec)
            if fused:
                return self._read_tokens(self._last_graph.samp, n)
        else:
            hidden = self.forward(batch)
            rows = torch.tensor(sample_rows, dtype=torch.long, device=self.dev)
            lg = self.logits(hidden[rows])
            if spec.get("edits"):
                t0 = _Ctx()
                t0.out_val = t0.out_idx = torch.empty(n, 1, device=self.dev)
                st = self._make_sampler_state(lg, n, t0)
                self._upload_sampling(st, n, spec)
                F.logits_edit(st.edit)
                self._launches += 1
            vals, idx = self._topk_rows(lg, n, k)
        if not fused:
            vals = torch.cat(self.comm.all_gather(vals.contiguous()), dim=-1)
            idx = torch.cat(self.comm.all_gather(idx.contiguous()), dim=-1)
        t1 = _Ctx()
        t1.out_val, t1.out_idx = vals.contiguous(), idx.contiguous()
        st = self._make_sampler_state(t1.out_val, n, t1)
        spec = dict(spec, edits=[])                    # edits were applied before the top-k
        self._upload_sampling(st, n, spec)
        F.sample(st.sample)
        self._launches += 1
        return self._read_tokens(st, n)

    def peer_status(self) -> int:
        return int(self.ctrl[1].item())


class B200HybridModel(_ModelBase, _StepMixin, _RunMixin):
    """See the module docstring."""
