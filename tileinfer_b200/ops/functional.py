"""Tensor-level wrappers of the sm_100a kernels (torch tensors in, launches on the current stream).

Nothing here allocates unless the docstring says so; the model keeps its activations, workspaces and
parameter blocks alive, which also makes every launch capturable into a CUDA graph.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import lib as _l
from .lib import ChainParams, GemvParams, MAX_CHAIN, MAX_RANKS, check, ptr, stream

_I, _P, _F = ctypes.c_int, ctypes.c_void_p, ctypes.c_float

XGLOBAL, XNORM = 0, 1
EPI_STORE, EPI_SWIGLU, EPI_ROWPAR, EPI_F32, EPI_ARGMAX = 0, 1, 2, 3, 4
W_INT8, W_BF16 = 0, 1


def _device_sm_count() -> int:
    """Streaming multiprocessors of the current GPU (148 on a B200; the fallback when no GPU is visible).  The
    persistent GEMV launches one CTA per SM and its grid barrier needs every CTA resident, so the grid must follow
    the device, not a constant."""
    try:
        if torch.cuda.is_available():
            return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    except Exception:
        pass
    return 148


NUM_SMS = _device_sm_count()
GEMV_WARPS = int(os.environ.get("TI_GEMV_WARPS", "16"))   # must match the -DTI_GEMV_WARPS the library was built with
GEMV_TPS = int(os.environ.get("TI_GEMV_TPS", "8"))            # 512-byte tiles per ring stage
GEMV_MAX_STAGES = int(os.environ.get("TI_GEMV_STAGES", "6"))
GEMV_UNITS_PER_WARP = int(os.environ.get("TI_GEMV_UPW", "4"))


class GdnParams(ctypes.Structure):
    _fields_ = [("proj", _P), ("conv_w", _P), ("neg_a_exp", _P), ("dt_bias", _P), ("norm_w", _P), ("state", _P),
                ("conv_state", _P), ("slots", _P), ("cu", _P), ("out", _P), ("snap_rel", _P), ("snap_state", _P),
                ("snap_conv", _P), ("ld", _I), ("hk", _I), ("hv", _I), ("num_snap", _I), ("eps", _F), ("snap_idx", _P), ("status", _P)]


class GdnChunkParams(ctypes.Structure):
    _fields_ = [("proj", _P), ("conv_w", _P), ("neg_a_exp", _P), ("dt_bias", _P), ("norm_w", _P), ("state", _P),
                ("conv_state", _P), ("slots", _P), ("cu", _P), ("out", _P), ("snap_rel", _P), ("snap_idx", _P),
                ("snap_state", _P), ("snap_conv", _P), ("ck_seq", _P), ("ck_tok0", _P), ("ck_ntok", _P), ("ck_snap", _P),
                ("seq_ck", _P), ("wf", _P), ("qf", _P), ("mf", _P), ("kf", _P), ("u", _P), ("gamma", _P),
                ("ld", _I), ("hk", _I), ("hv", _I), ("num_snap", _I), ("nc", _I), ("eps", _F)]


class QkvPrepParams(ctypes.Structure):
    _fields_ = [("proj", _P), ("q_norm", _P), ("k_norm", _P), ("positions", _P), ("slot_mapping", _P),
                ("q_out", _P), ("kcache", _P), ("vcache", _P), ("ld", _I), ("hq", _I), ("hkv", _I),
                ("rotary_dim", _I), ("eps", _F), ("log2_theta", _F), ("num_blocks", _I), ("status", _P)]


class AttnParams(ctypes.Structure):
    _fields_ = [("q", _P), ("kcache", _P), ("vcache", _P), ("block_tables", _P), ("positions", _P),
                ("qg_seq", _P), ("qg_tok0", _P), ("qg_ntok", _P), ("o_part", _P), ("ml_part", _P),
                ("gate_src", _P), ("out", _P), ("hq", _I), ("hkv", _I), ("max_blocks", _I), ("nsplit", _I),
                ("ld", _I), ("num_qg", _I), ("scale_log2e", _F), ("num_blocks", _I), ("status", _P)]


class TopkParams(ctypes.Structure):
    _fields_ = [("logits", _P), ("ws_val", _P), ("ws_idx", _P), ("out_val", _P), ("out_idx", _P),
                ("step_ptr", _P), ("status", _P), ("peer_buf", ctypes.c_uint64 * MAX_RANKS),
                ("timeout_ns", ctypes.c_ulonglong),
                ("M", _I), ("V", _I), ("ld", _I), ("k", _I), ("chunks", _I), ("chunk_size", _I),
                ("vocab_start", _I), ("tp", _I), ("rank", _I), ("order", _I), ("m_cap", _I)]


class ArRowsParams(ctypes.Structure):
    _fields_ = [("part_peer", ctypes.c_uint64 * MAX_RANKS), ("part_mc", ctypes.c_uint64),
                ("flag_peer", ctypes.c_uint64 * MAX_RANKS), ("resid", _P), ("h_out", _P), ("norm_w", _P), ("xh", _P),
                ("xl", _P), ("xscale", _P), ("xn", _P), ("step_ptr", _P), ("status", _P),
                ("timeout_ns", ctypes.c_ulonglong), ("M", _I), ("N", _I), ("tp", _I), ("rank", _I), ("order", _I),
                ("mode", _I), ("eps", _F), ("rows_cap", _I), ("two_shot", _I)]


class EditParams(ctypes.Structure):
    _fields_ = [("logits", _P), ("row_slot", _P), ("add_rows", _P), ("add_valid", _P), ("pen_ids", _P), ("pen_cnt", _P),
                ("pen_rp", _P), ("M", _I), ("V", _I), ("ld", _I), ("pen_cap", _I), ("chunk", _I)]


class SampleParams(ctypes.Structure):
    _fields_ = [("cand_val", _P), ("cand_idx", _P), ("temperature", _P), ("top_k", _P), ("top_p", _P), ("u", _P),
                ("out_tok", _P), ("status_src", _P), ("M", _I), ("n_cand", _I)]


_l.register("ti_ar_rows_params_size", _I, [])
_l.register("ti_ar_rows", _I, [ctypes.POINTER(ArRowsParams), _P])
_l.register("ti_edit_params_size", _I, [])
_l.register("ti_sample_params_size", _I, [])
_l.register("ti_logits_edit", _I, [ctypes.POINTER(EditParams), _P])
_l.register("ti_sample", _I, [ctypes.POINTER(SampleParams), _P])
_l.register("ti_embed", _I, [_P, _P, _P, _I, _I, _I, _P, _P])
_l.register("ti_rmsnorm", _I, [_P, _P, _P, _P, _P, _I, _I, _F, _I, _P])
_l.register("ti_act_mul", _I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P])
_l.register("ti_swiglu_interleaved", _I, [_P, _P, _I, _I, _I, _I, _P])
_l.register("ti_gdn_params_size", _I, [])
_l.register("ti_gdn_step", _I, [ctypes.POINTER(GdnParams), _I, _I, _I, _I, _I, _P])
_l.register("ti_gdn_chunk_params_size", _I, [])
_l.register("ti_gdn_chunk_ws_bytes", _I, [_I, _I, _I])
_l.register("ti_gdn_chunked", _I, [ctypes.POINTER(GdnChunkParams), _I, _I, _I, _I, _I, _P])
_l.register("ti_qkv_prep_params_size", _I, [])
_l.register("ti_attn_params_size", _I, [])
_l.register("ti_qkv_prep", _I, [ctypes.POINTER(QkvPrepParams), _I, _I, _P])
_l.register("ti_attn_paged", _I, [ctypes.POINTER(AttnParams), _I, _P])
_l.register("ti_attn_prefill", _I, [_P, _I, _P, _P, _I, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P])
_l.register("ti_topk_params_size", _I, [])
_l.register("ti_topk", _I, [ctypes.POINTER(TopkParams), _P])
_l.register("ti_topk_merge", _I, [ctypes.POINTER(TopkParams), _P])
_l.register("ti_symm_alloc", _I, [ctypes.POINTER(_P), ctypes.c_size_t])
_l.register("ti_symm_free", _I, [_P])
_l.register("ti_ipc_handle_size", _I, [])
_l.register("ti_ipc_get_handle", _I, [_P, _P])
_l.register("ti_ipc_open", _I, [_P, ctypes.POINTER(_P)])
_l.register("ti_ipc_close", _I, [_P])
_l.register("ti_memset_async", _I, [_P, _I, ctypes.c_size_t, _P])
_l.register("ti_wait_flag_probe", _I, [_P, ctypes.c_uint, ctypes.c_ulonglong, _P, _P, _P])

_l.register("ti_quant_rows", _I, [_P, _I, _P, _F, _I, _I, _P, _P, _P, _P])
_l.register("ti_gemm_bf16", _I, [_P, _I, _I, _I, _P, _I, _P, _P, _I, _I, _P, _P, ctypes.c_size_t, _P, _I, _P])
_l.register("ti_gemm_w8a16", _I, [_P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _I, _I, _P, _P, ctypes.c_size_t, _P, _I, _P])

_checked = False


def L():
    global _checked
    lib = _l.lib()
    if not _checked:
        for fn, st in (("ti_gdn_params_size", GdnParams), ("ti_gdn_chunk_params_size", GdnChunkParams), ("ti_qkv_prep_params_size", QkvPrepParams),
                       ("ti_attn_params_size", AttnParams), ("ti_topk_params_size", TopkParams),
                       ("ti_edit_params_size", EditParams), ("ti_sample_params_size", SampleParams),
                       ("ti_ar_rows_params_size", ArRowsParams)):
            if getattr(lib, fn)() != ctypes.sizeof(st):
                raise RuntimeError(f"{st.__name__} layout mismatch between Python and CUDA")
        _checked = True
    return lib


# ------------------------------------------------------------------------------------ GEMV
class LinearW:
    """A weight matrix in kernel layout: 512-byte tiles [N/8][K/64 or K/32][8][64 B] (+ bf16 row scales)."""

    def __init__(self, w: torch.Tensor, quantize: bool, device="cuda"):
        from ..models.weights import pad_rows, quantize_int8_rowwise, tile_bf16, tile_int8
        self.N, self.K = w.shape
        w = pad_rows(w.to(device), 8)
        self.n_pad = w.shape[0]
        if quantize:
            assert self.K % 64 == 0, self.K
            q, s = quantize_int8_rowwise(w)
            self.tiles = tile_int8(q)
            self.scale = s.contiguous()
            self.wt, self.tile_k = W_INT8, 64
        else:
            assert self.K % 32 == 0, self.K
            self.tiles = tile_bf16(w.to(torch.bfloat16))
            self.scale = None
            self.wt, self.tile_k = W_BF16, 32
        self.KB = self.K // self.tile_k
        self.n_tiles = self.n_pad // 8

    def state(self) -> dict:
        """Everything needed to rebuild this object without the source weight (on-disk shard cache)."""
        return {"tiles": self.tiles, "scale": self.scale, "N": self.N, "K": self.K, "n_pad": self.n_pad, "wt": self.wt}

    @classmethod
    def from_state(cls, d: dict, device="cuda") -> "LinearW":
        w = cls.__new__(cls)
        w.N, w.K, w.n_pad, w.wt = d["N"], d["K"], d["n_pad"], d["wt"]
        w.tiles = d["tiles"].to(device)
        w.scale = None if d["scale"] is None else d["scale"].to(device)
        w.tile_k = 64 if w.wt == W_INT8 else 32
        w.KB = w.K // w.tile_k
        w.n_tiles = w.n_pad // 8
        return w

    def dense(self) -> torch.Tensor:
        """Row-major bf16 copy [N, K] (tests and the prefill GEMM baseline)."""
        from ..models.weights import untile_int8
        if self.wt == W_INT8:
            return (untile_int8(self.tiles).float() * self.scale.float()[:, None])[:self.N].to(torch.bfloat16)
        nt, kt = self.tiles.shape[:2]
        return self.tiles.permute(0, 2, 1, 3).reshape(nt * 8, kt * 32)[:self.N]

    def nbytes(self) -> int:
        return self.tiles.numel() * self.tiles.element_size()


def _limb_stride(kslice: int) -> int:
    return kslice + ((64 - (kslice % 128)) + 128) % 128


def x_smem_bytes(wt: int, xmode: int, M: int, K: int, kslice: int) -> int:
    """Shared memory the staged activations take (must mirror x_smem_bytes_impl in gemv_w8a16.cu)."""
    b = 0
    if wt == W_INT8:
        b = 2 * M * _limb_stride(kslice)
    elif xmode == XNORM:
        b = (16 if M > 8 else 8) * (K + 8) * 2
    return (b + 2048 + 127) // 128 * 128


PART_BYTES = 0
SMEM_LIMIT = 227 * 1024 - 4096      # dynamic shared memory of the GEMV kernel (4 KB of the 227 are static)
GEMV_TPS = int(os.environ.get("TI_GEMV_TPS", "8"))       # must match the -DTI_GEMV_TPS the library was built with
_RING_CHOICES = tuple((GEMV_TPS, s) for s in range(48 // GEMV_TPS, 0, -1))


def plan_gemv(wt: int, xmode: int, M: int, n_tiles: int, KB: int, ncta: int = NUM_SMS):
    """(R, tps, stages) or None when M rows of this K do not fit in shared memory.
    R: row tiles per unit; (tps, stages): geometry of the per-warp weight ring that fits beside the staged
    activations and the partial-sum buffers in 227 KB."""
    tk = 64 if wt == W_INT8 else 32
    xb = x_smem_bytes(wt, xmode, M, KB * tk, KB * tk)
    R = 2 if n_tiles >= 8 * ncta * GEMV_WARPS else 1
    for tps, stages in _RING_CHOICES:
        if xb + PART_BYTES + GEMV_WARPS * (stages * (tps * 512 + 8) + 64) <= SMEM_LIMIT:
            return R, tps, stages
    return None


TEAM_BYTES = 2 * GEMV_WARPS * 32 * 16      # exchange buffer of team mode (must mirror kTeamBytes)


def plan_team(n_tiles: int, KB: int, R: int, team: int | None = None, ncta: int = NUM_SMS) -> int:
    """Team size T for a product: how many adjacent warps of a CTA share one unit, each streaming a slice of k.
    A product with fewer units than warps would leave warps (and the bytes they keep in flight) idle.
    `team` (or TI_GEMV_T) forces a size.

    Cost model (in 512-byte tiles a warp streams one after the other): a CTA holds GEMV_WARPS // T whole teams,
    the units are dealt to the teams in waves, a unit costs ceil(KB / T) tiles per warp plus a fixed part (team
    exchange and epilogue, about six tiles' worth).  Measured on the 27B layer at one row (chain of the four layer
    products): out_proj / down with T = 2 -> 91.4 us, T = 3 -> 87.5 us, T = 5 or 16 -> 90-95 us; the half shards
    of a 2-way tensor-parallel group 60.7 -> 58.2 us."""
    if team is None and "TI_GEMV_T" in os.environ:
        team = int(os.environ["TI_GEMV_T"])
    U = -(-n_tiles // R)
    if team is not None:
        return team if KB >= team else 1
    W = ncta * GEMV_WARPS
    if U >= 0.8 * W:
        return 1
    fixed = 6
    best, best_cost = 1, -(-U // W) * (KB + fixed)
    for T in range(2, GEMV_WARPS + 1):
        if KB < 8 * T:                       # a slice shorter than one ring stage is all overhead
            break
        teams = (GEMV_WARPS // T) * ncta
        cost = -(-U // teams) * (-(-KB // T) + fixed)
        if cost < 0.97 * best_cost:          # near-ties go to the smaller team
            best, best_cost = T, cost
    return best


def max_rows(wt: int, xmode: int, K: int) -> int:
    """Largest row count (<= 16) one launch can take for this K."""
    tk = 64 if wt == W_INT8 else 32
    for m in (16, 12, 8, 6, 4, 3, 2, 1):
        if plan_gemv(wt, xmode, m, 1024, K // tk) is not None:
            return m
    raise ValueError(f"K={K} does not fit in shared memory even for one row")


_STATUS = None


def status_ptr() -> int:
    """A process-wide device word that kernels OR error bits into when no communicator supplies one."""
    global _STATUS
    if _STATUS is None:
        _STATUS = torch.zeros(4, dtype=torch.int32, device="cuda")
    return _STATUS.data_ptr()


class GemvWorkspace:
    """Split-k partial buffer and per-tile arrival counters shared by all GEMV launches of a stream."""

    def __init__(self, device="cuda", max_units: int = 1 << 16, max_tiles: int = 1 << 16):
        self.ws = torch.empty(max_units * 128, dtype=torch.float32, device=device)
        self.counters = torch.zeros(max_tiles, dtype=torch.int32, device=device)
        self.sched = torch.zeros(128, dtype=torch.int32, device=device)     # dynamic unit scheduling state
        self.max_units, self.max_tiles = max_units, max_tiles


_DEFAULT_WS = None


def default_workspace():
    global _DEFAULT_WS
    if _DEFAULT_WS is None:
        _DEFAULT_WS = GemvWorkspace()
    return _DEFAULT_WS


def make_gemv_params(W: LinearW, x, out, M, *, xmode=XGLOBAL, epi=EPI_STORE, norm_w=None, resid=None, ws=None,
                     eps=1e-6, ldx=None, ldo=None, comm=None, order=0, ncta=NUM_SMS, team=None, xll=False,
                     out_idx=None) -> GemvParams:
    p = GemvParams()
    p.w, p.scale, p.x, p.norm_w = ptr(W.tiles), ptr(W.scale), ptr(x), ptr(norm_w)
    p.out, p.resid, p.out_idx = ptr(out), ptr(resid), ptr(out_idx)
    plan = plan_gemv(W.wt, xmode, M, W.n_tiles, W.KB, ncta)
    if plan is None:
        raise ValueError(f"{M} rows of K={W.K} do not fit in shared memory; split the rows (max_rows)")
    R, tps, stages = plan
    if ws is None:
        ws = default_workspace()
    p.M, p.N, p.n_tiles, p.K, p.KB, p.S, p.kb_per_split = M, W.N, W.n_tiles, W.K, W.KB, 1, W.KB
    p.ws = ptr(ws.ws)
    p.ldx = ldx if ldx is not None else (x.stride(0) if x.dim() > 1 else W.K)
    p.ldo = ldo if ldo is not None else (out.stride(0) if out.dim() > 1 else W.N)
    p.eps = eps
    p.stages, p.T, p.tps, p.R = stages, plan_team(W.n_tiles, W.KB, R, team, ncta), tps, R
    p._xb = x_smem_bytes(W.wt, xmode, M, W.K, W.K)
    p.xmode, p.epi = xmode, epi
    p.xll = int(bool(xll))
    if ws is None:
        ws = default_workspace()
    p.sched = ptr(ws.sched)
    p.status = status_ptr()
    p.tp, p.rank, p.order, p.m_cap = 1, 0, order, 0
    if comm is not None and comm.tp > 1:
        p.tp, p.rank, p.m_cap = comm.tp, comm.rank, comm.m_cap
        for r in range(comm.tp):
            p.peer_ll[r] = comm.ll_ptrs[r]
        p.step_ptr, p.status, p.timeout_ns = comm.step_ptr, comm.status_ptr, comm.timeout_ns
    return p


def make_chain(params: list) -> ChainParams:
    """Up to MAX_CHAIN dependent products for one launch; the ring depth is the smallest of the ops'."""
    assert 1 <= len(params) <= MAX_CHAIN
    c = ChainParams()
    c.n_ops = len(params)
    # one ring geometry per launch: the one of the op that has the least room
    tps, stages = min((p.tps * p.stages, p.tps, p.stages) for p in params)[1:]
    # team mode needs its exchange buffer next to the rings: give up ring stages for it, or, failing that, teams
    xb = max(getattr(p, "_xb", 0) for p in params)
    while any(p.T > 1 for p in params) and xb + TEAM_BYTES + GEMV_WARPS * (stages * (tps * 512 + 8) + 64) > SMEM_LIMIT:
        if stages > 1:
            stages -= 1
        else:
            for p in params:
                p.T = 1
    for i, p in enumerate(params):
        p.tps, p.stages = tps, stages
        c.op[i] = p
    return c


def gemv_chain_launch(params: list, wt: int, ncta: int = NUM_SMS):
    c = make_chain(params)
    check(L().ti_gemv_chain(ctypes.byref(c), wt, ncta, stream()), "ti_gemv_chain")


def gemv_launch(p: GemvParams, wt: int, xmode: int = None, epi: int = None, ncta: int = NUM_SMS):
    if xmode is not None:
        p.xmode = xmode
    if epi is not None:
        p.epi = epi
    gemv_chain_launch([p], wt, ncta)


def gemv(W: LinearW, x: torch.Tensor, *, out=None, xmode=XGLOBAL, epi=EPI_STORE, norm_w=None, resid=None, ws=None,
         eps=1e-6, comm=None, order=0, team=None) -> torch.Tensor:
    """Convenience form (allocates `out`); loops over row chunks that fit in shared memory."""
    M = x.shape[0]
    step = max_rows(W.wt, xmode, W.K)
    if out is None:
        cols = W.N // 2 if epi == EPI_SWIGLU else W.N
        dt = torch.float32 if epi == EPI_F32 else torch.bfloat16
        out = torch.empty(M, cols, dtype=dt, device=x.device)
    for m0 in range(0, M, step):
        m = min(step, M - m0)
        p = make_gemv_params(W, x[m0:m0 + m], out[m0:m0 + m], m, xmode=xmode, epi=epi, norm_w=norm_w,
                             resid=None if resid is None else resid[m0:m0 + m], ws=ws, eps=eps,
                             ldx=x.stride(0), ldo=out.stride(0), comm=comm, order=order, team=team)
        gemv_launch(p, W.wt, xmode, epi)
    return out


# ------------------------------------------------------------------------------------ pointwise
def embed(ids, table, out, step_ptr=0):
    M, H = out.shape
    check(L().ti_embed(ptr(ids), ptr(table), ptr(out), M, H, table.shape[0], step_ptr, stream()), "ti_embed")


def rmsnorm(x, w, eps, *, add=None, out=None, r_out=None, one_plus=True):
    M, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    check(L().ti_rmsnorm(ptr(x), ptr(add), ptr(w), ptr(out), ptr(r_out), M, H, eps, int(one_plus), stream()), "ti_rmsnorm")
    return out


def act_mul(a, b, out=None, mode=0):
    M, n = a.shape
    if out is None:
        out = torch.empty(M, n, dtype=torch.bfloat16, device=a.device)
    check(L().ti_act_mul(ptr(a), ptr(b), ptr(out), M, n, a.stride(0), b.stride(0), out.stride(0), mode, stream()), "ti_act_mul")
    return out


def swiglu_interleaved(gu, out=None):
    M, n2 = gu.shape
    if out is None:
        out = torch.empty(M, n2 // 2, dtype=torch.bfloat16, device=gu.device)
    check(L().ti_swiglu_interleaved(ptr(gu), ptr(out), M, n2 // 2, gu.stride(0), out.stride(0), stream()), "ti_swiglu")
    return out


# ------------------------------------------------------------------------------------ launches by params
def gdn_step(p: GdnParams, num_seqs: int, dk: int, dv: int, state_bf16: bool, split: bool = False, single: bool = False,
             staged: bool = False):
    """single: every sequence has exactly one token (decode): the single-pass kernels (one block per head and sequence;
    for large batches column-split blocks, or, with `staged` or when snapshots are wanted, blocks that walk several
    sequences with the state staged through shared memory).  split: the state columns of a head go to a cluster of
    blocks (prefill; optional)."""
    mode = (3 if staged else 2) if single else int(split)
    if not p.status:
        p.status = status_ptr()
    check(L().ti_gdn_step(ctypes.byref(p), num_seqs, dk, dv, int(state_bf16), mode, stream()), "ti_gdn_step")


GDN_CHUNK = 64


def gdn_chunk_table(cu_seqlens, snapshot_rel=None, snapshot_entry=None):
    """Chunk table of the chunked DeltaNet prefill: every sequence is cut into chunks of at most 64 tokens that
    also end wherever a state snapshot is wanted.  `snapshot_rel[s]`: token counts (relative to the start of the
    step) after which sequence s snapshots, `snapshot_entry[s]`: the entries of the snapshot buffers.
    Returns int32 tensors (ck [4, nc] = sequence | first flat token | tokens | snapshot entry or -1, seq_ck [S+1])."""
    seq, tok0, ntok, snap, seq_ck = [], [], [], [], [0]
    for s in range(len(cu_seqlens) - 1):
        t0, t1 = cu_seqlens[s], cu_seqlens[s + 1]
        pts = {}
        if snapshot_rel is not None:
            for r, e in zip(snapshot_rel[s], snapshot_entry[s]):
                if 0 < r <= t1 - t0:
                    pts[r] = e
        cuts = sorted(set(range(GDN_CHUNK, t1 - t0, GDN_CHUNK)) | set(pts) | {t1 - t0})
        # chunks never straddle a snapshot point; between two cuts they are at most 64 tokens long
        a = 0
        for c in cuts:
            while a < c:
                n = min(GDN_CHUNK, c - a)
                seq.append(s); tok0.append(t0 + a); ntok.append(n)
                a += n
                snap.append(pts.get(a, -1))
        seq_ck.append(len(seq))
    return torch.tensor([seq, tok0, ntok, snap], dtype=torch.int32), torch.tensor(seq_ck, dtype=torch.int32)


class GdnChunkWorkspace:
    """Fragment-order operands of the scan kernel for up to `nc * hv` (chunk, head) pairs; grows on demand."""

    def __init__(self, device):
        self.device, self.cap, self.bufs = device, 0, None

    def get(self, n_items: int, dk: int, dv: int):
        if n_items > self.cap or self.bufs is None or self.key != (dk, dv):
            lib = L()
            sizes = [lib.ti_gdn_chunk_ws_bytes(dk, dv, i) for i in range(6)]
            cap = max(n_items, 2 * self.cap)
            self.bufs = [torch.empty(cap * sz, dtype=torch.uint8, device=self.device) for sz in sizes]
            self.cap, self.key = cap, (dk, dv)
        return self.bufs


def gdn_chunked(p: GdnChunkParams, num_seqs: int, T: int, dk: int, dv: int, state_bf16: bool):
    check(L().ti_gdn_chunked(ctypes.byref(p), num_seqs, T, dk, dv, int(state_bf16), stream()), "ti_gdn_chunked")


def qkv_prep(p: QkvPrepParams, T: int, D: int):
    if not p.status:
        p.status = status_ptr()
    check(L().ti_qkv_prep(ctypes.byref(p), T, D, stream()), "ti_qkv_prep")


def attn_paged(p: AttnParams, D: int):
    if not p.status:
        p.status = status_ptr()
    check(L().ti_attn_paged(ctypes.byref(p), D, stream()), "ti_attn_paged")


def attn_prefill(q, kcache, vcache, num_blocks, block_tables, positions, tiles, gate_src, out, *, hq, hkv, D,
                 max_blocks, ld):
    """Causal GQA attention of prefill query tiles on the tcgen05 tensor cores (ops/csrc/attn_prefill.cu).
    `tiles`: int32 [3, n] = (sequence, first flat token, tokens <= 128) per tile, longest KV first."""
    n = tiles.shape[1]
    scale = D ** -0.5 * 1.4426950408889634
    check(L().ti_attn_prefill(ptr(q), q.shape[0], ptr(kcache), ptr(vcache), num_blocks, ptr(block_tables), ptr(positions),
                              ptr(tiles[0]), ptr(tiles[1]), ptr(tiles[2]), n, ptr(gate_src), ptr(out), hq, hkv,
                              max_blocks, ld, scale, D, status_ptr(), stream()), "ti_attn_prefill")


AR_NONE, AR_LIMBS, AR_BF16 = 0, 1, 2


def ar_rows(comm, parity: int, M: int, N: int, resid, h_out, *, order: int, mode: int = AR_NONE, norm_w=None,
            limbs: "Limbs" = None, xn=None, eps: float = 1e-6, two_shot: int = 0):
    """All-reduce of the row-parallel partials in `comm`'s symmetric buffer `parity` + residual -> h_out, fused with
    the RMSNorm / activation-quantisation prologue of the consuming product (ops/csrc/fused_ar.cu).
    two_shot = 1: every rank first reduces its 1/tp of the rows and broadcasts the sums into all ranks' buffers, the
    row kernel then reads local memory (many rows on >= 4 ranks); 2 / 3 run only the first / second launch (tests
    that emulate the ranks one after the other on one GPU)."""
    p = ArRowsParams()
    for r in range(comm.tp):
        p.part_peer[r] = comm.part_ptrs[parity][r]
        p.flag_peer[r] = comm.flag_ptrs[r]
    p.part_mc = comm.part_mc[parity]
    p.resid, p.h_out, p.norm_w = ptr(resid), ptr(h_out), ptr(norm_w)
    if mode == AR_LIMBS:
        p.xh, p.xl, p.xscale = ptr(limbs.hi), ptr(limbs.lo), ptr(limbs.scale)
    elif mode == AR_BF16:
        p.xn = ptr(xn)
    p.step_ptr, p.status, p.timeout_ns = comm.step_ptr, comm.status_ptr, comm.timeout_ns
    p.M, p.N, p.tp, p.rank, p.order, p.mode, p.eps = M, N, comm.tp, comm.rank, order, mode, eps
    p.rows_cap = int(getattr(comm, "ar_rows", 0) or 0)
    p.two_shot = int(two_shot)
    check(L().ti_ar_rows(ctypes.byref(p), stream()), "ti_ar_rows")


def logits_edit(p: EditParams):
    check(L().ti_logits_edit(ctypes.byref(p), stream()), "ti_logits_edit")


def sample(p: SampleParams):
    check(L().ti_sample(ctypes.byref(p), stream()), "ti_sample")


def topk(p: TopkParams):
    check(L().ti_topk(ctypes.byref(p), stream()), "ti_topk")


def topk_merge(p: TopkParams):
    """Second stage only: merges the per-chunk candidates already in ws_val / ws_idx (written, for instance, by the
    arg-max epilogue of the lm_head GEMV: one candidate per row and CTA) and exchanges the winners between ranks."""
    check(L().ti_topk_merge(ctypes.byref(p), stream()), "ti_topk_merge")


# ------------------------------------------------------------------------------------ prefill GEMM (tcgen05)
GEPI_STORE, GEPI_SWIGLU, GEPI_ROWPAR, GEPI_F32 = 0, 1, 2, 3


class Limbs:
    """Activation rows split into two int8 planes plus the per-row value of one fixed-point unit."""

    def __init__(self, M: int, K: int, device):
        self.M, self.K = M, K
        self.hi = torch.empty(M, K, dtype=torch.int8, device=device)
        self.lo = torch.empty(M, K, dtype=torch.uint8, device=device)
        self.scale = torch.empty(M, dtype=torch.float32, device=device)


def quant_rows(x: torch.Tensor, norm_w=None, eps: float = 1e-6, out: Limbs = None) -> Limbs:
    """Limb planes of x [M, K] (bf16, row stride x.stride(0)); RMSNorm(1+w) fused when norm_w is given."""
    M, K = x.shape
    if out is None:
        out = Limbs(M, K, x.device)
    check(L().ti_quant_rows(ptr(x), x.stride(0), ptr(norm_w), eps, M, K, ptr(out.hi), ptr(out.lo), ptr(out.scale),
                            stream()), "ti_quant_rows")
    return out


def gemm_w8a16(W: "LinearW", limbs: Limbs, *, out=None, epi=GEPI_STORE, resid=None) -> torch.Tensor:
    """y = x W^T on the tcgen05 tensor cores for int8-tiled W and the limb planes of x (any M)."""
    assert W.wt == W_INT8 and limbs.K == W.K
    M = limbs.M
    if out is None:
        out = torch.empty(M, W.N // 2 if epi == GEPI_SWIGLU else W.N, dtype=torch.bfloat16, device=limbs.hi.device)
    part, count = _gemm_workspace(limbs.hi.device)
    check(L().ti_gemm_w8a16(ptr(W.tiles), ptr(W.scale), W.n_tiles, W.N, W.K, ptr(limbs.hi), ptr(limbs.lo),
                            ptr(limbs.scale), M, ptr(resid), ptr(out), out.stride(0), epi, status_ptr(), ptr(part),
                            part.numel() * 4, ptr(count), count.numel(), stream()), "ti_gemm_w8a16")
    return out


def gemm_bf16(W: "LinearW", x: torch.Tensor, *, out=None, epi=GEPI_STORE, resid=None) -> torch.Tensor:
    """y = x W^T on the tcgen05 tensor cores (kind::f16) for bf16-tiled W and bf16 x [M, K] with contiguous rows.
    epi GEPI_F32 stores fp32 (logits)."""
    assert W.wt == W_BF16 and x.shape[1] == W.K and x.stride(1) == 1 and x.stride(0) == W.K and x.dtype == torch.bfloat16
    M = x.shape[0]
    if out is None:
        cols = W.N // 2 if epi == GEPI_SWIGLU else W.N
        out = torch.empty(M, cols, dtype=torch.float32 if epi == GEPI_F32 else torch.bfloat16, device=x.device)
    part, count = _gemm_workspace(x.device)
    check(L().ti_gemm_bf16(ptr(W.tiles), W.n_tiles, W.N, W.K, ptr(x), M, ptr(resid), ptr(out), out.stride(0), epi,
                           status_ptr(), ptr(part), part.numel() * 4, ptr(count), count.numel(), stream()), "ti_gemm_bf16")
    return out


_GEMM_WS = {}


def _gemm_workspace(device):
    """Split-k partials (fp32, 32 MB: 16 slices of 128 rows x 4096 columns, or fewer of wider products) and the
    per-tile arrival counters, one set per device; launches on one stream use them one after the other."""
    key = str(device)
    if key not in _GEMM_WS:
        _GEMM_WS[key] = (torch.empty(8 << 20, dtype=torch.float32, device=device),
                         torch.zeros(256, dtype=torch.int32, device=device))
    return _GEMM_WS[key]
