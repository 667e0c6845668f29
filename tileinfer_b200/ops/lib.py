"""ctypes binding of libtileinfer_b200.so.

The library must exist on a machine with a GPU: there is no PyTorch fallback for the device ops,
loading fails loudly instead."""
from __future__ import annotations

import ctypes
import os

import torch

from . import build as _build

_LIB = None
MAX_RANKS = 8


class GemvParams(ctypes.Structure):
    _fields_ = [
        ("w", ctypes.c_void_p), ("scale", ctypes.c_void_p), ("x", ctypes.c_void_p), ("norm_w", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("resid", ctypes.c_void_p), ("ws", ctypes.c_void_p), ("counters", ctypes.c_void_p),
        ("step_ptr", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("peer_ll", ctypes.c_uint64 * MAX_RANKS),
        ("timeout_ns", ctypes.c_ulonglong),
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("n_tiles", ctypes.c_int), ("K", ctypes.c_int),
        ("KB", ctypes.c_int), ("S", ctypes.c_int), ("kb_per_split", ctypes.c_int),
        ("ldx", ctypes.c_int), ("ldo", ctypes.c_int),
        ("tp", ctypes.c_int), ("rank", ctypes.c_int), ("order", ctypes.c_int), ("m_cap", ctypes.c_int),
        ("eps", ctypes.c_float), ("stages", ctypes.c_int), ("T", ctypes.c_int), ("dbg", ctypes.c_void_p), ("sched", ctypes.c_void_p), ("tps", ctypes.c_int), ("xmode", ctypes.c_int), ("epi", ctypes.c_int), ("R", ctypes.c_int), ("xll", ctypes.c_int), ("out_idx", ctypes.c_void_p),
    ]


MAX_CHAIN = 4


class ChainParams(ctypes.Structure):
    _fields_ = [("n_ops", ctypes.c_int), ("x_bytes", ctypes.c_int), ("op", GemvParams * MAX_CHAIN)]


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if os.environ.get("TI_DEBUG_LIB", "0") == "1":
            path = _build.build_debug()          # bounds-checked + jittered variant (tests, debugging)
        else:
            path = _build.LIB
            if not _build.is_current():
                path = _build.build()
        _LIB = ctypes.CDLL(path)
        for name in dir(_Sigs):
            if name.startswith("ti_"):
                fn = getattr(_LIB, name, None)
                if fn is None:
                    raise RuntimeError(f"{path} lacks symbol {name}; rebuild with python -m tileinfer_b200.ops.build --force")
                fn.restype, fn.argtypes = getattr(_Sigs, name)
        if _LIB.ti_gemv_params_size() != ctypes.sizeof(GemvParams) or \
                _LIB.ti_chain_params_size() != ctypes.sizeof(ChainParams):
            raise RuntimeError("GemvParams / ChainParams layout mismatch between Python and CUDA")
    return _LIB


_I, _P, _F, _U64 = ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_uint64


class _Sigs:
    ti_gemv_chain = (_I, [ctypes.POINTER(ChainParams), _I, _I, _P])
    ti_gemv_chain_prepare = (_I, [ctypes.POINTER(ChainParams), _I, _I])
    ti_gemv_ranks = (_I, [ctypes.POINTER(ChainParams), _P, _I, _I, _P])
    ti_gemv_params_size = (_I, [])
    ti_chain_params_size = (_I, [])


def register(name: str, restype, argtypes):
    setattr(_Sigs, name, (restype, argtypes))


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
