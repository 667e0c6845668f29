"""The allocation-free top-k entry point (ti_topk_static), called through its exported C symbol the way a
caller without PyTorch's allocator would: raw device pointers in, results out, nothing allocated by the
library.  Checked against the regular entry point on two calls in a row (the calls share one static scratch
array).  Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from tileinfer_b200.ops import build
    lib = ctypes.CDLL(build.LIB if build.is_current() else build.build())
    lib.ti_topk_static.restype = ctypes.c_int
    lib.ti_topk_static.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.ti_topk_static_error.restype = ctypes.c_char_p
    lib.ti_topk_static_error.argtypes = [ctypes.c_int]
    return lib


def _reference_entry(logits, k, vocab_start):
    """The existing entry point (ti_topk with caller-provided workspace)."""
    from tileinfer_b200.models.hybrid_b200 import _RunMixin

    class Host(_RunMixin):
        pass
    h = Host()
    h.v_local, h.dev, h.vocab_start, h.tp, h.rank, h.peer, h._launches = logits.shape[1], logits.device, vocab_start, 1, 0, None, 0
    return h._topk_rows(logits, logits.shape[0], k)


def test_static_scratch_topk_matches_regular_entry_twice():
    lib = _lib()
    torch.manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream
    cases = [(5, 31040, 50, 1000), (16, 248320, 64, 0), (1, 1024, 1, 3)]
    # tensors that earlier tests left in reference cycles must not be released in the middle of the measurement
    import gc
    gc.collect()
    torch.cuda.synchronize()
    for rows, vocab, k, start in cases:
        logits = torch.randn(rows, vocab, device="cuda")
        out_val = torch.empty(rows, k, dtype=torch.float32, device="cuda")
        out_idx = torch.empty(rows, k, dtype=torch.int32, device="cuda")
        for call in range(2):                      # two calls in a row share the static scratch
            if call == 1:
                logits = torch.randn(rows, vocab, device="cuda")
            gc.disable()
            try:
                used_before = torch.cuda.memory_allocated()
                rc = lib.ti_topk_static(logits.data_ptr(), rows, vocab, logits.stride(0), k, start, out_val.data_ptr(),
                                        out_idx.data_ptr(), stream)
                assert rc == 0, lib.ti_topk_static_error(rc)
                torch.cuda.synchronize()
                assert torch.cuda.memory_allocated() == used_before
            finally:
                gc.enable()
            ref_val, ref_idx = _reference_entry(logits, k, start)
            torch.cuda.synchronize()
            torch.testing.assert_close(out_val, ref_val, rtol=0, atol=0)
            assert torch.equal(out_idx, ref_idx)
            tv, ti = torch.topk(logits, k, dim=-1)
            torch.testing.assert_close(out_val, tv)


def test_static_scratch_topk_rejects_oversize():
    lib = _lib()
    x = torch.zeros(17, 512, device="cuda")
    o = torch.zeros(17, 4, device="cuda")
    oi = torch.zeros(17, 4, dtype=torch.int32, device="cuda")
    rc = lib.ti_topk_static(x.data_ptr(), 17, 512, 512, 4, 0, o.data_ptr(), oi.data_ptr(), 0)
    assert rc == -1 and b"16 rows" in lib.ti_topk_static_error(rc)
    assert lib.ti_topk_static(x.data_ptr(), 4, 512, 512, 65, 0, o.data_ptr(), oi.data_ptr(), 0) == -2
    assert lib.ti_topk_static(x.data_ptr(), 4, 600000, 600000, 4, 0, o.data_ptr(), oi.data_ptr(), 0) == -3
    assert lib.ti_topk_static(0, 4, 512, 512, 4, 0, o.data_ptr(), oi.data_ptr(), 0) == -4
