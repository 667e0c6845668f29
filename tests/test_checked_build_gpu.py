"""The bounds-checked, jittered build of the kernel library (-DTI_BOUNDS_CHECK -DTI_JITTER, selected with
TI_DEBUG_LIB=1): the multi-rank protocols give the same results with random delays in front of every send and
collect, and an index outside the range the kernel was told about sets the bounds bit of the status word and is
skipped.  (The out-of-range indices used here still lie inside the memory that was really allocated, so nothing can
fault whatever the check does.)  Every case runs in a child process: the library variant is chosen at load time."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROBE = r'''
import math, sys, torch
sys.path.insert(0, %r)
from tileinfer_b200.ops import functional as F
from tileinfer_b200.ops import build as B
F.L()
assert F._l._LIB._name.endswith("_dbg.so"), F._l._LIB._name
BF16 = torch.bfloat16
D, hq, hkv = 64, 2, 1
nb_real, nb_told = 16, 8                       # the cache really has 16 pages; the kernels are told 8
st = torch.zeros(4, dtype=torch.int32, device="cuda")
F._STATUS = st
kc = torch.zeros(nb_real, hkv, 16, D, dtype=BF16, device="cuda")
vc = torch.zeros(nb_real, hkv, D, 16, dtype=BF16, device="cuda")
T = 4
ld = hq * 2 * D + 2 * hkv * D
proj = torch.randn(T, ld, device="cuda").to(BF16)
qn = torch.zeros(D, dtype=BF16, device="cuda"); kn = torch.zeros(D, dtype=BF16, device="cuda")
pos = torch.arange(T, dtype=torch.int32, device="cuda")
slots = torch.tensor([0, 1, 12 * 16 + 2, 3], dtype=torch.long, device="cuda")     # token 2 -> page 12 >= 8
qbuf = torch.zeros(T, hq, D, dtype=BF16, device="cuda")
q = F.QkvPrepParams()
q.proj, q.q_norm, q.k_norm, q.positions, q.slot_mapping = proj.data_ptr(), qn.data_ptr(), kn.data_ptr(), pos.data_ptr(), slots.data_ptr()
q.q_out, q.kcache, q.vcache = qbuf.data_ptr(), kc.data_ptr(), vc.data_ptr()
q.ld, q.hq, q.hkv, q.rotary_dim, q.eps, q.log2_theta, q.num_blocks = ld, hq, hkv, 16, 1e-6, math.log2(1e7), nb_told
F.qkv_prep(q, T, D)
torch.cuda.synchronize()
assert int(st[0]) & 4, "the bounds bit must be set"
assert float(kc[12].abs().sum()) == 0.0 and float(vc[12].abs().sum()) == 0.0, "the out-of-range page must stay untouched"
assert float(kc[0].abs().sum()) > 0.0
# attention: a block table that names page 12
st.zero_()
bt = torch.tensor([[12]], dtype=torch.int32, device="cuda")
qg = torch.tensor([[0], [0], [1]], dtype=torch.int32, device="cuda")
o_part = torch.zeros(16 * D, device="cuda"); ml = torch.zeros(32, device="cuda")
out = torch.zeros(T, hq * D, dtype=BF16, device="cuda")
a = F.AttnParams()
a.q, a.kcache, a.vcache, a.block_tables, a.positions = qbuf.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), pos.data_ptr()
a.qg_seq, a.qg_tok0, a.qg_ntok = qg[0].data_ptr(), qg[1].data_ptr(), qg[2].data_ptr()
a.o_part, a.ml_part, a.gate_src, a.out = o_part.data_ptr(), ml.data_ptr(), proj.data_ptr(), out.data_ptr()
a.hq, a.hkv, a.max_blocks, a.nsplit, a.ld, a.num_qg, a.num_blocks = hq, hkv, 1, 1, ld, 1, nb_told
a.scale_log2e = D ** -0.5 * 1.4426950408889634
F.attn_paged(a, D)
torch.cuda.synchronize()
assert int(st[0]) & 4
assert float(torch.ones(4, device="cuda").sum()) == 4.0
print("CHECKED_BUILD_OK")
'''


def _env():
    return dict(os.environ, TI_DEBUG_LIB="1")


def test_bad_indices_set_the_bounds_bit_and_are_skipped():
    r = subprocess.run([sys.executable, "-c", PROBE % ROOT], capture_output=True, text=True, env=_env(), timeout=600)
    assert "CHECKED_BUILD_OK" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])


def test_rank_protocols_under_arrival_jitter():
    """Emulated tensor-parallel ranks (one cooperative launch), the many-row all-reduce, the top-k kernels: same
    results with random delays before every packet send / collect and flag publication."""
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_kernels_gpu.py"), "-q", "-x",
                        "-k", "emulated_ranks or ar_rows or topk or chain_of_four"],
                       capture_output=True, text=True, env=_env(), timeout=900, cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-2500:], r.stderr[-1500:])
    assert " passed" in r.stdout and "failed" not in r.stdout
