"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def _F():
    from tileinfer_b200.ops import functional as F
    F.L()
    return F


def _rand_w(n, k, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(BF16).float()


@pytest.mark.parametrize("M", [1, 3, 8, 16, 37])
@pytest.mark.parametrize("N,K", [(1552, 384), (5120, 2176), (8192, 5120)])
@pytest.mark.parametrize("quant", [True, False])
def test_gemv_store(M, N, K, quant):
    F = _F()
    w = _rand_w(N, K, seed=N + K)
    W = F.LinearW(w, quant)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(BF16)
    ws = F.GemvWorkspace()
    y = F.gemv(W, x, ws=ws)
    ref = x.float() @ W.dense().float().t()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    # split-k counters must be back at zero for the next launch
    assert int(ws.counters.abs().sum()) == 0
    y2 = F.gemv(W, x, ws=ws)
    assert torch.equal(y, y2), "deterministic across launches"
    # team mode: the warps of a team share a unit, each a slice of k; partial sums meet in shared memory
    for team in (1, 4, 16):
        y3 = F.gemv(W, x, ws=ws, team=team)
        torch.testing.assert_close(y3.float(), ref, rtol=2e-2, atol=2e-2)
        assert torch.equal(y3, F.gemv(W, x, ws=ws, team=team))


@pytest.mark.parametrize("M", [1, 5, 16])
def test_gemv_norm_prologue_and_swiglu(M):
    F = _F()
    H, I = 5120, 2176
    w = _rand_w(2 * I, H, seed=3)
    W = F.LinearW(w, True)
    h = (torch.randn(M, H, device="cuda") * 2).to(BF16)
    nw = (torch.randn(H, device="cuda") * 0.1).to(BF16)
    ws = F.GemvWorkspace()
    act = F.gemv(W, h, xmode=F.XNORM, epi=F.EPI_SWIGLU, norm_w=nw, ws=ws)
    hf = h.float()
    xn = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())).to(BF16).float()
    gu = (xn @ W.dense().float().t()).to(BF16).float()
    ref = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
    # products of two bf16-rounded projections of magnitude ~4: one bf16 ulp of either moves the result by ~0.1
    torch.testing.assert_close(act.float(), ref, rtol=3e-2, atol=0.25)


@pytest.mark.parametrize("M", [1, 9, 12, 16])
@pytest.mark.parametrize("K", [384, 5120])
def test_gemv_bf16_weights_norm_prologue(M, K):
    F = _F()
    N = 1024
    W = F.LinearW(_rand_w(N, K, seed=21), False)
    h = (torch.randn(M, K, device="cuda") * 2).to(BF16)
    nw = (torch.randn(K, device="cuda") * 0.1).to(BF16)
    y = F.gemv(W, h, xmode=F.XNORM, epi=F.EPI_F32, norm_w=nw)
    hf = h.float()
    xn = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())).to(BF16).float()
    torch.testing.assert_close(y, xn @ W.dense().float().t(), rtol=1e-2, atol=2e-2)
    x = torch.randn(M, K, device="cuda").to(BF16)
    r = torch.randn(M, N, device="cuda").to(BF16)
    out = F.gemv(W, x, epi=F.EPI_ROWPAR, resid=r)
    torch.testing.assert_close(out.float(), r.float() + x.float() @ W.dense().float().t(), rtol=2e-2, atol=3e-2)


def test_gemv_rowpar_residual_tp1_and_f32():
    F = _F()
    N, K, M = 5120, 768, 4
    W = F.LinearW(_rand_w(N, K, seed=5), True)
    x = (torch.randn(M, K, device="cuda")).to(BF16)
    r = (torch.randn(M, N, device="cuda")).to(BF16)
    ws = F.GemvWorkspace()
    out = F.gemv(W, x, epi=F.EPI_ROWPAR, resid=r, ws=ws)
    ref = r.float() + x.float() @ W.dense().float().t()
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=3e-2)
    lg = F.gemv(W, x, epi=F.EPI_F32, ws=ws)
    torch.testing.assert_close(lg, x.float() @ W.dense().float().t(), rtol=1e-2, atol=2e-2)   # dense() rounds q*scale to bf16


@pytest.mark.parametrize("tp,Kfull", [(2, 2048), (4, 2048), (2, 8192)])
def test_gemv_rowpar_allreduce_emulated_ranks(tp, Kfull):
    """All ranks of a TP group emulated on ONE GPU inside one cooperative launch: the tagged-packet
    all-reduce in the GEMV epilogue must equal the sum of the per-rank partial products."""
    import ctypes
    F = _F()
    from tileinfer_b200.ops.lib import ChainParams
    from tileinfer_b200.parallel.symm_mem import LocalRanks
    N, M = 5120, 3
    K = Kfull // tp                       # Kfull = 8192: team mode (four warps share a unit)
    wfull = _rand_w(N, Kfull, seed=7)
    x = (torch.randn(M, Kfull, device="cuda")).to(BF16)
    resid = (torch.randn(M, N, device="cuda")).to(BF16)
    ranks = LocalRanks(tp, N, m_cap=16)
    ncta = 148 // tp
    Ws, outs, params, keep = [], [], [], []
    for r in range(tp):
        W = F.LinearW(wfull[:, r * K:(r + 1) * K].contiguous(), True)
        xr = x[:, r * K:(r + 1) * K].contiguous()
        out = torch.zeros(M, N, dtype=BF16, device="cuda")
        ws = F.GemvWorkspace()
        p = F.make_gemv_params(W, xr, out, M, epi=F.EPI_ROWPAR, resid=resid, ws=ws, comm=ranks.view(r), order=0, ncta=ncta,
                               team=4 if Kfull == 8192 else 1)
        assert p.T == (4 if Kfull == 8192 else 1)
        Ws.append(W); outs.append(out); params.append(p); keep.append((xr, ws))
    size = ctypes.sizeof(ChainParams)
    chains = [F.make_chain([p]) for p in params]
    for c in chains:
        assert F.L().ti_gemv_chain_prepare(ctypes.byref(c), F.W_INT8, ncta) == 0
    blob = b"".join(bytes(c) for c in chains)
    dev_params = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
    rc = F.L().ti_gemv_ranks(ctypes.byref(chains[0]), dev_params.data_ptr(), tp, ncta,
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(ranks.ctrl[1]) == 0, "no peer wait may time out"
    ref = resid.float()
    for r in range(tp):
        ref = ref + x[:, r * K:(r + 1) * K].float() @ Ws[r].dense().float().t()
    for r in range(tp):
        torch.testing.assert_close(outs[r].float(), ref, rtol=2e-2, atol=6e-2 if Kfull > 4096 else 3e-2)
        assert torch.equal(outs[r], outs[0]), "every rank must hold bit-identical results"
    assert size * tp == dev_params.numel()


@pytest.mark.parametrize("quant,M,H", [(True, 3, 1024), (False, 12, 384), (True, 12, 384), (False, 1, 1024)])
def test_gemv_chain_of_four_matches_separate_launches(quant, M, H):
    """out_proj -> gate_up(SwiGLU) -> down -> in_proj in ONE launch (grid barriers in between) must equal the
    same four products launched one by one."""
    F = _F()
    I, KO, NI = 2048, 768, 1536
    wt = F.W_INT8 if quant else F.W_BF16
    Wo, Wgu = F.LinearW(_rand_w(H, KO, 11), quant), F.LinearW(_rand_w(2 * I, H, 12), quant)
    Wd, Wi = F.LinearW(_rand_w(H, I, 13), quant), F.LinearW(_rand_w(NI, H, 14), quant)
    x = torch.randn(M, KO, device="cuda").to(BF16)
    h0 = torch.randn(M, H, device="cuda").to(BF16)
    n1 = (torch.randn(H, device="cuda") * 0.1).to(BF16)
    n2 = (torch.randn(H, device="cuda") * 0.1).to(BF16)

    def run(chained):
        ws = F.GemvWorkspace()
        h1, h2 = torch.zeros_like(h0), torch.zeros_like(h0)
        act = torch.zeros(M, I, dtype=BF16, device="cuda")
        proj = torch.zeros(M, NI, dtype=BF16, device="cuda")
        ps = [F.make_gemv_params(Wo, x, h1, M, xmode=F.XGLOBAL, epi=F.EPI_ROWPAR, resid=h0, ws=ws),
              F.make_gemv_params(Wgu, h1, act, M, xmode=F.XNORM, epi=F.EPI_SWIGLU, norm_w=n1, ws=ws, team=2),
              F.make_gemv_params(Wd, act, h2, M, xmode=F.XGLOBAL, epi=F.EPI_ROWPAR, resid=h1, ws=ws, team=2),
              F.make_gemv_params(Wi, h2, proj, M, xmode=F.XNORM, epi=F.EPI_STORE, norm_w=n2, ws=ws)]
        if chained:
            F.gemv_chain_launch(ps, wt)
        else:
            for p in ps:
                F.gemv_launch(p, wt)
        torch.cuda.synchronize()
        assert int(ws.sched[2]) == 0 and int(ws.sched[8:72].abs().sum()) == 0 and int(ws.counters.abs().sum()) == 0
        return h1, act, h2, proj
    a, b = run(False), run(True)
    for name, u, v in zip(("h1", "act", "h2", "proj"), a, b):
        assert torch.equal(u, v), f"{name}: max diff {(u.float() - v.float()).abs().max().item()}"
    ref_h1 = h0.float() + x.float() @ Wo.dense().float().t()
    torch.testing.assert_close(a[0].float(), ref_h1, rtol=2e-2, atol=3e-2)
    for _ in range(3):                      # replays keep working (tickets and barrier counter reset themselves)
        c = run(True)
        assert all(torch.equal(u, v) for u, v in zip(b, c))


def test_bounded_wait_reports_timeout_and_context_survives():
    F = _F()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    result = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    # nothing ever sets the flag: the wait must give up after its 20 ms budget
    assert F.L().ti_wait_flag_probe(flag.data_ptr(), 1, 20_000_000, status.data_ptr(), result.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(result) == 0 and int(status) & 1
    flag.fill_(5)
    status.zero_()
    assert F.L().ti_wait_flag_probe(flag.data_ptr(), 3, 20_000_000, status.data_ptr(), result.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(result) == 1 and int(status) == 0
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_pointwise():
    F = _F()
    M, H = 5, 5120
    x = torch.randn(M, H, device="cuda").to(BF16)
    a = torch.randn(M, H, device="cuda").to(BF16)
    w = (torch.randn(H, device="cuda") * 0.1).to(BF16)
    y = F.rmsnorm(x, w, 1e-6)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + w.float())
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    r = torch.empty_like(x)
    y = F.rmsnorm(x, w, 1e-6, add=a, r_out=r)
    s = (x.float() + a.float()).to(BF16)
    assert torch.equal(r, s)
    sf = s.float()
    torch.testing.assert_close(y.float(), sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + w.float()),
                               rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(F.act_mul(x, a, mode=0).float(), torch.nn.functional.silu(x.float()) * a.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(F.act_mul(x, a, mode=1).float(), x.float() * torch.sigmoid(a.float()), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(F.swiglu_interleaved(x).float(),
                               torch.nn.functional.silu(x.float()[:, 0::2]) * x.float()[:, 1::2], rtol=2e-2, atol=2e-2)
    table = torch.randn(100, H, device="cuda").to(BF16)
    ids = torch.tensor([3, 99, 0, 7, 50], device="cuda")
    out = torch.empty(M, H, dtype=BF16, device="cuda")
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    F.embed(ids, table, out, step.data_ptr())
    assert torch.equal(out, table[ids]) and int(step) == 1


@pytest.mark.parametrize("dk,hk,hv,state_bf16", [(128, 2, 6, False), (64, 4, 8, False), (128, 2, 6, True)])
def test_gdn_step_matches_recurrence(dk, hk, hv, state_bf16):
    from tileinfer_b200.models.reference_cpu import gdn_recurrent, l2norm, rmsnorm, softplus20
    F = _F()
    torch.manual_seed(0)
    dv = dk
    lens = [1, 7, 33]
    S, T = len(lens), sum(lens)
    nch = 2 * dk + dv
    kd, vd = hk * dk, hv * dv
    ld = 2 * kd + 2 * vd + 2 * hv + 6
    proj = (torch.randn(T, ld, device="cuda")).to(BF16)
    conv_w = torch.randn(2 * kd + vd, 4, device="cuda") * 0.5
    A_log = torch.randn(hv, device="cuda") * 0.5
    dt_bias = torch.randn(hv, device="cuda") * 0.5
    norm_w = 1 + 0.1 * torch.randn(dv, device="cuda")
    slots = torch.tensor([2, 0, 3], dtype=torch.int32, device="cuda")
    sdt = BF16 if state_bf16 else torch.float32
    state = (torch.randn(4, hv, dk, dv, device="cuda") * 0.1).to(sdt)
    hist = (torch.randn(4, 3, 2 * kd + vd, device="cuda")).to(BF16)      # logical conv history per slot
    # kernel layout: every v-head keeps [q of its k-head | k of its k-head | its v] history
    rep = hv // hk
    cs = torch.zeros(4, hv, 3, nch, dtype=BF16, device="cuda")
    for vh in range(hv):
        kh = vh // rep
        cs[:, vh, :, :dk] = hist[:, :, kh * dk:(kh + 1) * dk]
        cs[:, vh, :, dk:2 * dk] = hist[:, :, kd + kh * dk:kd + (kh + 1) * dk]
        cs[:, vh, :, 2 * dk:] = hist[:, :, 2 * kd + vh * dv:2 * kd + (vh + 1) * dv]
    state0, cs0 = state.clone(), cs.clone()
    cu = torch.tensor([0, 1, 8, 41], dtype=torch.int32, device="cuda")
    out = torch.zeros(T, vd, dtype=BF16, device="cuda")
    snap_rel = torch.tensor([[0], [3], [16]], dtype=torch.int32, device="cuda")
    snap_state = torch.zeros(S, 1, hv, dk, dv, device="cuda")
    snap_conv = torch.zeros(S, 1, hv, 3, nch, dtype=BF16, device="cuda")
    p = F.GdnParams()
    p.proj, p.conv_w, p.neg_a_exp = proj.data_ptr(), conv_w.data_ptr(), (-A_log.exp()).contiguous().data_ptr()
    neg = (-A_log.exp()).contiguous()
    p.neg_a_exp, p.dt_bias, p.norm_w = neg.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr()
    p.state, p.conv_state, p.slots, p.cu, p.out = state.data_ptr(), cs.data_ptr(), slots.data_ptr(), cu.data_ptr(), out.data_ptr()
    p.snap_rel, p.snap_state, p.snap_conv, p.num_snap = snap_rel.data_ptr(), snap_state.data_ptr(), snap_conv.data_ptr(), 1
    p.ld, p.hk, p.hv, p.eps = ld, hk, hv, 1e-6
    # the column-split (cluster) form first, on copies: it must agree with the one-block form
    st2, cs2, out2 = state0.clone(), cs0.clone(), torch.zeros_like(out)
    sn2, sc2 = torch.zeros_like(snap_state), torch.zeros_like(snap_conv)
    p.state, p.conv_state, p.out, p.snap_state, p.snap_conv = st2.data_ptr(), cs2.data_ptr(), out2.data_ptr(), sn2.data_ptr(), sc2.data_ptr()
    F.gdn_step(p, S, dk, dv, state_bf16, split=True)
    # ... and the single-pass decode kernel (it walks longer sequences too)
    st3, cs3, out3 = state0.clone(), cs0.clone(), torch.zeros_like(out)
    sn3, sc3 = torch.zeros_like(snap_state), torch.zeros_like(snap_conv)
    p.state, p.conv_state, p.out, p.snap_state, p.snap_conv = st3.data_ptr(), cs3.data_ptr(), out3.data_ptr(), sn3.data_ptr(), sc3.data_ptr()
    F.gdn_step(p, S, dk, dv, state_bf16, single=True)
    p.state, p.conv_state, p.out = state.data_ptr(), cs.data_ptr(), out.data_ptr()
    p.snap_state, p.snap_conv = snap_state.data_ptr(), snap_conv.data_ptr()
    F.gdn_step(p, S, dk, dv, state_bf16)
    torch.cuda.synchronize()
    # same arithmetic per token; the two instantiations may contract a multiply-add differently (one bf16 ulp)
    torch.testing.assert_close(out.float(), out2.float(), rtol=8e-3, atol=2e-3)
    torch.testing.assert_close(state.float(), st2.float(), rtol=1e-2 if state_bf16 else 1e-5, atol=1e-3 if state_bf16 else 1e-6)
    assert torch.equal(cs, cs2) and torch.equal(snap_conv, sc2)
    torch.testing.assert_close(snap_state, sn2, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(out.float(), out3.float(), rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(state.float(), st3.float(), rtol=1e-2 if state_bf16 else 1e-4, atol=1e-3 if state_bf16 else 1e-5)
    assert torch.equal(cs, cs3) and torch.equal(snap_conv, sc3)
    tol = dict(rtol=3e-2, atol=3e-2)
    for s in range(S):
        t0, t1, slot = int(cu[s]), int(cu[s + 1]), int(slots[s])
        raw = proj[t0:t1, :2 * kd + vd].float()
        seq = torch.cat([hist[slot].float(), raw], 0)
        conv = torch.nn.functional.silu((seq.unfold(0, 4, 1) * conv_w[None]).sum(-1))
        Tn = t1 - t0
        q = l2norm(conv[:, :kd].reshape(Tn, hk, dk)).repeat_interleave(rep, 1) * dk ** -0.5
        k = l2norm(conv[:, kd:2 * kd].reshape(Tn, hk, dk)).repeat_interleave(rep, 1)
        v = conv[:, 2 * kd:].reshape(Tn, hv, dv)
        z = proj[t0:t1, 2 * kd + vd:2 * kd + 2 * vd].float().reshape(Tn, hv, dv)
        b = proj[t0:t1, 2 * kd + 2 * vd:2 * kd + 2 * vd + hv].float()
        a = proj[t0:t1, 2 * kd + 2 * vd + hv:2 * kd + 2 * vd + 2 * hv].float()
        g = -A_log.exp()[None] * softplus20(a + dt_bias[None])
        o, Sn = gdn_recurrent(q, k, v, g, torch.sigmoid(b), state0[slot].float())
        ref = rmsnorm(o, norm_w, 1e-6, one_plus=False) * torch.nn.functional.silu(z)
        torch.testing.assert_close(out[t0:t1].float(), ref.reshape(Tn, vd), **tol)
        torch.testing.assert_close(state[slot].float(), Sn, **tol)
        # conv history afterwards = last three raw inputs
        last3 = seq[-3:]
        torch.testing.assert_close(cs[slot, 0, :, :dk].float(), last3[:, :dk], rtol=0, atol=1e-2)
        torch.testing.assert_close(cs[slot, hv - 1, :, 2 * dk:].float(), last3[:, 2 * kd + (hv - 1) * dv:], rtol=0, atol=1e-2)
        n = int(snap_rel[s, 0])
        if n > 0:
            _, Ssnap = gdn_recurrent(q[:n], k[:n], v[:n], g[:n], torch.sigmoid(b)[:n], state0[slot].float())
            torch.testing.assert_close(snap_state[s, 0], Ssnap, **tol)
    # untouched slot stays untouched
    assert torch.equal(state[1], state0[1]) and torch.equal(cs[1], cs0[1])


@pytest.mark.parametrize("D,hq,hkv,rot", [(256, 6, 1, 64), (64, 6, 1, 16), (128, 8, 2, 32), (256, 3, 1, 64)])
def test_paged_attention_prefill_and_decode(D, hq, hkv, rot):
    from tileinfer_b200.models.reference_cpu import rmsnorm, rope_partial
    F = _F()
    torch.manual_seed(1)
    G = hq // hkv
    nb = 64
    theta = 1e7
    # sequence 0: prefill of 37 tokens after 20 cached; sequence 1: decode token at context 70; sequence 2: prefill of 5 from scratch
    ctx0, lens = [20, 69, 0], [37, 1, 5]
    S, T = 3, sum(lens)
    ld = hq * 2 * D + 2 * hkv * D
    qn = (torch.randn(D, device="cuda") * 0.1).to(BF16)
    kn = (torch.randn(D, device="cuda") * 0.1).to(BF16)
    kcache = torch.zeros(nb, hkv, 16, D, dtype=BF16, device="cuda")
    vcache = torch.zeros(nb, hkv, D, 16, dtype=BF16, device="cuda")
    perm = torch.randperm(nb).tolist()
    tables = [perm[0:8], perm[8:16], perm[16:24]]
    maxb = 8

    def run(proj, positions, slot_mapping, qg, num_qg, nsplit, Tn):
        qbuf = torch.zeros(Tn, hq, D, dtype=BF16, device="cuda")
        q = F.QkvPrepParams()
        q.proj, q.q_norm, q.k_norm, q.positions, q.slot_mapping = proj.data_ptr(), qn.data_ptr(), kn.data_ptr(), positions.data_ptr(), slot_mapping.data_ptr()
        q.q_out, q.kcache, q.vcache = qbuf.data_ptr(), kcache.data_ptr(), vcache.data_ptr()
        q.ld, q.hq, q.hkv, q.rotary_dim, q.eps, q.log2_theta = ld, hq, hkv, rot, 1e-6, math.log2(theta)
        F.qkv_prep(q, Tn, D)
        bt = torch.zeros(S, maxb, dtype=torch.int32)
        for s in range(S):
            bt[s] = torch.tensor(tables[s], dtype=torch.int32)
        bt = bt.cuda()
        items = num_qg * hkv * nsplit
        o_part = torch.empty(items * 16 * D, device="cuda")
        ml = torch.empty(items * 32, device="cuda")
        out = torch.zeros(Tn, hq * D, dtype=BF16, device="cuda")
        a = F.AttnParams()
        a.q, a.kcache, a.vcache, a.block_tables, a.positions = qbuf.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), bt.data_ptr(), positions.data_ptr()
        a.qg_seq, a.qg_tok0, a.qg_ntok = qg[0].data_ptr(), qg[1].data_ptr(), qg[2].data_ptr()
        a.o_part, a.ml_part, a.gate_src, a.out = o_part.data_ptr(), ml.data_ptr(), proj.data_ptr(), out.data_ptr()
        a.hq, a.hkv, a.max_blocks, a.nsplit, a.ld, a.num_qg = hq, hkv, maxb, nsplit, ld, num_qg
        a.scale_log2e = D ** -0.5 * 1.4426950408889634
        F.attn_paged(a, D)
        torch.cuda.synchronize()
        return out, qbuf

    def slot(s, pos):
        return tables[s][pos // 16] * 16 + pos % 16

    # reference K/V history (full precision path on the same bf16 inputs)
    hist_k = [[] for _ in range(S)]
    hist_v = [[] for _ in range(S)]

    def ref_step(proj, seqs, starts, ns):
        outs = []
        t = 0
        for s, st, n in zip(seqs, starts, ns):
            rows = proj[t:t + n].float()
            pos = torch.arange(st, st + n, device="cuda")
            qg_ = rows[:, :hq * 2 * D].reshape(n, hq, 2 * D)
            qq, gate = qg_[..., :D], qg_[..., D:].reshape(n, hq * D)
            kk = rows[:, hq * 2 * D:hq * 2 * D + hkv * D].reshape(n, hkv, D)
            vv = rows[:, hq * 2 * D + hkv * D:].reshape(n, hkv, D)
            qq = rope_partial(rmsnorm(qq, qn, 1e-6).to(BF16).float(), pos, rot, theta).to(BF16).float()
            kk = rope_partial(rmsnorm(kk, kn, 1e-6).to(BF16).float(), pos, rot, theta).to(BF16).float()
            hist_k[s].append(kk); hist_v[s].append(vv.to(BF16).float())
            K = torch.cat(hist_k[s]); V = torch.cat(hist_v[s])
            L = K.shape[0]
            sc = torch.einsum("tkgd,lkd->tkgl", qq.reshape(n, hkv, G, D), K) * D ** -0.5
            mask = torch.arange(L, device="cuda")[None] > pos[:, None]
            pr = torch.softmax(sc.masked_fill(mask[:, None, None], float("-inf")), -1)
            o = torch.einsum("tkgl,lkd->tkgd", pr, V).reshape(n, hq * D) * torch.sigmoid(gate)
            outs.append(o)
            t += n
        return torch.cat(outs)

    gt = 2 if G * 2 <= 16 else 1
    # step A: fill the caches of sequences 0 and 1 with their context (as one prefill each)
    nsA = [ctx0[0], ctx0[1]]
    TA = sum(nsA)
    projA = (torch.randn(TA, ld, device="cuda")).to(BF16)
    posA = torch.tensor(list(range(nsA[0])) + list(range(nsA[1])), dtype=torch.int32, device="cuda")
    slotsA = torch.tensor([slot(0, p) for p in range(nsA[0])] + [slot(1, p) for p in range(nsA[1])], dtype=torch.long, device="cuda")
    qgA = [[], [], []]
    t = 0
    for s, n in zip([0, 1], nsA):
        for a0 in range(t, t + n, gt):
            qgA[0].append(s); qgA[1].append(a0); qgA[2].append(min(gt, t + n - a0))
        t += n
    qgA = torch.tensor(qgA, dtype=torch.int32, device="cuda")
    outA, _ = run(projA, posA, slotsA, qgA, qgA.shape[1], 1, TA)
    refA = ref_step(projA, [0, 1], [0, 0], nsA)
    torch.testing.assert_close(outA.float(), refA, rtol=3e-2, atol=3e-2)
    # step B: mixed batch with split-KV
    projB = (torch.randn(T, ld, device="cuda")).to(BF16)
    posB = torch.tensor(sum([list(range(c, c + n)) for c, n in zip(ctx0, lens)], []), dtype=torch.int32, device="cuda")
    slotsB = torch.tensor(sum([[slot(s, p) for p in range(c, c + n)] for s, (c, n) in enumerate(zip(ctx0, lens))], []),
                          dtype=torch.long, device="cuda")
    qgB = [[], [], []]
    t = 0
    for s, n in enumerate(lens):
        for a0 in range(t, t + n, gt):
            qgB[0].append(s); qgB[1].append(a0); qgB[2].append(min(gt, t + n - a0))
        t += n
    qgB[0].append(0); qgB[1].append(0); qgB[2].append(0)      # a padding group is skipped
    qgB = torch.tensor(qgB, dtype=torch.int32, device="cuda")
    outB, _ = run(projB, posB, slotsB, qgB, qgB.shape[1], 3, T)
    refB = ref_step(projB, [0, 1, 2], ctx0, lens)
    torch.testing.assert_close(outB.float(), refB, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("k", [1, 50, 64])
def test_topk(k):
    F = _F()
    torch.manual_seed(2)
    M, V = 5, 31040
    logits = torch.randn(M, V, device="cuda")
    logits[0, 17] = logits[0, 4000] = 9.0        # tie: the smaller token id wins
    from tileinfer_b200.models.hybrid_b200 import _RunMixin

    class Dummy(_RunMixin):
        pass
    d = Dummy()
    d.v_local, d.dev, d.vocab_start, d.tp, d.rank, d.peer, d._launches = V, torch.device("cuda"), 1000, 1, 0, None, 0
    vals, idx = d._topk_rows(logits, M, k)
    torch.cuda.synchronize()
    rv, ri = torch.topk(logits, k, dim=-1)
    torch.testing.assert_close(vals, rv)
    assert int(idx[0, 0]) == 1017
    assert torch.equal(idx[1:].long() - 1000, ri[1:])


# token tiles of 32 / 64 / 128; (24, 1024, 4096), (48, 1552, 2048) and (64, 5120, 4096) also split k over gridDim.z
@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (200, 1552, 384), (64, 5120, 768), (300, 2048, 5120),
                                   (24, 1024, 4096), (48, 1552, 2048), (64, 5120, 4096), (17, 640, 1024),
                                   (1024, 9480, 512), (1100, 9600, 1024),      # these two: 256-row tiles
                                   (40, 512, 320), (300, 640, 832)])           # an odd number of 64-byte k slabs
def test_tcgen05_gemm_w8a16(M, N, K):
    """TMA-fed tcgen05 kind::i8 GEMM with two-limb activations against fp32 matmul, all three epilogues."""
    F = _F()
    W = F.LinearW(_rand_w(N, K, seed=31), True)
    x = (torch.randn(M, K, device="cuda") * 1.5).to(BF16)
    limbs = F.quant_rows(x)
    recon = (limbs.hi.float() * 256 + limbs.lo.float()) * limbs.scale[:, None]
    torch.testing.assert_close(recon, x.float(), rtol=0, atol=float(x.float().abs().max()) * 2.0 ** -14)
    y = F.gemm_w8a16(W, limbs)
    torch.cuda.synchronize()
    assert torch.equal(y, F.gemm_w8a16(W, limbs)), "deterministic (split-k partials are added in a fixed order)"
    ref = x.float() @ W.dense().float().t()
    tol = dict(rtol=2e-2, atol=3e-2 if K < 2048 else 8e-2)      # outputs of magnitude ~10: one bf16 ulp is 0.06
    torch.testing.assert_close(y.float(), ref, **tol)
    r = torch.randn(M, N, device="cuda").to(BF16)
    y2 = F.gemm_w8a16(W, limbs, epi=F.GEPI_ROWPAR, resid=r)
    torch.testing.assert_close(y2.float(), r.float() + ref, rtol=2e-2, atol=tol["atol"] + 1e-2)
    y3 = F.gemm_w8a16(W, limbs, epi=F.GEPI_SWIGLU)
    gu = ref.to(BF16).float()
    torch.testing.assert_close(y3.float(), torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2], rtol=3e-2,
                               atol=0.3 if K < 2048 else 0.6)
    # fused RMSNorm in the limb kernel
    nw = (torch.randn(K, device="cuda") * 0.1).to(BF16)
    ln = F.quant_rows(x, norm_w=nw)
    xf = x.float()
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())).to(BF16).float()
    y4 = F.gemm_w8a16(W, ln)
    torch.testing.assert_close(y4.float(), xn @ W.dense().float().t(), **tol)
    assert int(torch.zeros(1, device="cuda").item()) == 0


@pytest.mark.parametrize("M,N,K", [(24, 1024, 2048), (64, 5128, 768), (200, 1552, 384), (130, 2048, 5120),
                                   (1024, 9480, 512)])                          # 256-row tiles
def test_tcgen05_gemm_bf16(M, N, K):
    """kind::f16 variant (bf16 weights in the GEMV tile layout, bf16 activations, fp32 accumulation in TMEM)."""
    F = _F()
    W = F.LinearW(_rand_w(N, K, seed=41), False)
    x = (torch.randn(M, K, device="cuda") * 1.5).to(BF16)
    ref = x.float() @ W.dense().float().t()
    lg = F.gemm_bf16(W, x, epi=F.GEPI_F32)
    torch.cuda.synchronize()
    torch.testing.assert_close(lg, ref, rtol=1e-3, atol=1e-2)
    assert torch.equal(lg, F.gemm_bf16(W, x, epi=F.GEPI_F32))
    y = F.gemm_bf16(W, x)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=3e-2 if K < 2048 else 8e-2)
    r = torch.randn(M, N, device="cuda").to(BF16)
    y2 = F.gemm_bf16(W, x, epi=F.GEPI_ROWPAR, resid=r)
    torch.testing.assert_close(y2.float(), r.float() + ref, rtol=2e-2, atol=4e-2 if K < 2048 else 9e-2)
    y3 = F.gemm_bf16(W, x, epi=F.GEPI_SWIGLU)
    gu = ref.to(BF16).float()
    torch.testing.assert_close(y3.float(), torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2], rtol=3e-2,
                               atol=0.3 if K < 2048 else 0.6)


@pytest.mark.parametrize("tp,M", [(2, 1), (2, 5), (4, 3)])
def test_gemv_rowpar_handoff_to_next_product_emulated_ranks(tp, M):
    """Chain [row-parallel product -> product that consumes its all-reduced output] with `xll`: the consumer's
    CTAs collect the packets themselves (no collect pass, no grid barrier).  All ranks in one cooperative launch."""
    import ctypes
    F = _F()
    from tileinfer_b200.parallel.symm_mem import LocalRanks
    N, Kfull, N2 = 1024, 2048, 1536
    K = Kfull // tp
    w1 = _rand_w(N, Kfull, seed=21)
    W2 = F.LinearW(_rand_w(N2, N, seed=22), True)
    x = torch.randn(M, Kfull, device="cuda").to(BF16)
    resid = torch.randn(M, N, device="cuda").to(BF16)
    nw = (torch.randn(N, device="cuda") * 0.1).to(BF16)
    ranks = LocalRanks(tp, N, m_cap=16)
    ncta = 148 // tp
    chains, keep, hs, projs = [], [], [], []
    for r in range(tp):
        W1 = F.LinearW(w1[:, r * K:(r + 1) * K].contiguous(), True)
        xr = x[:, r * K:(r + 1) * K].contiguous()
        h = torch.zeros(M, N, dtype=BF16, device="cuda")
        proj = torch.zeros(M, N2, dtype=BF16, device="cuda")
        ws = F.GemvWorkspace()
        p1 = F.make_gemv_params(W1, xr, h, M, epi=F.EPI_ROWPAR, resid=resid, ws=ws, comm=ranks.view(r), order=0, ncta=ncta)
        p2 = F.make_gemv_params(W2, h, proj, M, xmode=F.XNORM, epi=F.EPI_STORE, norm_w=nw, ws=ws, ncta=ncta, xll=True)
        c = F.make_chain([p1, p2])
        assert F.L().ti_gemv_chain_prepare(ctypes.byref(c), F.W_INT8, ncta) == 0
        chains.append(c); keep.append((W1, xr, ws)); hs.append(h); projs.append(proj)
    dev_params = torch.frombuffer(bytearray(b"".join(bytes(c) for c in chains)), dtype=torch.uint8).cuda()
    rc = F.L().ti_gemv_ranks(ctypes.byref(chains[0]), dev_params.data_ptr(), tp, ncta, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(ranks.ctrl[1]) == 0, "no peer wait may time out"
    ref_h = resid.float()
    for r in range(tp):
        ref_h = ref_h + x[:, r * K:(r + 1) * K].float() @ keep[r][0].dense().float().t()
    hb = ref_h.to(BF16).float()
    xn = (hb * torch.rsqrt(hb.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())).to(BF16).float()
    ref_p = xn @ W2.dense().float().t()
    for r in range(tp):
        torch.testing.assert_close(hs[r].float(), ref_h, rtol=2e-2, atol=4e-2)
        torch.testing.assert_close(projs[r].float(), ref_p, rtol=3e-2, atol=6e-2)
        assert torch.equal(hs[r], hs[0]) and torch.equal(projs[r], projs[0])


@pytest.mark.parametrize("staged", [False, True])
@pytest.mark.parametrize("state_bf16", [False, True])
def test_gdn_decode_many_sequences_staged(state_bf16, staged):
    """64 single-token sequences x 6 heads, the two decode kernels for large batches: column-split blocks (a cluster
    of four blocks per head and sequence, 32 state columns each), and blocks that walk several sequences with the state
    staged through shared memory (bulk copies, inputs fetched one sequence ahead).  Both must equal the tiled kernel."""
    F = _F()
    torch.manual_seed(1)
    dk = dv = 128
    hk, hv, S = 2, 6, 64
    nch, kd, vd = 2 * dk + dv, hk * dk, hv * dv
    ld = 2 * kd + 2 * vd + 2 * hv + 6
    proj = torch.randn(S, ld, device="cuda").to(BF16)
    conv_w = torch.randn(2 * kd + vd, 4, device="cuda") * 0.5
    neg = (-(torch.randn(hv, device="cuda") * 0.5).exp()).contiguous()
    dt_bias = torch.randn(hv, device="cuda") * 0.5
    norm_w = 1 + 0.1 * torch.randn(dv, device="cuda")
    slots = torch.randperm(S + 3, device="cuda")[:S].to(torch.int32)
    sdt = BF16 if state_bf16 else torch.float32
    state0 = (torch.randn(S + 3, hv, dk, dv, device="cuda") * 0.1).to(sdt)
    cs0 = torch.randn(S + 3, hv, 3, nch, device="cuda").to(BF16)
    outs = []
    for single in (True, False):
        state, cs = state0.clone(), cs0.clone()
        out = torch.zeros(S, vd, dtype=BF16, device="cuda")
        p = F.GdnParams()
        p.proj, p.conv_w, p.neg_a_exp = proj.data_ptr(), conv_w.data_ptr(), neg.data_ptr()
        p.dt_bias, p.norm_w = dt_bias.data_ptr(), norm_w.data_ptr()
        p.state, p.conv_state, p.slots, p.out = state.data_ptr(), cs.data_ptr(), slots.data_ptr(), out.data_ptr()
        p.ld, p.hk, p.hv, p.eps = ld, hk, hv, 1e-6
        F.gdn_step(p, S, dk, dv, state_bf16, single=single, staged=staged and single)
        torch.cuda.synchronize()
        outs.append((out, state, cs))
    (o1, s1, c1), (o2, s2, c2) = outs
    torch.testing.assert_close(o1.float(), o2.float(), rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(s1.float(), s2.float(), rtol=1e-2 if state_bf16 else 1e-4, atol=1e-3 if state_bf16 else 1e-5)
    assert torch.equal(c1, c2)
    untouched = [i for i in range(S + 3) if i not in set(slots.tolist())]
    assert torch.equal(s1[untouched], state0[untouched])


@pytest.mark.parametrize("D,hq,hkv", [(256, 6, 1), (128, 4, 2), (64, 2, 1), (256, 3, 1)])
def test_attn_prefill_tcgen05(D, hq, hkv):
    """Prefill attention on tcgen05 against fp32 softmax attention: a 4096-token prompt from scratch, a 300-token
    chunk that continues an 8192-token cached prefix, and a short prompt (partial query tile); scattered pages."""
    F = _F()
    torch.manual_seed(3)
    G = hq // hkv
    ctx0, lens = [0, 8192, 0], [4096, 300, 70]
    S, T = 3, sum(lens)
    need = [(c + n + 15) // 16 for c, n in zip(ctx0, lens)]
    nb = sum(need) + 7
    perm = torch.randperm(nb).tolist()
    tables, o = [], 0
    for n in need:
        tables.append(perm[o:o + n]); o += n
    maxb = max(need)
    bt = torch.zeros(S, maxb, dtype=torch.int32)
    for s in range(S):
        bt[s, :need[s]] = torch.tensor(tables[s], dtype=torch.int32)
    bt = bt.cuda()
    kcache = torch.zeros(nb, hkv, 16, D, dtype=BF16, device="cuda")
    vcache = torch.zeros(nb, hkv, D, 16, dtype=BF16, device="cuda")
    Ks, Vs = [], []
    for s in range(S):
        L = ctx0[s] + lens[s]
        K = torch.randn(L, hkv, D, device="cuda").to(BF16)
        V = torch.randn(L, hkv, D, device="cuda").to(BF16)
        Ks.append(K); Vs.append(V)
        Lp = need[s] * 16
        Kp = torch.zeros(Lp, hkv, D, dtype=BF16, device="cuda"); Kp[:L] = K
        Vp = torch.zeros(Lp, hkv, D, dtype=BF16, device="cuda"); Vp[:L] = V
        idx = torch.tensor(tables[s], device="cuda")
        kcache[idx] = Kp.view(need[s], 16, hkv, D).permute(0, 2, 1, 3)
        vcache[idx] = Vp.view(need[s], 16, hkv, D).permute(0, 2, 3, 1)
    q = (3.0 * torch.randn(T, hq, D, device="cuda")).to(BF16)        # peaky softmax: outputs of order 1
    ld = hq * 2 * D
    proj = torch.randn(T, ld, device="cuda").to(BF16)
    positions = torch.tensor(sum([list(range(c, c + n)) for c, n in zip(ctx0, lens)], []), dtype=torch.int32, device="cuda")
    tiles, t = [], 0
    for s, n in enumerate(lens):
        for a in range(t, t + n, 128):
            tiles.append((ctx0[s] + (a - t) + min(128, t + n - a), s, a, min(128, t + n - a)))
        t += n
    tiles.sort(reverse=True)
    tiles.append((0, 0, 0, 0))                         # a padding tile is skipped
    tl = torch.tensor([[x[1] for x in tiles], [x[2] for x in tiles], [x[3] for x in tiles]], dtype=torch.int32, device="cuda")
    out = torch.zeros(T, hq * D, dtype=BF16, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    F._STATUS = st
    F.attn_prefill(q, kcache, vcache, nb, bt, positions, tl, proj, out, hq=hq, hkv=hkv, D=D, max_blocks=maxb, ld=ld)
    torch.cuda.synchronize()
    assert int(st[0]) == 0, "a bounded wait inside the kernel ran out"
    t = 0
    for s, n in enumerate(lens):
        pos = positions[t:t + n].long()
        K, V = Ks[s].float(), Vs[s].float()
        qq = q[t:t + n].float().reshape(n, hkv, G, D)
        gate = proj[t:t + n].float().reshape(n, hq, 2 * D)[..., D:].reshape(n, hq * D)
        ref = torch.empty(n, hq * D, device="cuda")
        for a in range(0, n, 512):
            b = min(n, a + 512)
            sc = torch.einsum("tkgd,lkd->tkgl", qq[a:b], K) * D ** -0.5
            mask = torch.arange(K.shape[0], device="cuda")[None] > pos[a:b, None]
            pr = torch.softmax(sc.masked_fill(mask[:, None, None], float("-inf")), -1)
            ref[a:b] = torch.einsum("tkgl,lkd->tkgd", pr, V).reshape(b - a, hq * D) * torch.sigmoid(gate[a:b])
        assert ref.abs().mean() > 0.05
        torch.testing.assert_close(out[t:t + n].float(), ref, rtol=2e-2, atol=1.5e-2)
        t += n


def test_logits_edit_kernel():
    """Repetition penalty on listed ids followed by the additive row (bias / -inf mask), rows without a slot untouched."""
    F = _F()
    torch.manual_seed(5)
    M, V, R, PC = 5, 20000, 8, 512
    logits = torch.randn(M, V, device="cuda")
    ref = logits.clone()
    slot = torch.tensor([-1, 2, 0, -1, 5], dtype=torch.int32, device="cuda")
    add = torch.zeros(R, V, device="cuda")
    add[2, ::3] = float("-inf"); add[2, 7] = 4.0
    add[5] = torch.randn(V, device="cuda")
    add_valid = torch.tensor([0, 0, 1, 0, 0, 1, 0, 0], dtype=torch.int32, device="cuda")
    pen_ids = torch.zeros(R, PC, dtype=torch.int32, device="cuda")
    pen_cnt = torch.zeros(R, dtype=torch.int32, device="cuda")
    pen_rp = torch.ones(R, device="cuda")
    ids0 = torch.sort(torch.randperm(V)[:300]).values.int().cuda()
    ids5 = torch.sort(torch.randperm(V)[:PC]).values.int().cuda()
    pen_ids[0, :300] = ids0; pen_cnt[0] = 300; pen_rp[0] = 1.3
    pen_ids[5] = ids5; pen_cnt[5] = PC; pen_rp[5] = 2.0
    p = F.EditParams()
    p.logits, p.row_slot, p.add_rows, p.add_valid = logits.data_ptr(), slot.data_ptr(), add.data_ptr(), add_valid.data_ptr()
    p.pen_ids, p.pen_cnt, p.pen_rp = pen_ids.data_ptr(), pen_cnt.data_ptr(), pen_rp.data_ptr()
    p.M, p.V, p.ld, p.pen_cap, p.chunk = M, V, V, PC, 8192
    F.logits_edit(p)
    torch.cuda.synchronize()
    v = ref[2, ids0.long()]; ref[2, ids0.long()] = torch.where(v > 0, v / 1.3, v * 1.3)       # row 2 -> slot 0: penalty only
    ref[1] += add[2]                                                                          # row 1 -> slot 2: add only
    v = ref[4, ids5.long()]; ref[4, ids5.long()] = torch.where(v > 0, v / 2.0, v * 2.0)       # row 4 -> slot 5: both
    ref[4] += add[5]
    assert torch.equal(torch.isinf(logits), torch.isinf(ref))
    torch.testing.assert_close(torch.nan_to_num(logits, neginf=-1e9), torch.nan_to_num(ref, neginf=-1e9), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("n_cand", [1, 4, 64, 512])
def test_sample_kernel_matches_host_sampler(n_cand):
    """The device draw picks the token the host sampler picks for the same candidates and the same uniform numbers
    (greedy rows, temperature, top-k, top-p; candidate lists with empty entries and ties)."""
    from tileinfer_b200.engine.sampler import Sampler
    from tileinfer_b200.parallel.comm import SingleComm
    F = _F()
    torch.manual_seed(7)
    M = 24

    class S:
        pass
    seqs = []
    for i in range(M):
        s = S()
        s.temperature = [0.0, 0.7, 1.0, 1.5][i % 4]
        s.top_k = [-1, 1, 5, 50][(i // 4) % 4]
        s.top_p = [1.0, 0.9, 0.5][i % 3]
        s.repetition_penalty, s.constraint, s.token_ids = 1.0, None, [1]
        seqs.append(s)
    vals = torch.randn(M, n_cand) * 3
    idx = torch.stack([torch.randperm(100000)[:n_cand] for _ in range(M)]).int()
    if n_cand >= 4:
        vals[:, -1] = float("-inf"); idx[:, -1] = -1                  # an empty entry
        vals[:, 1] = vals[:, 0]                                        # a tie: the smaller id wins
    host, dev = Sampler(SingleComm(), 0, (), seed=3), Sampler(SingleComm(), 0, (), seed=3)
    want = host.sample_from_candidates(vals.clone(), idx.clone().long(), seqs, gathered=True)
    spec = dev.device_spec(seqs, [])
    dv, di = vals.cuda(), idx.cuda()
    fpar = torch.tensor([spec["temperature"], spec["top_p"], spec["u"]], dtype=torch.float32, device="cuda")
    topk = torch.tensor(spec["top_k"], dtype=torch.int32, device="cuda")
    out = torch.full((M + 1,), -7, dtype=torch.int32, device="cuda")
    status = torch.tensor([9], dtype=torch.int32, device="cuda")
    p = F.SampleParams()
    p.cand_val, p.cand_idx, p.temperature, p.top_p, p.u, p.top_k = dv.data_ptr(), di.data_ptr(), fpar[0].data_ptr(), fpar[1].data_ptr(), fpar[2].data_ptr(), topk.data_ptr()
    p.out_tok, p.status_src, p.M, p.n_cand = out.data_ptr(), status.data_ptr(), M, n_cand
    F.sample(p)
    got = out.cpu().tolist()
    assert got[M] == 9                                                 # the status word rides along
    # the draw is a float computation: allow the rare row where the uniform number lands within 1e-5 of a CDF step
    diff = [i for i in range(M) if got[i] != want[i]]
    assert len(diff) <= 1, (diff, got, want)


@pytest.mark.parametrize("dk,hk,hv,state_bf16", [(128, 2, 6, False), (64, 4, 8, False), (128, 2, 4, True)])
def test_gdn_chunked_matches_recurrence(dk, hk, hv, state_bf16):
    """Chunk-parallel (WY) DeltaNet prefill against the fp32 token-serial rule and against the serial kernel:
    sequences of 1 .. 300 tokens in one flattened batch, non-zero initial state and conv history, snapshots at
    block-aligned points inside and at the end of chunks."""
    from tileinfer_b200.models.reference_cpu import gdn_recurrent, l2norm, rmsnorm, softplus20
    F = _F()
    torch.manual_seed(0)
    dv = dk
    lens = [1, 7, 33, 200, 64, 300]
    S, T = len(lens), sum(lens)
    nch = 2 * dk + dv
    kd, vd = hk * dk, hv * dv
    ld = 2 * kd + 2 * vd + 2 * hv + 6
    proj = (torch.randn(T, ld, device="cuda")).to(BF16)
    conv_w = torch.randn(2 * kd + vd, 4, device="cuda") * 0.5
    A_log = torch.randn(hv, device="cuda") * 0.5
    dt_bias = torch.randn(hv, device="cuda") * 0.5
    norm_w = 1 + 0.1 * torch.randn(dv, device="cuda")
    nslots = 8
    slots = torch.tensor([2, 0, 3, 5, 7, 6], dtype=torch.int32, device="cuda")
    sdt = BF16 if state_bf16 else torch.float32
    state = (torch.randn(nslots, hv, dk, dv, device="cuda") * 0.1).to(sdt)
    hist = (torch.randn(nslots, 3, 2 * kd + vd, device="cuda")).to(BF16)
    rep = hv // hk
    cs = torch.zeros(nslots, hv, 3, nch, dtype=BF16, device="cuda")
    for vh in range(hv):
        kh = vh // rep
        cs[:, vh, :, :dk] = hist[:, :, kh * dk:(kh + 1) * dk]
        cs[:, vh, :, dk:2 * dk] = hist[:, :, kd + kh * dk:kd + (kh + 1) * dk]
        cs[:, vh, :, 2 * dk:] = hist[:, :, 2 * kd + vh * dv:2 * kd + (vh + 1) * dv]
    state0, cs0 = state.clone(), cs.clone()
    cu_l = [0]
    for n in lens:
        cu_l.append(cu_l[-1] + n)
    cu = torch.tensor(cu_l, dtype=torch.int32, device="cuda")
    # snapshot points (relative token counts): none, none, 16 and 32, 48 and 192, 64, 80 and 288
    snap_pts = [[], [], [16, 32], [48, 192], [64], [80, 288]]
    NS = 2
    snap_rel = torch.zeros(S, NS, dtype=torch.int32)
    snap_idx = torch.zeros(S, NS, dtype=torch.int32)
    ent = 0
    for s, pts in enumerate(snap_pts):
        for j, r in enumerate(pts):
            snap_rel[s, j], snap_idx[s, j] = r, ent
            ent += 1
    snap_state = torch.zeros(ent, hv, dk, dv, device="cuda")
    snap_conv = torch.zeros(ent, hv, 3, nch, dtype=BF16, device="cuda")
    rel_d, idx_d = snap_rel.cuda(), snap_idx.cuda()
    neg = (-A_log.exp()).contiguous()

    # ---- serial kernel (exact recurrence) on copies
    st1, cs1, out1 = state0.clone(), cs0.clone(), torch.zeros(T, vd, dtype=BF16, device="cuda")
    sn1, sc1 = torch.zeros_like(snap_state), torch.zeros_like(snap_conv)
    p = F.GdnParams()
    p.proj, p.conv_w, p.neg_a_exp, p.dt_bias, p.norm_w = proj.data_ptr(), conv_w.data_ptr(), neg.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr()
    p.state, p.conv_state, p.slots, p.cu, p.out = st1.data_ptr(), cs1.data_ptr(), slots.data_ptr(), cu.data_ptr(), out1.data_ptr()
    p.snap_rel, p.snap_idx, p.snap_state, p.snap_conv, p.num_snap = rel_d.data_ptr(), idx_d.data_ptr(), sn1.data_ptr(), sc1.data_ptr(), NS
    p.ld, p.hk, p.hv, p.eps = ld, hk, hv, 1e-6
    F.gdn_step(p, S, dk, dv, state_bf16)

    # ---- chunked kernels
    out = torch.zeros(T, vd, dtype=BF16, device="cuda")
    ck, seq_ck = F.gdn_chunk_table(cu_l, snap_rel.tolist(), snap_idx.tolist())
    assert int(ck[2].sum()) == T and int(ck[2].max()) <= 64
    ck, seq_ck = ck.cuda(), seq_ck.cuda()
    c = F.GdnChunkParams()
    c.proj, c.conv_w, c.neg_a_exp, c.dt_bias, c.norm_w = proj.data_ptr(), conv_w.data_ptr(), neg.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr()
    c.state, c.conv_state, c.slots, c.cu, c.out = state.data_ptr(), cs.data_ptr(), slots.data_ptr(), cu.data_ptr(), out.data_ptr()
    c.snap_rel, c.snap_idx, c.snap_state, c.snap_conv, c.num_snap = rel_d.data_ptr(), idx_d.data_ptr(), snap_state.data_ptr(), snap_conv.data_ptr(), NS
    c.ck_seq, c.ck_tok0, c.ck_ntok, c.ck_snap, c.seq_ck, c.nc = ck[0].data_ptr(), ck[1].data_ptr(), ck[2].data_ptr(), ck[3].data_ptr(), seq_ck.data_ptr(), ck.shape[1]
    ws = F.GdnChunkWorkspace("cuda").get(ck.shape[1] * hv, dk, dv)
    c.wf, c.qf, c.mf, c.kf, c.u, c.gamma = (b.data_ptr() for b in ws)
    c.ld, c.hk, c.hv, c.eps = ld, hk, hv, 1e-6
    F.gdn_chunked(c, S, T, dk, dv, state_bf16)
    torch.cuda.synchronize()

    # conv history and conv snapshots are copies of raw inputs: bit-equal to the serial kernel's
    assert torch.equal(cs, cs1) and torch.equal(snap_conv, sc1)

    def close(got, want, atol):
        """bf16 tensor-core operands: 1 % overall (Frobenius), the typical (token, head) vector within 1 % in the L2
        norm, and all but one element in 10^4 inside the element-wise tolerance of the serial kernel's own test.
        (An output is the sum of an inter-chunk and an intra-chunk part; where the two nearly cancel a few more
        bits are lost than in the single product of the token-serial form.  Measured: median 0.4 % per vector,
        a few vectors in a thousand at 2-6 %, absolute errors below 0.08, scattered over positions; states
        within 0.9 %.)"""
        g2, w2 = got.float().reshape(-1, dv), want.float().reshape(-1, dv)
        rel = (g2 - w2).norm(dim=-1) / w2.norm(dim=-1).clamp_min(1e-3)
        assert float((g2 - w2).norm() / w2.norm()) < 1e-2 and float(rel.median()) < 1e-2
        bad = ((g2 - w2).abs() > atol + 3e-2 * w2.abs()).float().mean()
        assert float(bad) < 1e-4, float(bad)
        assert float((g2 - w2).abs().max()) < 0.25

    close(out, out1, 3e-2)
    close(state.transpose(-1, -2), st1.transpose(-1, -2), 1e-2)
    close(snap_state.transpose(-1, -2), sn1.transpose(-1, -2), 1e-2)
    # and against the fp32 reference of the rule itself
    for s in range(S):
        t0, t1, slot = cu_l[s], cu_l[s + 1], int(slots[s])
        raw = proj[t0:t1, :2 * kd + vd].float()
        seq = torch.cat([hist[slot].float(), raw], 0)
        conv = torch.nn.functional.silu((seq.unfold(0, 4, 1) * conv_w[None]).sum(-1))
        Tn = t1 - t0
        q = l2norm(conv[:, :kd].reshape(Tn, hk, dk)).repeat_interleave(rep, 1) * dk ** -0.5
        k = l2norm(conv[:, kd:2 * kd].reshape(Tn, hk, dk)).repeat_interleave(rep, 1)
        v = conv[:, 2 * kd:].reshape(Tn, hv, dv)
        z = proj[t0:t1, 2 * kd + vd:2 * kd + 2 * vd].float().reshape(Tn, hv, dv)
        b = proj[t0:t1, 2 * kd + 2 * vd:2 * kd + 2 * vd + hv].float()
        a = proj[t0:t1, 2 * kd + 2 * vd + hv:2 * kd + 2 * vd + 2 * hv].float()
        g = -A_log.exp()[None] * softplus20(a + dt_bias[None])
        o, Sn = gdn_recurrent(q, k, v, g, torch.sigmoid(b), state0[slot].float())
        ref = rmsnorm(o, norm_w, 1e-6, one_plus=False) * torch.nn.functional.silu(z)
        close(out[t0:t1], ref.reshape(Tn, vd), 3e-2)
        close(state[slot].transpose(-1, -2), Sn.transpose(-1, -2), 1e-2)
    assert torch.equal(state[1], state0[1]) and torch.equal(cs[1], cs0[1])      # an unused slot stays untouched


def _limbs_equal_up_to_one_unit(a, b):
    """Two quantisations of the same rows by kernels that add the squares of a row in a different order (the RMS factor
    may differ in its last bit): the same scales; the normalised values are rounded to bf16 before they are quantised, so
    isolated elements may sit one bf16 step (2^-7 of their magnitude) apart, all others are equal."""
    assert torch.equal(a.scale, b.scale)
    qa = a.hi.int() * 256 + a.lo.int()
    qb = b.hi.int() * 256 + b.lo.int()
    d = (qa - qb).abs()
    assert bool((d <= 1 + qa.abs() // 128).all()) and float((d > 0).float().mean()) < 1e-2, \
        (int(d.max()), float((d > 0).float().mean()))


@pytest.mark.parametrize("M,N,tp", [(40, 384, 2), (300, 5120, 4), (17, 1024, 8)])
def test_ar_rows_fused_allreduce_residual_norm_quant(M, N, tp):
    """The many-row all-reduce kernel with emulated ranks on one GPU (plain peer loads; the flags of all ranks are set
    beforehand, so nothing waits): sum of the ranks' bf16 partials + residual, then the consumer's prologue, against
    torch and against the stand-alone quantisation kernel run on the reduced rows."""
    F = _F()
    torch.manual_seed(11)

    class Comm:
        pass
    comm = Comm()
    comm.tp, comm.rank = tp, 1
    parts = [(torch.randn(M, N, device="cuda") * 2).to(BF16) for _ in range(tp)]
    flags = torch.full((64,), 7 * 65536 + 500, dtype=torch.int32, device="cuda")      # already ahead of every tag used here
    ctrl = torch.tensor([7, 0, 0, 0], dtype=torch.int32, device="cuda")               # step counter 7, status 0
    comm.part_ptrs = [[p.data_ptr() for p in parts], [p.data_ptr() for p in parts]]
    comm.part_mc = [0, 0]
    comm.flag_ptrs = [flags.data_ptr()] * tp
    comm.step_ptr, comm.status_ptr, comm.timeout_ns = ctrl.data_ptr(), ctrl.data_ptr() + 4, 10 ** 9
    resid = torch.randn(M, N, device="cuda").to(BF16)
    nw = (torch.randn(N, device="cuda") * 0.1).to(BF16)
    want_h = (sum(p.float() for p in parts) + resid.float()).to(BF16)
    # mode 0
    h = torch.zeros(M, N, dtype=BF16, device="cuda")
    F.ar_rows(comm, 0, M, N, resid, h, order=3)
    torch.cuda.synchronize()
    assert torch.equal(h, want_h) and int(ctrl[1]) == 0
    # mode 1: limbs of RMSNorm(h) == what the stand-alone kernel makes of the reduced rows
    h1 = torch.zeros_like(h)
    limbs = F.Limbs(M, N, "cuda")
    F.ar_rows(comm, 1, M, N, resid, h1, order=4, mode=F.AR_LIMBS, norm_w=nw, limbs=limbs)
    ref = F.quant_rows(want_h, norm_w=nw)
    torch.cuda.synchronize()
    assert torch.equal(h1, want_h)
    _limbs_equal_up_to_one_unit(limbs, ref)
    # mode 2: normalised bf16 rows
    h2 = torch.zeros_like(h)
    xn = torch.zeros(M, N, dtype=BF16, device="cuda")
    F.ar_rows(comm, 0, M, N, resid, h2, order=5, mode=F.AR_BF16, norm_w=nw, xn=xn)
    torch.cuda.synchronize()
    hf = want_h.float()
    want_n = (hf * torch.rsqrt((hf * hf).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())).to(BF16)
    torch.testing.assert_close(xn.float(), want_n.float(), rtol=1e-2, atol=1e-2)
    # two-shot form, the ranks emulated one after the other: every rank reduces the rows m = rank (mod tp) and writes
    # the bf16 sums over those rows in ALL buffers; afterwards one rank's row kernel reads its local buffer only
    sums = sum(p.float() for p in parts).to(BF16)
    flags[:8] = 7 * 65536 + 500                     # the one-shot calls above published rank 1's flag with their smaller tags
    flags[16] = 0                                   # word 16: count of finished blocks of the first shot (reset by the last one)
    for r in range(tp):
        comm.rank = r
        F.ar_rows(comm, 0, M, N, resid, h2, order=7, two_shot=2)
        assert int(flags[16]) == 0 and int(flags[8 + r]) == 7 * 65536 + 8      # counter back at zero, second flag published
    torch.cuda.synchronize()
    assert all(torch.equal(p, sums) for p in parts) and int(ctrl[1]) == 0
    comm.rank = 1
    h3 = torch.zeros_like(h)
    limbs3 = F.Limbs(M, N, "cuda")
    F.ar_rows(comm, 0, M, N, resid, h3, order=7, mode=F.AR_LIMBS, norm_w=nw, limbs=limbs3, two_shot=3)
    want_h3 = (sums.float() + resid.float()).to(BF16)
    ref3 = F.quant_rows(want_h3, norm_w=nw)
    torch.cuda.synchronize()
    assert torch.equal(h3, want_h3)
    _limbs_equal_up_to_one_unit(limbs3, ref3)
    # a flag that never arrives: the wait runs out, the status word says so, the context survives
    flags.zero_()
    comm.timeout_ns = 2 * 10 ** 6
    F.ar_rows(comm, 0, min(M, 4), N, resid, h2, order=6)
    torch.cuda.synchronize()
    assert int(ctrl[1]) & 1 == 1
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


@pytest.mark.parametrize("shift", [10, 13])
def test_two_limb_activation_format_on_outlier_rows(shift):
    """Activation rows with one channel 2^10 / 2^13 above the rest, through the W8A16 GEMV and the tcgen05 GEMM.

    The kernels turn a bf16 row into 16-bit fixed point with ONE power-of-two exponent per row, so an element 2^s
    below the row maximum keeps 15 - s bits.  The error of an output n is then a sum of K independent rounding errors
    of at most half a fixed-point unit u = 2^(e-14): standard deviation u / sqrt(12) * |w_n|_2.  The test pins that
    bound (6 sigma, plus the bf16 rounding of the stored output), and reports the same rows through the bf16-weight
    kernels (bf16 activations, exact products), whose only error is the output rounding."""
    F = _F()
    torch.manual_seed(shift)
    N, K = 1024, 5120
    w = _rand_w(N, K, seed=shift)
    from tileinfer_b200.models.weights import untile_int8
    W = F.LinearW(w, True)
    # exactly what the kernel multiplies with: int8 values times the bf16 row scales, no intermediate rounding
    wd = untile_int8(W.tiles)[:N].double() * W.scale.double()[:N, None]
    Wb = F.LinearW(W.dense().float(), False)                    # (nearly) the same values as bf16 weights
    wbd = Wb.dense().double()
    for M in (1, 4, 64):
        x = torch.randn(M, K, device="cuda")
        x[:, 77] = 2.0 ** shift * (1 + 0.25 * torch.rand(M, device="cuda"))
        x = x.to(BF16)
        ref = x.double() @ wd.t()
        refb = x.double() @ wbd.t()
        if M <= 8:
            y = F.gemv(W, x).double()
            yb = F.gemv(Wb, x).double()
        else:
            y = F.gemm_w8a16(W, F.quant_rows(x)).double()
            yb = F.gemm_bf16(Wb, x.contiguous()).double()
        torch.cuda.synchronize()
        e = torch.floor(torch.log2(x.float().abs().amax(dim=1))).double()            # exponent of the row maximum
        unit = torch.exp2(e - 14)[:, None]
        sigma = unit / math.sqrt(12.0) * wd.norm(dim=1)[None, :]
        bound = 6.0 * sigma + 2.0 ** -8 * ref.abs() + 1e-3
        err, errb = (y - ref).abs(), (yb - refb).abs()
        assert bool((err <= bound).all()), f"M={M}: worst excess {float((err - bound).max())}"
        # the bf16-activation path is limited by the output rounding alone
        assert bool((errb <= 2.0 ** -8 * refb.abs() + 1e-3).all())
        # how much is lost: error of the fixed-point form in units of the part of the output that does NOT come from
        # the outlier channel (what later layers can still distinguish)
        rest = (x.double() @ wd.t() - x[:, 77:78].double() * wd[:, 77][None, :]).abs().mean()
        rel = float(err.mean() / rest)
        assert rel < (0.05 if shift == 10 else 0.4), rel


def test_paged_attention_direct_load_kernel():
    """The paged attention kernel has two forms: the cp.async-pipelined one (the default, exercised by
    test_paged_attention_prefill_and_decode) and the direct-load one; this runs the same cases on the second,
    forced with TI_ATTN_PIPE=0 in a child process."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_kernels_gpu.py"), "-q", "-x", "-k",
                        "test_paged_attention_prefill_and_decode"], capture_output=True, text=True,
                       env=dict(os.environ, TI_ATTN_PIPE="0"), timeout=600, cwd=root)
    assert r.returncode == 0 and "4 passed" in r.stdout, (r.stdout[-2500:], r.stderr[-1000:])
