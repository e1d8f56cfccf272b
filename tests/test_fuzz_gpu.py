"""GPU: seeded random sweep of shapes and options against the CPU oracle, forward and backward, dense and packed.

The hand-written parity lists cover the reference's own cases; this sweep draws what they do not name: odd
lengths on both sides, every head-dim bucket (both kernel families), GQA ratios, windows of any size, softcap
and ALiBi together, negative scales, both dtypes. Every draw is fixed by its seed.
"""
import random

import pytest
import torch

from tests._cases import BWD_TOL, FWD_TOL

pytestmark = pytest.mark.gpu

HEAD_DIMS = [8, 32, 40, 64, 72, 96, 104, 128, 136, 160, 192, 200, 224, 256]


def _draw(seed):
    r = random.Random(seed)
    hk = r.choice([1, 2, 3])
    h = hk * r.choice([1, 1, 2, 4])
    d = r.choice(HEAD_DIMS)
    dtype = r.choice([torch.float16, torch.bfloat16])
    opt = {}
    mask = r.choice(["full", "causal", "causal", "window", "local"])
    if mask in ("causal", "local"):
        opt["causal"] = True
    if mask == "window":
        opt["window_left"] = r.choice([0, 1, 17, 64, 200])
        opt["window_right"] = r.choice([0, 5, 64, 130])
    if mask == "local":
        opt["window_left"] = r.choice([1, 33, 128, 300])
    if r.random() < 0.25:
        opt["softcap"] = r.choice([15.0, 30.0, 50.0])
    if r.random() < 0.2:
        opt["softmax_scale"] = r.choice([0.03, 0.2, -0.05])
    alibi = r.random() < 0.25
    return r, h, hk, d, dtype, opt, alibi


def _close(got, ref, tol, name):
    got = got.float().cpu()
    assert torch.isfinite(got).all(), name
    torch.testing.assert_close(got, ref, atol=tol["atol"], rtol=tol["rtol"], msg=lambda m: f"{name}: {m}")


@pytest.mark.parametrize("seed", range(120))
def test_dense_random_case(seed):
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward, attention_forward

    r, h, hk, d, dtype, opt, alibi = _draw(1000 + seed)
    b = r.choice([1, 2])
    sq = r.choice([1, 17, 64, 127, 128, 129, 200, 257, 333, 512])
    sk = r.choice([1, 31, 64, 128, 130, 255, 256, 300, 400, 640])
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, sq, h, d, generator=g).to(dtype)
    k = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    v = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    do = torch.randn(b, sq, h, d, generator=g).to(dtype)
    slopes = (torch.arange(1, h + 1, dtype=torch.float32) * 0.07) if alibi else None
    sl = None if slopes is None else slopes.cuda()
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, alibi_slopes=sl, **opt)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, alibi_slopes=sl, **opt)
    assert ops.device_status() == 0
    o_ref, lse_ref = attention_forward(q, k, v, alibi_slopes=slopes, **opt)
    ftol, btol = FWD_TOL[dtype], BWD_TOL[dtype]
    _close(out, o_ref, ftol, "out")
    empty = torch.isposinf(lse_ref)
    assert (torch.isposinf(lse.cpu()) == empty).all()
    torch.testing.assert_close(lse.cpu()[~empty], lse_ref[~empty], atol=ftol["lse"], rtol=0)
    dq_ref, dk_ref, dv_ref, _ = attention_backward(q, k, v, do, out=out.float().cpu(), alibi_slopes=slopes, **opt)
    _close(dq, dq_ref, btol, "dq")
    _close(dk, dk_ref, btol, "dk")
    _close(dv, dv_ref, btol, "dv")


@pytest.mark.parametrize("seed", range(60))
def test_packed_random_case(seed):
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import varlen_backward, varlen_forward

    r, h, hk, d, dtype, opt, _ = _draw(2000 + seed)
    opt.pop("softcap", None)  # the packed oracle takes masks and the scale
    n = r.choice([1, 2, 3, 5])
    lq = [r.choice([0, 1, 7, 64, 100, 128, 130, 257, 300]) for _ in range(n)]
    same = r.random() < 0.6
    lk = lq if same else [r.choice([0, 1, 19, 64, 128, 200, 256, 290]) for _ in range(n)]
    if sum(lq) == 0 or sum(lk) == 0:
        lq, lk = lq + [65], lk + [65]
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(sum(lq), h, d, generator=g).to(dtype)
    k = torch.randn(sum(lk), hk, d, generator=g).to(dtype)
    v = torch.randn(sum(lk), hk, d, generator=g).to(dtype)
    do = torch.randn(sum(lq), h, d, generator=g).to(dtype)
    cu = lambda ls: torch.tensor([0] + list(torch.tensor(ls).cumsum(0)), dtype=torch.int32)  # noqa: E731
    cu_q, cu_k = cu(lq), cu(lk)
    qc, kc, vc, doc, cq, ck = q.cuda(), k.cuda(), v.cuda(), do.cuda(), cu_q.cuda(), cu_k.cuda()
    out, lse = ops.varlen_fwd(qc, kc, vc, cq, ck, max(lq), max(lk), **opt)
    delta = ops.bwd_preprocess(doc, out, cu_seqlens_q=cq, max_seqlen_q=max(lq))
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, cu_seqlens_q=cq, cu_seqlens_k=ck, max_seqlen_q=max(lq),
                         max_seqlen_k=max(lk), **opt)
    assert ops.device_status() == 0
    o_ref, lse_ref = varlen_forward(q, k, v, cu_q, cu_k, **opt)
    ftol, btol = FWD_TOL[dtype], BWD_TOL[dtype]
    _close(out, o_ref, ftol, "out")
    empty = torch.isposinf(lse_ref)
    assert (torch.isposinf(lse.cpu()) == empty).all()
    torch.testing.assert_close(lse.cpu()[~empty], lse_ref[~empty], atol=ftol["lse"], rtol=0)
    dq_ref, dk_ref, dv_ref, _ = varlen_backward(q, k, v, do, cu_q, cu_k, out=out.float().cpu(), lse=lse.cpu(), **opt)
    _close(dq, dq_ref, btol, "dq")
    _close(dk, dk_ref, btol, "dk")
    _close(dv, dv_ref, btol, "dv")


@pytest.mark.parametrize("seed", range(16))
def test_medium_random_case(seed):
    """Enough (batch, head, query block) tiles that the persistent forward gives every CTA several of them with
    different key ranges, and the backward several CTAs per SM; the oracle checks four sampled (batch, head)
    units."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward, attention_forward

    r = random.Random(3000 + seed)
    hk = r.choice([2, 4, 8])
    group = r.choice([1, 2, 4])
    h = hk * group
    b = r.choice([2, 3, 4])
    d = r.choice([64, 128, 128, 192, 256])
    sq = r.choice([600, 777, 1024, 1300, 1700, 2048])
    sk = r.choice([sq, sq, r.choice([640, 1111, 1536, 2200])])
    dtype = r.choice([torch.float16, torch.bfloat16])
    opt = r.choice([dict(causal=True), dict(causal=True), {}, dict(causal=True, window_left=r.choice([100, 300, 700])),
                    dict(window_left=r.choice([50, 400]), window_right=r.choice([0, 64, 500]))])
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, sq, h, d, generator=g).to(dtype)
    k = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    v = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    do = torch.randn(b, sq, h, d, generator=g).to(dtype)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, **opt)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, **opt)
    assert ops.device_status() == 0
    out, lse, dq, dk, dv = out.cpu(), lse.cpu(), dq.cpu(), dk.cpu(), dv.cpu()
    ftol, btol = FWD_TOL[dtype], BWD_TOL[dtype]
    for _ in range(4):
        bi, kh = r.randrange(b), r.randrange(hk)
        hs = slice(kh * group, (kh + 1) * group)  # the whole GQA group of one kv head: dK and dV sum over it
        qs, ks, vs, dos = q[bi:bi + 1, :, hs], k[bi:bi + 1, :, kh:kh + 1], v[bi:bi + 1, :, kh:kh + 1], do[bi:bi + 1, :, hs]
        o_ref, lse_ref = attention_forward(qs, ks, vs, **opt)
        _close(out[bi:bi + 1, :, hs], o_ref, ftol, "out")
        empty = torch.isposinf(lse_ref)
        got_lse = lse[bi:bi + 1, hs]
        assert (torch.isposinf(got_lse) == empty).all()
        torch.testing.assert_close(got_lse[~empty], lse_ref[~empty], atol=ftol["lse"], rtol=0)
        dq_ref, dk_ref, dv_ref, _ = attention_backward(qs, ks, vs, dos, out=out[bi:bi + 1, :, hs].float(), **opt)
        _close(dq[bi:bi + 1, :, hs], dq_ref, btol, "dq")
        _close(dk[bi:bi + 1, :, kh:kh + 1], dk_ref, btol, "dk")
        _close(dv[bi:bi + 1, :, kh:kh + 1], dv_ref, btol, "dv")
