"""GPU parity of the packed (varlen) forward and backward against the CPU oracle.

Follows the reference's packed tests (flash-attn2-rs/tests/test_gold.py:482-534: GQA, an empty
sequence, delta of shape [H, total_q + 128 * batch]) and the packed benchmark workload (32 sequences with
lengths uniform in [128, 4096] from seed 3, H_q = 32, H_kv = 8, D = 128, causal, bf16).
"""
import pytest
import torch

from tests._cases import BWD_TOL, FWD_TOL

pytestmark = pytest.mark.gpu


def _packed(seed, lengths_q, lengths_k, h, hk, d, dtype, with_do=False):
    g = torch.Generator().manual_seed(seed)
    tq, tk = sum(lengths_q), sum(lengths_k)
    q = torch.randn(tq, h, d, generator=g).to(dtype)
    k = torch.randn(tk, hk, d, generator=g).to(dtype)
    v = torch.randn(tk, hk, d, generator=g).to(dtype)
    cu = lambda ls: torch.tensor([0] + list(torch.tensor(ls).cumsum(0)), dtype=torch.int32)  # noqa: E731
    res = [q, k, v, cu(lengths_q), cu(lengths_k)]
    if with_do:
        res.append(torch.randn(tq, h, d, generator=g).to(dtype))
    return res


def _fwd_close(out, lse, o_ref, lse_ref, dtype):
    tol = FWD_TOL[dtype]
    out, lse = out.float().cpu(), lse.cpu()
    assert torch.isfinite(out).all()
    empty = torch.isposinf(lse_ref)
    assert (torch.isposinf(lse) == empty).all()
    torch.testing.assert_close(out, o_ref, atol=tol["atol"], rtol=tol["rtol"])
    torch.testing.assert_close(lse[~empty], lse_ref[~empty], atol=tol["lse"], rtol=0)


VARLEN_CASES = [
    ("gqa-with-empty-seq", [7, 0, 18], [7, 0, 18], 4, 2, dict(causal=True)),
    ("ragged-causal", [130, 257, 64, 1, 300], [130, 257, 64, 1, 300], 4, 4, dict(causal=True)),
    ("ragged-full", [100, 256, 31], [100, 256, 31], 4, 1, {}),
    ("cross-lengths-causal", [128, 200, 50], [256, 130, 90], 4, 2, dict(causal=True)),
    ("window", [300, 140], [300, 140], 2, 2, dict(window_left=64, window_right=0)),
    ("keys-missing-for-one-seq", [40, 64], [0, 64], 2, 2, {}),
]


@pytest.mark.parametrize("name,lq,lk,h,hk,opt", VARLEN_CASES, ids=[c[0] for c in VARLEN_CASES])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
def test_varlen_forward_parity(name, lq, lk, h, hk, opt, dtype):
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import varlen_forward

    q, k, v, cu_q, cu_k = _packed(0, lq, lk, h, hk, 128, dtype)
    o_ref, lse_ref = varlen_forward(q, k, v, cu_q, cu_k, **opt)
    out, lse = ops.varlen_fwd(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), max(lq), max(lk), **opt)
    assert ops.device_status() == 0
    assert lse.shape == (h, sum(lq))
    _fwd_close(out, lse, o_ref, lse_ref, dtype)


@pytest.mark.parametrize("name,lq,lk,h,hk,opt", VARLEN_CASES[:5], ids=[c[0] for c in VARLEN_CASES[:5]])
def test_varlen_backward_parity(name, lq, lk, h, hk, opt):
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import varlen_backward

    dtype = torch.bfloat16
    q, k, v, cu_q, cu_k, do = _packed(1, lq, lk, h, hk, 128, dtype, with_do=True)
    qc, kc, vc, doc, cq, ck = q.cuda(), k.cuda(), v.cuda(), do.cuda(), cu_q.cuda(), cu_k.cuda()
    out, lse = ops.varlen_fwd(qc, kc, vc, cq, ck, max(lq), max(lk), **opt)
    delta = ops.bwd_preprocess(doc, out, cu_seqlens_q=cq, max_seqlen_q=max(lq))
    assert delta.shape == (h, sum(lq) + 128 * len(lq))
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, cu_seqlens_q=cq, cu_seqlens_k=ck, max_seqlen_q=max(lq),
                         max_seqlen_k=max(lk), **opt)
    assert ops.device_status() == 0
    dq_ref, dk_ref, dv_ref, delta_ref = varlen_backward(q, k, v, do, cu_q, cu_k, out=out.float().cpu(),
                                                        lse=lse.cpu(), **opt)
    torch.testing.assert_close(delta.cpu(), delta_ref, atol=2e-5, rtol=1e-5)
    tol = BWD_TOL[dtype]
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float().cpu(), ref, atol=tol["atol"], rtol=tol["rtol"])


def test_varlen_through_tvm_ffi_ops():
    """varlen_fwd / varlen_bwd of the Python surface: [out, lse, probs, state] and
    [dq, dk, dv, delta] with delta [H, total_q + 128 * batch] (test_gold.py:531)."""
    import flash_attn2_b200 as fa
    from oracle.attention_oracle import varlen_backward, varlen_forward

    lq = [7, 0, 18]
    q, k, v, cu, _, do = _packed(2, lq, lq, 4, 2, 128, torch.float16, with_do=True)
    qc, kc, vc, doc, cc = q.cuda(), k.cuda(), v.cuda(), do.cuda(), cu.cuda()
    out, lse, probs, state = fa.varlen_fwd(qc, kc, vc, cc, cc, max_seqlen_q=18, max_seqlen_k=18, is_causal=True)
    o_ref, lse_ref = varlen_forward(q, k, v, cu, cu, causal=True)
    _fwd_close(out, lse, o_ref, lse_ref, torch.float16)
    assert probs.numel() == 0
    dq, dk, dv, delta = fa.varlen_bwd(doc, qc, kc, vc, out, lse, cc, cc, max_seqlen_q=18, max_seqlen_k=18,
                                      is_causal=True)
    assert delta.shape == (4, 25 + 128 * 3)
    dq_ref, dk_ref, dv_ref, delta_ref = varlen_backward(q, k, v, do, cu, cu, causal=True, out=out.float().cpu(),
                                                        lse=lse.cpu())
    torch.testing.assert_close(delta.cpu(), delta_ref, atol=2e-5, rtol=1e-5)
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        torch.testing.assert_close(got.float().cpu(), ref, atol=0.008, rtol=0.04)
    qa, ka, va = (t.clone().requires_grad_() for t in (qc, kc, vc))
    fa.flash_attn_varlen_func(qa, ka, va, cc, cc, 18, 18, causal=True).backward(doc)
    torch.testing.assert_close(qa.grad.float().cpu(), dq_ref, atol=0.008, rtol=0.04)


def test_config4_full_size():
    """32 packed sequences, lengths U[128, 4096] from seed 3, H 32/8, D 128, causal, bf16, forward and
    backward from ONE launch of each kernel. Oracle on three whole sequences (all heads of one KV group)
    for O, LSE, dQ, dK, dV, the factor-of-two criterion against the reference-class kernel on the same
    sequences, dense-vs-packed equality on one sequence, finiteness and +inf-free LSE everywhere."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward, attention_forward
    from tests._cases import assert_error_within_twice, reference_class_kernel

    g = torch.Generator().manual_seed(3)
    lengths = torch.randint(128, 4097, (32,), generator=g).tolist()
    total = sum(lengths)
    q = torch.randn(total, 32, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(total, 8, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(total, 8, 128, generator=g).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    qc, kc, vc, cc = q.cuda(), k.cuda(), v.cuda(), cu.cuda()
    out, lse = ops.varlen_fwd(qc, kc, vc, cc, cc, max(lengths), max(lengths), causal=True)
    assert ops.device_status() == 0
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    do = torch.randn(total, 32, 128, generator=g).to(torch.bfloat16)
    doc = do.cuda()
    delta = ops.bwd_preprocess(doc, out, cu_seqlens_q=cc, max_seqlen_q=max(lengths))
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, cu_seqlens_q=cc, cu_seqlens_k=cc, max_seqlen_q=max(lengths),
                         max_seqlen_k=max(lengths), causal=True)
    assert ops.device_status() == 0
    for t in (dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    fa = reference_class_kernel()
    qa, ka, va = (t.clone().requires_grad_() for t in (qc, kc, vc))
    theirs, their_lse, _ = fa.flash_attn_varlen_func(qa, ka, va, cc, cc, max(lengths), max(lengths), causal=True,
                                                     return_attn_probs=True)
    theirs.backward(doc)
    tol = BWD_TOL[torch.bfloat16]
    order = sorted(range(32), key=lambda i: lengths[i])
    for i in (order[0], order[15], order[-1]):  # shortest, median, longest
        a, b = int(cu[i]), int(cu[i + 1])
        sl_q, sl_k = (slice(a, b), slice(4, 8)), (slice(a, b), slice(1, 2))
        o_ref, lse_ref = attention_forward(q[sl_q].unsqueeze(0), k[sl_k].unsqueeze(0), v[sl_k].unsqueeze(0), causal=True)
        _fwd_close(out[sl_q].unsqueeze(0), lse[4:8, a:b].unsqueeze(0), o_ref, lse_ref, torch.bfloat16)
        assert_error_within_twice("packed H32/8 causal:out", out[sl_q], theirs[sl_q].detach(), o_ref[0])
        # the stand-in returns LSE as [H, total_q] for packed input
        assert_error_within_twice("packed H32/8 causal:lse", lse[4:8, a:b], their_lse[4:8, a:b], lse_ref[0])
        # dK / dV of kv head 1 sum over its four query heads 4..7: this group is complete
        gq, gk, gv, _ = attention_backward(q[sl_q].unsqueeze(0), k[sl_k].unsqueeze(0), v[sl_k].unsqueeze(0),
                                           do[sl_q].unsqueeze(0), causal=True)
        for name, got, ref, their in (("dq", dq[sl_q], gq[0], qa.grad[sl_q]), ("dk", dk[sl_k], gk[0], ka.grad[sl_k]),
                                      ("dv", dv[sl_k], gv[0], va.grad[sl_k])):
            torch.testing.assert_close(got.float().cpu(), ref, atol=tol["atol"], rtol=tol["rtol"])
            assert_error_within_twice("packed H32/8 causal:" + name, got, their, ref)
    del qa, ka, va, theirs
    i = order[20]
    a, b = int(cu[i]), int(cu[i + 1])
    dense, dense_lse = ops.fwd(qc[a:b].unsqueeze(0), kc[a:b].unsqueeze(0), vc[a:b].unsqueeze(0), causal=True)
    assert torch.equal(dense[0], out[a:b]) and torch.equal(dense_lse[0], lse[:, a:b])


def test_varlen_other_head_dim_ragged():
    """Packed, ragged tiles take the predicated store paths: they must stop at the real head dim."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import varlen_backward, varlen_forward

    lq = [130, 7, 200]
    d = 96
    g = torch.Generator().manual_seed(12)
    q = torch.randn(sum(lq), 4, d, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(lq), 2, d, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(lq), 2, d, generator=g).to(torch.bfloat16)
    do = torch.randn(sum(lq), 4, d, generator=g).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lq).cumsum(0)), dtype=torch.int32)
    qc, kc, vc, doc, cc = q.cuda(), k.cuda(), v.cuda(), do.cuda(), cu.cuda()
    guard = torch.full((sum(lq) + 1, 4, d), 7.0, dtype=torch.bfloat16, device="cuda")  # catches writes past a row
    out, lse = ops.varlen_fwd(qc, kc, vc, cc, cc, max(lq), max(lq), causal=True)
    o_ref, lse_ref = varlen_forward(q, k, v, cu, cu, causal=True)
    _fwd_close(out, lse, o_ref, lse_ref, torch.bfloat16)
    delta = ops.bwd_preprocess(doc, out, cu_seqlens_q=cc, max_seqlen_q=max(lq))
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, cu_seqlens_q=cc, cu_seqlens_k=cc, max_seqlen_q=max(lq),
                         max_seqlen_k=max(lq), causal=True)
    assert ops.device_status() == 0
    dq_ref, dk_ref, dv_ref, _ = varlen_backward(q, k, v, do, cu, cu, out=out.float().cpu(), lse=lse.cpu(), causal=True)
    tol = BWD_TOL[torch.bfloat16]
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        torch.testing.assert_close(got.float().cpu(), ref, atol=tol["atol"], rtol=tol["rtol"])
    assert (guard == 7.0).all()


@pytest.mark.parametrize("d", [192, 256, 160])
@pytest.mark.parametrize("name,lq,lk,h,hk,opt", VARLEN_CASES, ids=[c[0] for c in VARLEN_CASES])
def test_varlen_forward_head_dims_above_128(name, lq, lk, h, hk, opt, d):
    """The packed forward for head dims 136..256 (ragged tiles store by predicate and must stop at the real
    head dim and at the end of the sequence: the oracle comparison covers every row of the output)."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import varlen_forward

    q, k, v, cu_q, cu_k = _packed(7, lq, lk, h, hk, d, torch.bfloat16)
    o_ref, lse_ref = varlen_forward(q, k, v, cu_q, cu_k, **opt)
    out, lse = ops.varlen_fwd(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), max(lq), max(lk), **opt)
    assert ops.device_status() == 0
    assert lse.shape == (h, sum(lq))
    _fwd_close(out, lse, o_ref, lse_ref, torch.bfloat16)


@pytest.mark.parametrize("d", [192, 256])
@pytest.mark.parametrize("name,lq,lk,h,hk,opt", VARLEN_CASES[:5], ids=[c[0] for c in VARLEN_CASES[:5]])
def test_varlen_backward_head_dims_above_128(name, lq, lk, h, hk, opt, d):
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import varlen_backward

    q, k, v, cu_q, cu_k, do = _packed(8, lq, lk, h, hk, d, torch.bfloat16, with_do=True)
    qc, kc, vc, doc, cq, ck = q.cuda(), k.cuda(), v.cuda(), do.cuda(), cu_q.cuda(), cu_k.cuda()
    out, lse = ops.varlen_fwd(qc, kc, vc, cq, ck, max(lq), max(lk), **opt)
    delta = ops.bwd_preprocess(doc, out, cu_seqlens_q=cq, max_seqlen_q=max(lq))
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, cu_seqlens_q=cq, cu_seqlens_k=ck, max_seqlen_q=max(lq),
                         max_seqlen_k=max(lk), **opt)
    assert ops.device_status() == 0
    dq_ref, dk_ref, dv_ref, _ = varlen_backward(q, k, v, do, cu_q, cu_k, out=out.float().cpu(), lse=lse.cpu(), **opt)
    tol = BWD_TOL[torch.bfloat16]
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float().cpu(), ref, atol=tol["atol"], rtol=tol["rtol"])


def test_rows_after_a_packed_sequence_do_not_leak_head_dim_256():
    """The NaN-neighbour test below for the kernels of the wide head dims (forward and backward)."""
    from flash_attn2_b200 import cabi_ops as ops

    lengths = [130, 77, 257, 40, 300, 64]
    q, k, v, cu, _, do = _packed(5, lengths, lengths, 4, 2, 256, torch.bfloat16, with_do=True)
    cc = cu.cuda()

    def run(poison):
        ts = [t.clone() for t in (q, k, v, do)]
        if poison:
            for i in (1, 3, 5):
                for t in ts:
                    t[int(cu[i]):int(cu[i + 1])] = float("nan")
        qc, kc, vc, doc = [t.cuda() for t in ts]
        out, lse = ops.varlen_fwd(qc, kc, vc, cc, cc, max(lengths), max(lengths), causal=True)
        delta = ops.bwd_preprocess(doc, out, cu_seqlens_q=cc, max_seqlen_q=max(lengths))
        dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, cu_seqlens_q=cc, cu_seqlens_k=cc,
                             max_seqlen_q=max(lengths), max_seqlen_k=max(lengths), causal=True)
        assert ops.device_status() == 0
        return out, lse, dq, dk, dv

    base, bad = run(False), run(True)
    for i in (0, 2, 4):
        a, b = int(cu[i]), int(cu[i + 1])
        assert torch.equal(base[0][a:b], bad[0][a:b]) and torch.equal(base[1][:, a:b], bad[1][:, a:b]), i
        assert torch.equal(base[3][a:b], bad[3][a:b]) and torch.equal(base[4][a:b], bad[4][a:b]), i
        assert torch.isfinite(bad[2][a:b].float()).all()
        torch.testing.assert_close(bad[2][a:b].float(), base[2][a:b].float(), atol=2e-2, rtol=2e-2)


def test_rows_after_a_packed_sequence_do_not_leak():
    """The reference zero-fills the rows of a tile that lie past the end of a sequence
    (flash-attn2-rs/src/device/forward/mod.rs:171-175,200), so what a neighbouring sequence holds can
    never reach this one. Here every second sequence of the batch is filled with NaN (Q, K, V, dO):
    the outputs and gradients of the clean sequences must equal, bit for bit, those of a batch whose
    other sequences hold ordinary numbers (dQ, which is summed in arrival order, within tolerance)."""
    from flash_attn2_b200 import cabi_ops as ops

    lengths = [130, 77, 257, 40, 300, 64]
    q, k, v, cu, _, do = _packed(5, lengths, lengths, 4, 2, 128, torch.bfloat16, with_do=True)
    cc = cu.cuda()
    clean = [0, 2, 4]

    def run(poison):
        ts = [t.clone() for t in (q, k, v, do)]
        if poison:
            for i in (1, 3, 5):
                for t in ts:
                    t[int(cu[i]):int(cu[i + 1])] = float("nan")
        qc, kc, vc, doc = [t.cuda() for t in ts]
        out, lse = ops.varlen_fwd(qc, kc, vc, cc, cc, max(lengths), max(lengths), causal=True)
        delta = ops.bwd_preprocess(doc, out, cu_seqlens_q=cc, max_seqlen_q=max(lengths))
        dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, cu_seqlens_q=cc, cu_seqlens_k=cc,
                             max_seqlen_q=max(lengths), max_seqlen_k=max(lengths), causal=True)
        assert ops.device_status() == 0
        return out, lse, dq, dk, dv

    base, bad = run(False), run(True)
    for i in clean:
        a, b = int(cu[i]), int(cu[i + 1])
        for name, x, y in zip(("out", "dq", "dk", "dv"), (base[0], base[2], base[3], base[4]),
                              (bad[0], bad[2], bad[3], bad[4])):
            assert torch.isfinite(y[a:b].float()).all(), (name, i)
            if name == "dq":
                torch.testing.assert_close(y[a:b].float(), x[a:b].float(), atol=2e-2, rtol=2e-2)
            else:
                assert torch.equal(x[a:b], y[a:b]), (name, i)
        assert torch.equal(base[1][:, a:b], bad[1][:, a:b])
