"""GPU parity of the backward path (delta preprocess, dQ/dK/dV) against the CPU oracle.

Shapes follow the reference's backward tests (flash-attn2-rs/tests/test_gold.py:269-363: MHA/GQA,
causal, odd lengths, strided inputs, delta parity at 2e-5) plus the benchmark's backward workload (B16 H16 S2048 D128 bf16 causal) at full size.
"""
import pytest
import torch

from tests._cases import BWD_TOL, make_qkv

pytestmark = pytest.mark.gpu

CASES = [
    ("full-s128", (1, 2, 2, 128, 128, 128), {}),
    ("causal-s256", (2, 4, 4, 256, 256, 128), dict(causal=True)),
    ("full-s256", (2, 4, 4, 256, 256, 128), {}),
    ("causal-gqa-h8-hk2", (2, 8, 2, 256, 256, 128), dict(causal=True)),
    ("mqa-h4-hk1", (1, 4, 1, 192, 192, 128), {}),
    ("odd-causal-s333", (2, 4, 4, 333, 333, 128), dict(causal=True)),
    ("causal-sq320-sk256", (1, 4, 4, 320, 256, 128), dict(causal=True)),
    ("full-sq128-sk256", (1, 4, 4, 128, 256, 128), {}),
    ("window-wl64-wr64", (1, 4, 4, 256, 256, 128), dict(window_left=64, window_right=64)),
    ("local-causal-wl64", (1, 4, 4, 300, 300, 128), dict(causal=True, window_left=64)),
    ("custom-scale", (1, 4, 4, 256, 256, 128), dict(causal=True, softmax_scale=0.05)),
    ("d64-causal-gqa", (2, 4, 2, 512, 512, 64), dict(causal=True)),
    ("d64-odd", (1, 2, 2, 200, 333, 64), {}),
    ("s1024-causal", (1, 4, 4, 1024, 1024, 128), dict(causal=True)),
]


def _run(q, k, v, do, **opt):
    from flash_attn2_b200 import cabi_ops as ops

    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, **opt)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, **opt)
    assert ops.device_status() == 0
    return out, lse, delta, dq, dk, dv


def _close(got, ref, dtype, name):
    tol = BWD_TOL[dtype]
    got = got.float().cpu()
    assert torch.isfinite(got).all(), name
    torch.testing.assert_close(got, ref, atol=tol["atol"], rtol=tol["rtol"], msg=lambda m: f"{name}: {m}")


@pytest.mark.parametrize("name,shape,opt", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
def test_backward_parity_cabi(name, shape, opt, dtype):
    from oracle.attention_oracle import attention_backward

    b, h, hk, sq, sk, d = shape
    q, k, v, do = make_qkv(2, b, h, hk, sq, sk, d, dtype, with_do=True)
    out, lse, delta, dq, dk, dv = _run(q, k, v, do, **opt)
    dq_ref, dk_ref, dv_ref, delta_ref = attention_backward(q, k, v, do, out=out.float().cpu(), **opt)
    torch.testing.assert_close(delta.cpu(), delta_ref, atol=2e-5, rtol=1e-5)
    _close(dq, dq_ref, dtype, "dq")
    _close(dk, dk_ref, dtype, "dk")
    _close(dv, dv_ref, dtype, "dv")


WIDE_CASES = [
    ("d256-full-s128", (1, 2, 2, 128, 128, 256), {}, False),
    ("d256-causal-gqa-odd", (2, 8, 2, 333, 333, 256), dict(causal=True), False),
    ("d192-causal", (2, 4, 4, 512, 512, 192), dict(causal=True), False),
    ("d192-mqa-sq320-sk256", (1, 4, 1, 320, 256, 192), dict(causal=True), False),
    ("d160-full-sq128-sk700", (1, 4, 4, 128, 700, 160), {}, False),
    ("d136-window-wl64-wr64", (1, 4, 4, 256, 256, 136), dict(window_left=64, window_right=64), False),
    ("d256-local-causal-wl100", (1, 4, 4, 300, 300, 256), dict(causal=True, window_left=100), False),
    ("d224-custom-scale", (1, 2, 2, 256, 256, 224), dict(causal=True, softmax_scale=0.05), False),
    ("d256-softcap30-causal", (1, 4, 4, 256, 256, 256), dict(causal=True, softcap=30.0), False),
    ("d192-alibi-causal-gqa", (2, 4, 2, 256, 256, 192), dict(causal=True), True),
    ("d256-alibi-softcap-window", (1, 4, 4, 200, 333, 256), dict(window_left=64, window_right=32, softcap=20.0), True),
    ("d256-rows-without-keys", (1, 2, 2, 384, 256, 256), dict(causal=True), False),
    ("d256-s1024-causal", (1, 4, 4, 1024, 1024, 256), dict(causal=True), False),
]


@pytest.mark.parametrize("name,shape,opt,use_alibi", WIDE_CASES, ids=[c[0] for c in WIDE_CASES])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
def test_backward_head_dims_above_128(name, shape, opt, use_alibi, dtype):
    """Head dims 136..256 (the reference's 192 and 256 buckets) run on the kernel that splits the head dim of dK,
    dV and dQ over two CTAs; the cases repeat the masks and score transforms of the lists above."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward

    b, h, hk, sq, sk, d = shape
    q, k, v, do = make_qkv(11, b, h, hk, sq, sk, d, dtype, with_do=True)
    slopes = (torch.arange(1, h + 1, dtype=torch.float32) * 0.05) if use_alibi else None
    sl_gpu = None if slopes is None else slopes.cuda()
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, alibi_slopes=sl_gpu, **opt)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, alibi_slopes=sl_gpu, **opt)
    assert ops.device_status() == 0
    dq_ref, dk_ref, dv_ref, delta_ref = attention_backward(q, k, v, do, out=out.float().cpu(), alibi_slopes=slopes, **opt)
    torch.testing.assert_close(delta.cpu(), delta_ref, atol=2e-5, rtol=1e-5)
    _close(dq, dq_ref, dtype, "dq")
    _close(dk, dk_ref, dtype, "dk")
    _close(dv, dv_ref, dtype, "dv")
    if "rows-without-keys" in name:
        assert torch.isposinf(lse[:, :, :128]).all() and (dq[:, :128] == 0).all()


def test_backward_head_dim_256_dq_only_dkv_only_and_autograd():
    """The deterministic pair of the reference (bwd_dq + bwd_dkv) and the autograd surface at head dim 256."""
    import flash_attn2_b200 as fa
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward

    q, k, v, do = make_qkv(12, 2, 4, 2, 300, 300, 256, torch.bfloat16, with_do=True)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, causal=True)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, causal=True)
    dq1, _, _ = ops.bwd(qc, kc, vc, doc, lse, delta, causal=True, which=1)
    _, dk2, dv2 = ops.bwd(qc, kc, vc, doc, lse, delta, causal=True, which=2)
    assert ops.device_status() == 0
    torch.testing.assert_close(dq1.float(), dq.float(), atol=2e-2, rtol=2e-2)  # arrival order differs run to run
    assert torch.equal(dk2, dk) and torch.equal(dv2, dv)
    qa, ka, va = (t.clone().requires_grad_() for t in (qc, kc, vc))
    fa.flash_attn_func(qa, ka, va, causal=True).backward(doc)
    gq, gk, gv, _ = attention_backward(q, k, v, do, causal=True)
    _close(qa.grad, gq, torch.bfloat16, "dq")
    _close(ka.grad, gk, torch.bfloat16, "dk")
    _close(va.grad, gv, torch.bfloat16, "dv")


def test_backward_rows_without_keys_get_zero_gradient():
    """Causal with Sq > Sk: the first Sq - Sk rows see no key (LSE = +inf) and must get dQ = 0."""
    q, k, v, do = make_qkv(3, 1, 2, 2, 384, 256, 128, torch.float16, with_do=True)
    out, lse, delta, dq, dk, dv = _run(q, k, v, do, causal=True)
    assert torch.isposinf(lse[:, :, :128]).all()
    assert (dq[:, :128] == 0).all()
    assert torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()


def test_backward_dq_only_and_dkv_only_match_all():
    from flash_attn2_b200 import cabi_ops as ops

    q, k, v, do = [t.cuda() for t in make_qkv(4, 2, 4, 2, 256, 256, 128, torch.bfloat16, with_do=True)]
    out, lse = ops.fwd(q, k, v, causal=True)
    delta = ops.bwd_preprocess(do, out)
    dq, dk, dv = ops.bwd(q, k, v, do, lse, delta, causal=True, which=3)
    dq1, _, _ = ops.bwd(q, k, v, do, lse, delta, causal=True, which=1)
    _, dk2, dv2 = ops.bwd(q, k, v, do, lse, delta, causal=True, which=2)
    assert ops.device_status() == 0
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)  # dK/dV never use atomics
    torch.testing.assert_close(dq1.float(), dq.float(), atol=2e-2, rtol=2e-2)  # fp32 add order may differ


def test_backward_strided_inputs():
    """Head-sliced views of larger tensors (test_gold.py:269-310 uses strided backward inputs)."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward

    q, k, v, do = make_qkv(5, 1, 8, 8, 256, 256, 128, torch.float16, with_do=True)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    sl = slice(2, 6)
    out, lse = ops.fwd(qc[:, :, sl], kc[:, :, sl], vc[:, :, sl], causal=True)
    delta = ops.bwd_preprocess(doc[:, :, sl], out)
    dq, dk, dv = ops.bwd(qc[:, :, sl], kc[:, :, sl], vc[:, :, sl], doc[:, :, sl], lse, delta, causal=True)
    dq_ref, dk_ref, dv_ref, _ = attention_backward(q[:, :, sl], k[:, :, sl], v[:, :, sl], do[:, :, sl], causal=True,
                                                   out=out.float().cpu())
    _close(dq, dq_ref, torch.float16, "dq")
    _close(dk, dk_ref, torch.float16, "dk")
    _close(dv, dv_ref, torch.float16, "dv")


def test_backward_through_tvm_ffi_ops_and_autograd():
    """bwd() returns [dQ, dK, dV, softmax_d]; deterministic=True takes the bwd_dq + bwd_dkv pair;
    flash_attn_func differentiates through both."""
    import flash_attn2_b200 as fa
    from oracle.attention_oracle import attention_backward

    q, k, v, do = make_qkv(6, 2, 8, 2, 256, 256, 128, torch.bfloat16, with_do=True)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse, _, _ = fa.fwd(qc, kc, vc, is_causal=True)
    dq_ref, dk_ref, dv_ref, delta_ref = attention_backward(q, k, v, do, causal=True, out=out.float().cpu())
    for det in (False, True):
        dq, dk, dv, delta = fa.bwd(doc, qc, kc, vc, out, lse, is_causal=True, deterministic=det)
        torch.testing.assert_close(delta.cpu(), delta_ref, atol=2e-5, rtol=1e-5)
        _close(dq, dq_ref, torch.bfloat16, "dq")
        _close(dk, dk_ref, torch.bfloat16, "dk")
        _close(dv, dv_ref, torch.bfloat16, "dv")
    qa, ka, va = (t.clone().requires_grad_() for t in (qc, kc, vc))
    fa.flash_attn_func(qa, ka, va, causal=True).backward(doc)
    _close(qa.grad, dq_ref, torch.bfloat16, "dq")
    _close(ka.grad, dk_ref, torch.bfloat16, "dk")
    _close(va.grad, dv_ref, torch.bfloat16, "dv")
    with pytest.raises((RuntimeError, ValueError)):
        fa.bwd(doc, qc, kc, vc, out, lse[:, :, :-1].contiguous(), is_causal=True)


def test_config3_full_size_slices_and_properties():
    """The benchmark's backward workload (B16 H16 S2048 D128 bf16 causal, dO from seed 2) at full size: oracle on
    sampled (batch, head) units; dV and dK/dQ are linear in dO; the last key's dK/dV only see the
    last query row."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward

    g1, g2 = torch.Generator().manual_seed(1), torch.Generator().manual_seed(2)
    q, k, v = [torch.randn(16, 2048, 16, 128, generator=g1).to(torch.bfloat16) for _ in range(3)]
    do = torch.randn(16, 2048, 16, 128, generator=g2).to(torch.bfloat16)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, causal=True)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, causal=True)
    assert ops.device_status() == 0
    for t in (dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    from tests._cases import assert_error_within_twice, reference_class_kernel, sample_units

    # the reference-class kernel's gradients on the same inputs, for the factor-of-two criterion
    qa, ka, va = (t.clone().requires_grad_() for t in (qc, kc, vc))
    reference_class_kernel().flash_attn_func(qa, ka, va, causal=True).backward(doc)
    for b, h in sample_units(16, 16):
        sl = (slice(b, b + 1), slice(None), slice(h, h + 1))
        dq_ref, dk_ref, dv_ref, delta_ref = attention_backward(q[sl], k[sl], v[sl], do[sl], causal=True,
                                                               out=out[sl].float().cpu())
        torch.testing.assert_close(delta[b:b + 1, h:h + 1].cpu(), delta_ref, atol=2e-5, rtol=1e-5)
        _close(dq[sl], dq_ref, torch.bfloat16, "dq")
        _close(dk[sl], dk_ref, torch.bfloat16, "dk")
        _close(dv[sl], dv_ref, torch.bfloat16, "dv")
        # the oracle's gradients for the factor-of-two criterion use its own fp32 O (no kernel's rounding)
        gq, gk, gv, _ = attention_backward(q[sl], k[sl], v[sl], do[sl], causal=True)
        assert_error_within_twice("B16 H16 S2048 causal:dq", dq[sl], qa.grad[sl], gq)
        assert_error_within_twice("B16 H16 S2048 causal:dk", dk[sl], ka.grad[sl], gk)
        assert_error_within_twice("B16 H16 S2048 causal:dv", dv[sl], va.grad[sl], gv)
    del qa, ka, va
    # key S-1 is visible to query S-1 only, with P = softmax weight p: dV[S-1] = p * dO[S-1]
    p_last = torch.exp((qc[:, -1].float() * kc[:, -1].float()).sum(-1) / 128 ** 0.5 - lse[:, :, -1])
    torch.testing.assert_close(dv[:, -1].float(), p_last.unsqueeze(-1) * doc[:, -1].float(), atol=2e-3, rtol=2e-2)
    # linearity in dO (delta scales too)
    delta2 = ops.bwd_preprocess(doc * 2, out)
    dq2, dk2, dv2 = ops.bwd(qc, kc, vc, doc * 2, lse, delta2, causal=True)
    torch.testing.assert_close(dv2.float(), dv.float() * 2, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(dk2.float(), dk.float() * 2, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(dq2.float(), dq.float() * 2, atol=2e-2, rtol=2e-2)


FANCY_CASES = [
    ("softcap30-causal", (1, 4, 4, 256, 256, 128), dict(causal=True, softcap=30.0), False),
    ("alibi-causal-gqa", (2, 4, 2, 256, 256, 128), dict(causal=True), True),
    ("alibi-full-odd", (1, 4, 4, 200, 333, 128), {}, True),
    ("alibi-softcap-window", (1, 4, 4, 256, 256, 64), dict(window_left=64, window_right=32, softcap=20.0), True),
]


@pytest.mark.parametrize("name,shape,opt,use_alibi", FANCY_CASES, ids=[c[0] for c in FANCY_CASES])
def test_backward_follows_softcap_and_alibi(name, shape, opt, use_alibi):
    """The reference's backward operators take alibi_slopes and softcap like its forward
    (flash-attn2-rs/src/host/backward.rs:15-34): the gradients must follow the transformed scores."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward

    dtype = torch.float16
    b, h, hk, sq, sk, d = shape
    q, k, v, do = make_qkv(7, b, h, hk, sq, sk, d, dtype, with_do=True)
    slopes = (torch.arange(1, h + 1, dtype=torch.float32) * 0.05) if use_alibi else None
    sl_gpu = None if slopes is None else slopes.cuda()
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, alibi_slopes=sl_gpu, **opt)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, alibi_slopes=sl_gpu, **opt)
    assert ops.device_status() == 0
    dq_ref, dk_ref, dv_ref, _ = attention_backward(q, k, v, do, out=out.float().cpu(), alibi_slopes=slopes, **opt)
    _close(dq, dq_ref, dtype, "dq")
    _close(dk, dk_ref, dtype, "dk")
    _close(dv, dv_ref, dtype, "dv")


def test_backward_softcap_alibi_through_tvm_ffi_ops():
    import flash_attn2_b200 as fa
    from oracle.attention_oracle import attention_backward

    q, k, v, do = make_qkv(8, 1, 4, 2, 256, 256, 128, torch.bfloat16, with_do=True)
    slopes = torch.tensor([0.1, 0.2, 0.3, 0.4])
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse, _, _ = fa.fwd(qc, kc, vc, alibi_slopes=slopes.cuda(), is_causal=True, softcap=25.0)
    dq, dk, dv, _ = fa.bwd(doc, qc, kc, vc, out, lse, alibi_slopes=slopes.cuda(), is_causal=True, softcap=25.0)
    dq_ref, dk_ref, dv_ref, _ = attention_backward(q, k, v, do, causal=True, out=out.float().cpu(), alibi_slopes=slopes,
                                                   softcap=25.0)
    _close(dq, dq_ref, torch.bfloat16, "dq")
    _close(dk, dk_ref, torch.bfloat16, "dk")
    _close(dv, dv_ref, torch.bfloat16, "dv")


@pytest.mark.parametrize("d", [32, 80, 96])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
def test_forward_and_backward_other_head_dims(d, dtype):
    """Head dims that are multiples of 8 below the kernels' 64 / 128 (the reference buckets 32..256,
    flash-attn2-rs/src/host/tiles.rs:3-127): loads past the real head dim read zeros, stores are clipped."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward, attention_forward
    from tests._cases import FWD_TOL

    q, k, v, do = make_qkv(9, 2, 4, 2, 200, 333, d, dtype, with_do=True)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, causal=True)
    o_ref, lse_ref = attention_forward(q, k, v, causal=True)
    tol = FWD_TOL[dtype]
    torch.testing.assert_close(out.float().cpu(), o_ref, atol=tol["atol"], rtol=tol["rtol"])
    torch.testing.assert_close(lse.cpu(), lse_ref, atol=tol["lse"], rtol=0)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, causal=True)
    assert ops.device_status() == 0
    dq_ref, dk_ref, dv_ref, delta_ref = attention_backward(q, k, v, do, causal=True, out=out.float().cpu())
    torch.testing.assert_close(delta.cpu(), delta_ref, atol=2e-5, rtol=1e-5)
    _close(dq, dq_ref, dtype, "dq")
    _close(dk, dk_ref, dtype, "dk")
    _close(dv, dv_ref, dtype, "dv")


@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
def test_dq_only_call_is_bit_reproducible(causal):
    """which = 1 (the deterministic bwd_dq of the reference, whose dQ kernel sums in registers in key
    order, flash-attn2-rs/src/device/backward/dq.rs:278-279) adds the key blocks in a fixed order:
    repeated runs give identical bits, also with many key blocks per query block and GQA."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward

    q, k, v, do = make_qkv(10, 2, 8, 2, 1536, 1536, 128, torch.bfloat16, with_do=True)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, causal=causal)
    delta = ops.bwd_preprocess(doc, out)
    runs = [ops.bwd(qc, kc, vc, doc, lse, delta, causal=causal, which=1)[0].clone() for _ in range(4)]
    assert ops.device_status() == 0
    for r in runs[1:]:
        assert torch.equal(r, runs[0])
    sl = (slice(1, 2), slice(None), slice(5, 6))
    dq_ref, _, _, _ = attention_backward(q[sl], k[:, :, 1:2][1:2], v[:, :, 1:2][1:2], do[sl], causal=causal,
                                         out=out[sl].float().cpu())
    _close(runs[0][sl], dq_ref, torch.bfloat16, "dq")


TWICE_BWD_CASES = [
    ("B2 H4 S1024 D128 bf16 causal", (2, 4, 4, 1024, 1024, 128), torch.bfloat16, True),
    ("B2 H8/2 S512 D128 f16 causal", (2, 8, 2, 512, 512, 128), torch.float16, True),
    ("B1 H4 S640 D64 bf16 full", (1, 4, 4, 640, 640, 64), torch.bfloat16, False),
    ("B1 H4 S768 D256 bf16 causal", (1, 4, 4, 768, 768, 256), torch.bfloat16, True),
    ("B1 H8/2 S512 D192 f16 full", (1, 8, 2, 512, 512, 192), torch.float16, False),
]


@pytest.mark.parametrize("name,shape,dtype,causal", TWICE_BWD_CASES, ids=[c[0] for c in TWICE_BWD_CASES])
def test_gradient_error_no_larger_than_twice_a_reference_class_kernel(name, shape, dtype, causal):
    """dQ, dK, dV: max|err| against the fp32 oracle must be <= 2x that of an FA2 kernel of the reference's
    family on the same inputs (tests/_cases.py: reference_class_kernel), each kernel differentiating its
    own forward."""
    from oracle.attention_oracle import attention_backward
    from tests._cases import assert_error_within_twice, reference_class_kernel

    b, h, hk, sq, sk, d = shape
    q, k, v, do = make_qkv(2, b, h, hk, sq, sk, d, dtype, with_do=True)
    _, _, _, dq, dk, dv = _run(q, k, v, do, causal=causal)
    qa, ka, va = (t.cuda().requires_grad_() for t in (q, k, v))
    reference_class_kernel().flash_attn_func(qa, ka, va, causal=causal).backward(do.cuda())
    gq, gk, gv, _ = attention_backward(q, k, v, do, causal=causal)
    assert_error_within_twice(name + ":dq", dq, qa.grad, gq)
    assert_error_within_twice(name + ":dk", dk, ka.grad, gk)
    assert_error_within_twice(name + ":dv", dv, va.grad, gv)


@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
def test_ordered_dq_with_more_key_blocks_than_sms(causal):
    """A dQ-only call adds the key blocks of a head in a fixed order, each waiting for the ones before it.
    With more key blocks than the GPU has SMs (160 here) the blocks waited for must already be running:
    the grid lists them in the order of their turns. The status word must stay clean, repeated runs
    must agree bit for bit, and the result must match the call that adds in arrival order."""
    from flash_attn2_b200 import cabi_ops as ops

    s = 160 * 128
    q, k, v, do = [t.cuda() for t in make_qkv(13, 1, 1, 1, s, s, 64, torch.bfloat16, with_do=True)]
    out, lse = ops.fwd(q, k, v, causal=causal)
    delta = ops.bwd_preprocess(do, out)
    a = ops.bwd(q, k, v, do, lse, delta, causal=causal, which=1)[0]
    b = ops.bwd(q, k, v, do, lse, delta, causal=causal, which=1)[0]
    assert ops.device_status() == 0
    assert torch.equal(a, b)
    free = ops.bwd(q, k, v, do, lse, delta, causal=causal, which=3)[0]
    torch.testing.assert_close(a.float(), free.float(), atol=2e-2, rtol=2e-2)
