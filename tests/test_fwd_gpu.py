"""GPU parity of the forward path against the CPU oracle, through the C ABI and the tvm-ffi ops.

Cases follow the reference's forward test (flash-attn2-rs/tests/test_fwd.py:93-134: masks, GQA/MQA,
Sq != Sk, windows, softcap, ALiBi, odd lengths; fp16, D = 128, seed 0) plus the benchmark's workloads at full size.
Tolerances are the reference's own (tests/_cases.py).
"""
from pathlib import Path

import pytest
import torch

from tests._cases import FWD_TOL, alibi_slopes, make_qkv

pytestmark = pytest.mark.gpu

PARITY_CASES = [
    ("full-mha", (2, 4, 4, 256, 256), {}),
    ("causal-mha", (2, 4, 4, 256, 256), dict(causal=True)),
    ("causal-gqa-h8-hk2", (2, 8, 2, 256, 256), dict(causal=True)),
    ("full-mqa-h4-hk1", (1, 4, 1, 192, 192), {}),
    ("causal-sq320-sk256", (1, 4, 4, 320, 256), dict(causal=True)),
    ("full-sq128-sk256", (1, 4, 4, 128, 256), {}),
    ("custom-scale", (2, 4, 4, 256, 256), dict(causal=True, softmax_scale=0.05)),
    ("local-causal-wl64", (2, 4, 4, 256, 256), dict(causal=True, window_left=64)),
    ("window-wl64-wr64", (1, 4, 4, 256, 256), dict(window_left=64, window_right=64)),
    ("softcap30-causal", (2, 4, 4, 256, 256), dict(causal=True, softcap=30.0)),
    ("softcap50-full", (1, 4, 4, 192, 192), dict(softcap=50.0)),
    ("alibi-causal", (2, 4, 4, 256, 256), dict(causal=True, alibi=True)),
    ("alibi-full", (1, 4, 4, 192, 192), dict(alibi=True)),
    ("alibi-local-wl64", (1, 4, 4, 256, 256), dict(causal=True, window_left=64, alibi=True)),
    ("softcap-alibi-gqa-causal", (2, 8, 2, 256, 256), dict(causal=True, softcap=20.0, alibi=True)),
    ("odd-causal-s333", (2, 4, 4, 333, 333), dict(causal=True)),
    ("odd-window-softcap-s300", (1, 4, 4, 300, 300), dict(causal=True, window_left=100, softcap=30.0)),
    ("odd-gqa-causal-s130", (2, 8, 2, 130, 130), dict(causal=True)),
    ("negative-scale", (1, 2, 2, 256, 256), dict(causal=True, softmax_scale=-0.08)),
    ("single-row", (2, 4, 2, 1, 200), {}),
]


def _check(out, lse, o_ref, lse_ref, dtype):
    tol = FWD_TOL[dtype]
    out, lse = out.float().cpu(), lse.float().cpu()
    assert torch.isfinite(out).all()
    empty = torch.isposinf(lse_ref)
    assert (torch.isposinf(lse) == empty).all()
    torch.testing.assert_close(out, o_ref, atol=tol["atol"], rtol=tol["rtol"])
    assert (out - o_ref).abs().mean() < tol["mean"]
    assert (out.transpose(1, 2)[empty] == 0).all()
    torch.testing.assert_close(lse[~empty], lse_ref[~empty], atol=tol["lse"], rtol=0)


@pytest.mark.parametrize("name,shape,opt", PARITY_CASES, ids=[c[0] for c in PARITY_CASES])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
def test_forward_parity_cabi(name, shape, opt, dtype):
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_forward

    b, h, hk, sq, sk = shape
    opt = dict(opt)
    q, k, v = make_qkv(0, b, h, hk, sq, sk, 128, dtype)
    slopes = alibi_slopes(h) if opt.pop("alibi", False) else None
    o_ref, lse_ref = attention_forward(q, k, v, alibi_slopes=slopes, **opt)
    out, lse = ops.fwd(q.cuda(), k.cuda(), v.cuda(), alibi_slopes=None if slopes is None else slopes.cuda(), **opt)
    assert ops.device_status() == 0
    _check(out, lse, o_ref, lse_ref, dtype)


def test_config1_d64_fp16_noncausal():
    """The reference's own CPU-runnable case: B1 H4 S128 D64 fp16, seed 0, scale 1/8."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_forward

    q, k, v = make_qkv(0, 1, 4, 4, 128, 128, 64, torch.float16)
    o_ref, lse_ref = attention_forward(q, k, v, softmax_scale=0.125)
    out, lse = ops.fwd(q.cuda(), k.cuda(), v.cuda(), softmax_scale=0.125)
    assert ops.device_status() == 0
    _check(out, lse, o_ref, lse_ref, torch.float16)


@pytest.mark.parametrize("shape,opt", [((2, 4, 2, 512, 512), dict(causal=True)), ((1, 2, 2, 200, 777), {}),
                                       ((1, 3, 1, 700, 300), dict(causal=True))])
def test_forward_d64(shape, opt):
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_forward

    b, h, hk, sq, sk = shape
    q, k, v = make_qkv(3, b, h, hk, sq, sk, 64, torch.bfloat16)
    o_ref, lse_ref = attention_forward(q, k, v, **opt)
    out, lse = ops.fwd(q.cuda(), k.cuda(), v.cuda(), **opt)
    assert ops.device_status() == 0
    _check(out, lse, o_ref, lse_ref, torch.bfloat16)


def test_forward_matches_reference_golden_vectors():
    """The D=64 golden case produced by the reference's own naive attention."""
    from flash_attn2_b200 import cabi_ops as ops
    from tests.golden.make_golden import CASES, make_inputs

    gold = torch.load(Path(__file__).parent / "golden" / "reference_attention.pt")
    idx = [c[0] for c in CASES].index("cfg1-b1-h4-s128-d64")
    _, b, h, hk, sq, sk, d, _ = CASES[idx]
    q, k, v = make_inputs(idx, b, h, hk, sq, sk, d)
    out, lse = ops.fwd(q.cuda(), k.cuda(), v.cuda())
    _check(out, lse, gold["cfg1-b1-h4-s128-d64"]["out"].float(), gold["cfg1-b1-h4-s128-d64"]["lse"], torch.float16)


def test_forward_strided_views_and_supplied_out():
    """Head-sharded strided views (outer strides multiples of 8 elements) need no packing copy."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_forward

    q, k, v = make_qkv(4, 1, 8, 8, 384, 384, 128, torch.bfloat16)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    out_full = torch.zeros_like(qc)
    for h0 in (0, 4):
        sl = slice(h0, h0 + 4)
        out, lse = ops.fwd(qc[:, :, sl], kc[:, :, sl], vc[:, :, sl], out=out_full[:, :, sl], causal=True)
        o_ref, lse_ref = attention_forward(q[:, :, sl], k[:, :, sl], v[:, :, sl], causal=True)
        _check(out, lse, o_ref, lse_ref, torch.bfloat16)
    o_ref, _ = attention_forward(q, k, v, causal=True)
    torch.testing.assert_close(out_full.float().cpu(), o_ref, atol=1e-2, rtol=5e-2)
    with pytest.raises(ValueError):  # 2-byte misaligned base
        ops.fwd(qc.view(-1)[1:1 + 384 * 7 * 128].view(1, 384, 7, 128), kc[:, :, :7], vc[:, :, :7])


def test_forward_empty_shapes():
    from flash_attn2_b200 import cabi_ops as ops

    q = torch.randn(2, 5, 3, 128, device="cuda", dtype=torch.float16)
    k = torch.randn(2, 0, 3, 128, device="cuda", dtype=torch.float16)
    out, lse = ops.fwd(q, k, k)
    assert (out == 0).all() and torch.isposinf(lse).all()
    out, lse = ops.fwd(q[:, :0], q, q)
    assert out.shape == (2, 0, 3, 128) and lse.shape == (2, 3, 0)


WIDE_CASES = [
    ("d256-full", 256, (1, 2, 2, 128, 128), {}),
    ("d256-causal-gqa", 256, (2, 8, 2, 333, 333), dict(causal=True)),
    ("d192-causal", 192, (2, 4, 4, 512, 512), dict(causal=True)),
    ("d192-sq320-sk256-causal", 192, (1, 4, 4, 320, 256), dict(causal=True)),
    ("d160-mqa-sq128-sk700", 160, (1, 4, 1, 128, 700), {}),
    ("d136-window-wl64-wr64", 136, (1, 4, 4, 256, 256), dict(window_left=64, window_right=64)),
    ("d256-local-causal-wl100-softcap", 256, (1, 4, 4, 300, 300), dict(causal=True, window_left=100, softcap=30.0)),
    ("d192-alibi-causal", 192, (2, 4, 4, 256, 256), dict(causal=True, alibi=True)),
    ("d256-alibi-full", 256, (1, 4, 4, 192, 192), dict(alibi=True)),
    ("d224-negative-scale", 224, (1, 2, 2, 256, 256), dict(causal=True, softmax_scale=-0.08)),
    ("d256-single-row", 256, (2, 4, 2, 1, 200), {}),
    ("d192-rows-without-keys", 192, (1, 2, 2, 300, 100), dict(causal=True)),
    ("d256-long", 256, (1, 2, 2, 1500, 2100), dict(causal=True)),
]


@pytest.mark.parametrize("name,d,shape,opt", WIDE_CASES, ids=[c[0] for c in WIDE_CASES])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
def test_forward_head_dims_above_128(name, d, shape, opt, dtype):
    """Head dims 136..256 (the reference's 192 and 256 buckets, flash-attn2-rs/src/host/tiles.rs:1) run on the
    kernel with 64-key tiles; the cases repeat the masks and transforms of the D = 128 parity list."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_forward

    b, h, hk, sq, sk = shape
    opt = dict(opt)
    q, k, v = make_qkv(5, b, h, hk, sq, sk, d, dtype)
    slopes = alibi_slopes(h) if opt.pop("alibi", False) else None
    o_ref, lse_ref = attention_forward(q, k, v, alibi_slopes=slopes, **opt)
    out, lse = ops.fwd(q.cuda(), k.cuda(), v.cuda(), alibi_slopes=None if slopes is None else slopes.cuda(), **opt)
    assert ops.device_status() == 0
    _check(out, lse, o_ref, lse_ref, dtype)


def test_rejects_unsupported_inputs():
    """flash-attn2-rs/tests/test_fwd.py:172-181."""
    import flash_attn2_b200 as fa

    for head_size, dtype in [(264, torch.float16), (9, torch.float16), (128, torch.float32)]:
        q = torch.randn(1, 128, 4, head_size, device="cuda", dtype=dtype)
        with pytest.raises((NotImplementedError, ValueError, TypeError)):
            fa.fwd_explicit(q, q, q, None, None, False, -1, -1, 0.0)
        with pytest.raises((NotImplementedError, ValueError, TypeError)):
            fa.cabi_ops.fwd(q, q, q)


def test_forward_through_tvm_ffi_ops():
    """fwd_explicit (ops.fwd -> Array[out, lse]) and fwd (ops.fwd_lse with a supplied out)."""
    import flash_attn2_b200 as fa
    from oracle.attention_oracle import attention_forward

    q, k, v = make_qkv(0, 2, 8, 2, 256, 256, 128, torch.float16)
    o_ref, lse_ref = attention_forward(q, k, v, causal=True)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    out, lse = fa.fwd_explicit(qc, kc, vc, None, None, True, -1, -1, 0.0)
    _check(out, lse, o_ref, lse_ref, torch.float16)
    out2, lse2, probs, state = fa.fwd(qc, kc, vc, is_causal=True)
    _check(out2, lse2, o_ref, lse_ref, torch.float16)
    assert probs.numel() == 0 and state.shape == (2,)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    # on a side stream the operator must use the caller's current stream
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        out3, lse3 = fa.fwd_explicit(qc, kc, vc, None, None, True, -1, -1, 0.0)
    s.synchronize()
    assert torch.equal(out, out3)


def _full_size_inputs(seed, with_do=False):
    g = torch.Generator().manual_seed(seed)
    n = 4 if with_do else 3
    return [torch.randn(16, 2048, 16, 128, generator=g).to(torch.bfloat16) for _ in range(n)]


def test_config2_full_size_slices_and_properties():
    """The benchmark's forward workload (B16 H16 S2048 D128 bf16 causal, seed 1) at full size: oracle on sampled (batch, head) units, plus properties
    that need no oracle (V = 1 gives O = 1; O is linear in V; first row attends only key 0)."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_forward

    q, k, v = _full_size_inputs(1)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    out, lse = ops.fwd(qc, kc, vc, causal=True)
    assert ops.device_status() == 0
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    from tests._cases import assert_error_within_twice, reference_class_kernel, sample_units

    theirs, their_lse, _ = reference_class_kernel().flash_attn_func(qc, kc, vc, causal=True, return_attn_probs=True)
    for b, h in sample_units(16, 16):
        o_ref, lse_ref = attention_forward(q[b:b + 1, :, h:h + 1], k[b:b + 1, :, h:h + 1], v[b:b + 1, :, h:h + 1],
                                           causal=True)
        _check(out[b:b + 1, :, h:h + 1], lse[b:b + 1, h:h + 1], o_ref, lse_ref, torch.bfloat16)
        assert_error_within_twice("B16 H16 S2048 causal:out", out[b:b + 1, :, h:h + 1], theirs[b:b + 1, :, h:h + 1], o_ref)
        assert_error_within_twice("B16 H16 S2048 causal:lse", lse[b:b + 1, h:h + 1], their_lse[b:b + 1, h:h + 1], lse_ref)
    del theirs, their_lse
    torch.testing.assert_close(out[:, 0].float(), vc[:, 0].float(), atol=0, rtol=0)  # row 0 sees key 0 only
    ones, _ = ops.fwd(qc, kc, torch.ones_like(vc), causal=True)
    torch.testing.assert_close(ones.float(), torch.ones_like(ones, dtype=torch.float32), atol=8e-3, rtol=0)
    out2, lse2 = ops.fwd(qc, kc, vc * 2, causal=True)
    assert torch.equal(lse, lse2)
    torch.testing.assert_close(out2.float(), out.float() * 2, atol=1.6e-2, rtol=1.6e-2)
    out3, _ = ops.fwd(qc, kc, vc, causal=True)
    assert torch.equal(out, out3)  # run-to-run deterministic


TWICE_CASES = [
    ("B1 H4 S128 D64 f16 full", 0, (1, 4, 4, 128, 128, 64), torch.float16, dict(softmax_scale=0.125)),
    ("B2 H4 S1024 D128 bf16 causal", 1, (2, 4, 4, 1024, 1024, 128), torch.bfloat16, dict(causal=True)),
    ("B2 H8/2 S512 D128 f16 causal", 1, (2, 8, 2, 512, 512, 128), torch.float16, dict(causal=True)),
    ("B1 H4 S777 D128 bf16 full", 1, (1, 4, 4, 777, 777, 128), torch.bfloat16, {}),
    ("B2 H4 S1024 D256 bf16 causal", 1, (2, 4, 4, 1024, 1024, 256), torch.bfloat16, dict(causal=True)),
    ("B1 H8/2 S640 D192 f16 full", 1, (1, 8, 2, 640, 640, 192), torch.float16, {}),
]


@pytest.mark.parametrize("name,seed,shape,dtype,opt", TWICE_CASES, ids=[c[0] for c in TWICE_CASES])
def test_error_no_larger_than_twice_a_reference_class_kernel(name, seed, shape, dtype, opt):
    """O and LSE: max|err| against the fp32 oracle must be <= 2x that of an FA2 kernel of the reference's
    family on the same inputs (tests/_cases.py: reference_class_kernel). The first case is the
    reference's own CPU-runnable configuration (B1 H4 S128 D64 fp16, seed 0, scale 1/8)."""
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_forward
    from tests._cases import assert_error_within_twice, reference_class_kernel

    b, h, hk, sq, sk, d = shape
    q, k, v = make_qkv(seed, b, h, hk, sq, sk, d, dtype)
    kw = dict(causal=opt.get("causal", False), softmax_scale=opt.get("softmax_scale"))
    theirs, their_lse, _ = reference_class_kernel().flash_attn_func(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True, **kw)
    o_ref, lse_ref = attention_forward(q, k, v, **opt)
    ours, lse = ops.fwd(q.cuda(), k.cuda(), v.cuda(), **opt)
    assert ops.device_status() == 0
    assert_error_within_twice(name + ":out", ours, theirs, o_ref)
    assert_error_within_twice(name + ":lse", lse, their_lse, lse_ref)


def test_unaddressable_views_are_packed_by_the_operator_layer():
    """Views whose base is not 16-byte aligned or whose outer strides are not multiples of 8 elements go
    through the packing copy of the operator layer (the reference packs them as well,
    flash-attn2-rs/src/host/layout.rs:80-100); forward and backward must match the oracle on them."""
    import flash_attn2_b200 as fa
    from oracle.attention_oracle import attention_backward, attention_forward
    from tests._cases import BWD_TOL

    g = torch.Generator().manual_seed(11)
    b, s, h, d = 1, 200, 3, 128
    big = [torch.randn(b, s, h, d + 1, generator=g).to(torch.float16) for _ in range(4)]
    views_cpu = [t[..., 1:] for t in big]                      # base off by 2 bytes, row stride 3 * 129
    q, k, v, do = [t.cuda()[..., 1:] for t in big]
    assert q.data_ptr() % 16 != 0 and q.stride(1) % 8 != 0
    out, lse, _, _ = fa.fwd(q, k, v, is_causal=True)
    o_ref, lse_ref = attention_forward(*[t.contiguous() for t in views_cpu[:3]], causal=True)
    _check(out, lse, o_ref, lse_ref, torch.float16)
    dq, dk, dv, _ = fa.bwd(do, q, k, v, out, lse, is_causal=True)
    dq_ref, dk_ref, dv_ref, _ = attention_backward(*[t.contiguous() for t in views_cpu], causal=True,
                                                   out=out.float().cpu())
    tol = BWD_TOL[torch.float16]
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        torch.testing.assert_close(got.float().cpu(), ref, atol=tol["atol"], rtol=tol["rtol"])


def test_supplied_out_layouts():
    """A caller-supplied `out` (flash-attn2-rs/src/host/forward/mod.rs:349-375, tests/test_gold.py:119-256): written
    in place when the kernels can address it and it shares no memory with an input, otherwise through a
    temporary and a copy; refused when its own elements overlap."""
    import flash_attn2_b200 as fa

    g = torch.Generator().manual_seed(5)
    # rows outside a simple stride nesting: shape (2, 2049, 2, 16) with strides (40, 88, 64, 1)
    q = torch.randn(2, 2049, 2, 16, generator=g).to(torch.float16).cuda()
    kv = q[:, :1]
    want = fa.fwd(q, kv, kv)[0]
    out = torch.empty(180344, device="cuda", dtype=q.dtype).as_strided(q.shape, (40, 88, 64, 1))
    got = fa.fwd(q, kv, kv, out=out)[0]
    assert got.data_ptr() == out.data_ptr()
    assert torch.equal(got, want)
    # a base that is off by one element: computed aside and copied, the element in front stays untouched
    q2 = torch.randn(2, 33, 4, 64, generator=g).to(torch.bfloat16).cuda()
    k2 = torch.randn(2, 47, 2, 64, generator=g).to(torch.bfloat16).cuda()
    want2 = fa.fwd(q2, k2, k2, is_causal=True)[0]
    storage = torch.full((q2.numel() + 1,), 123.0, device="cuda", dtype=q2.dtype)
    got2 = fa.fwd(q2, k2, k2, out=storage[1:].view(q2.shape), is_causal=True)[0]
    assert storage[0] == 123 and torch.equal(got2, want2)
    # out aliases q: the inputs must be read before anything is written over them
    q3 = q2.clone()
    got3 = fa.fwd(q3, k2, k2, out=q3, is_causal=True)[0]
    assert got3.data_ptr() == q3.data_ptr() and torch.equal(got3, want2)
    # a head-sliced view of a larger output is written in place
    big = torch.zeros(2, 33, 8, 64, device="cuda", dtype=q2.dtype)
    got4 = fa.fwd(q2, k2, k2, out=big[:, :, 2:6], is_causal=True)[0]
    assert torch.equal(got4, want2) and (big[:, :, :2] == 0).all() and (big[:, :, 6:] == 0).all()
    # elements that overlap each other cannot be a destination
    bad = torch.empty(33 * 4 * 64, device="cuda", dtype=q2.dtype).as_strided(q2.shape, (0, 4 * 64, 64, 1))
    with pytest.raises((ValueError, RuntimeError)):
        fa.fwd(q2, k2, k2, out=bad)
