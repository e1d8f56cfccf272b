"""GPU: fa2_bwd_static, the backward entry point for callers that cannot allocate device memory
(a serving loop with pre-partitioned memory, a runtime that owns the device heap, a sandboxed
plugin host). It keeps the fp32 dQ accumulator in a device array inside the library image instead
of taking one from the caller. The test calls it through the C ABI twice in a row - the shared
array keeps the previous call's contents, so the second call proves it is cleared - and compares
with fa2_bwd and with the CPU oracle on the same inputs; the pipeline status of these calls is read
with fa2_bwd_static_status, which allocates nothing either. It is collected last so that a failure
here cannot hide others.
"""
import ctypes as C

import pytest
import torch

from tests._cases import BWD_TOL, make_qkv

pytestmark = pytest.mark.gpu


def _args(q, k, v, do, lse, delta, dq, dk, dv, causal):
    from flash_attn2_b200 import _cabi

    a = _cabi.BwdArgs()
    a.q, a.k, a.v, a.dout = q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr()
    a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dtype = _cabi.FA2_BF16 if q.dtype == torch.bfloat16 else _cabi.FA2_F16
    b, sq, h, d = q.shape
    a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim = b, sq, k.shape[1], h, k.shape[2], d
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("do_stride", do)):
        setattr(a, name, (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2)))
    a.softmax_scale = 1.0 / d ** 0.5
    a.causal, a.window_left, a.window_right, a.which = int(causal), -1, -1, 3
    return a


def _run_static(q, k, v, do, lse, delta, causal):
    from flash_attn2_b200 import _cabi

    lib = _cabi.load()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    a = _args(q, k, v, do, lse, delta, dq, dk, dv, causal)  # dq_accum stays NULL: it is not used
    _cabi.check(lib.fa2_bwd_static(C.byref(a), torch.cuda.current_stream().cuda_stream))
    assert lib.fa2_bwd_static_status(torch.cuda.current_device()) == 0  # synchronises; 0 = no wait ran out
    return dq, dk, dv


def test_static_backward_matches_fa2_bwd_twice_in_a_row():
    from flash_attn2_b200 import cabi_ops as ops
    from oracle.attention_oracle import attention_backward

    tol = BWD_TOL[torch.bfloat16]
    # two different problems back to back: the second one reuses the accumulator the first one filled
    for seed, (b, h, hk, s), causal in ((11, (2, 4, 2, 384), True), (12, (1, 8, 8, 512), False)):
        host = make_qkv(seed, b, h, hk, s, s, 128, torch.bfloat16, with_do=True)
        q, k, v, do = [t.cuda() for t in host]
        out, lse = ops.fwd(q, k, v, causal=causal)
        delta = ops.bwd_preprocess(do, out)
        ref = ops.bwd(q, k, v, do, lse, delta, causal=causal)
        assert ops.device_status() == 0
        oracle = attention_backward(*host, causal=causal, out=out.float().cpu(), lse=lse.cpu())[:3]
        for _ in range(2):
            got = _run_static(q, k, v, do, lse, delta, causal)
            for g, r, o in zip(got, ref, oracle):
                assert torch.isfinite(g.float()).all()
                torch.testing.assert_close(g.float(), r.float(), atol=tol["atol"], rtol=tol["rtol"])
                torch.testing.assert_close(g.float().cpu(), o, atol=tol["atol"], rtol=tol["rtol"])
            # dK and dV involve no atomics: bit-identical to the allocating entry point
            assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])


def test_static_backward_rejects_what_does_not_fit():
    from flash_attn2_b200 import _cabi

    lib = _cabi.load()
    b, s, h, d = 4, 2048, 8, 128  # 8.4M accumulator elements > FA2_BWD_STATIC_MAX_ELEMENTS
    assert b * s * h * d > _cabi.FA2_BWD_STATIC_MAX_ELEMENTS
    q = torch.empty(b, s, h, d, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(b, h, s, device="cuda")
    a = _args(q, q, q, q, lse, lse, q, q, q, True)
    rc = lib.fa2_bwd_static(C.byref(a), None)
    assert rc == -1 and b"exceeds the built-in accumulator" in lib.fa2_last_error()
