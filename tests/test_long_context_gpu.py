"""GPU: the long-context configuration, B=1, H_q=H_kv=32, S=16384, D=128, bf16, causal, Q/K/V/dO ~ N(0,1)
from seed 4, forward and backward on one GPU, and its 4-of-32-heads shard as a strided view (what one of
eight GPUs runs when the heads are split) against the same heads as a contiguous copy.

The oracle needs 1 GiB per fp32 score matrix of one head, so it runs on whole heads one at a time.
"""
import pytest
import torch

from tests._cases import BWD_TOL, FWD_TOL

pytestmark = pytest.mark.gpu

S, H, D = 16384, 32, 128
ORACLE_HEADS = (0, 17, 31)


def _inputs():
    g = torch.Generator().manual_seed(4)
    return [torch.randn(1, S, H, D, generator=g).to(torch.bfloat16) for _ in range(4)]  # q, k, v, dO


def test_long_context_forward_backward_and_head_shards():
    from flash_attn2_b200 import cabi_ops as ops
    from flash_attn2_b200.sharding import shard_heads
    from oracle.attention_oracle import attention_backward, attention_forward
    from tests._cases import assert_error_within_twice, reference_class_kernel

    q, k, v, do = _inputs()
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse = ops.fwd(qc, kc, vc, causal=True)
    delta = ops.bwd_preprocess(doc, out)
    dq, dk, dv = ops.bwd(qc, kc, vc, doc, lse, delta, causal=True)
    assert ops.device_status() == 0
    for t in (out, lse, dq, dk, dv):
        assert torch.isfinite(t.float()).all()

    qa, ka, va = (t.clone().requires_grad_() for t in (qc, kc, vc))
    theirs, their_lse, _ = reference_class_kernel().flash_attn_func(qa, ka, va, causal=True, return_attn_probs=True)
    theirs.backward(doc)
    ftol, btol = FWD_TOL[torch.bfloat16], BWD_TOL[torch.bfloat16]
    for h in ORACLE_HEADS:
        sl = (slice(None), slice(None), slice(h, h + 1))
        o_ref, lse_ref = attention_forward(q[sl], k[sl], v[sl], causal=True)
        torch.testing.assert_close(out[sl].float().cpu(), o_ref, atol=ftol["atol"], rtol=ftol["rtol"])
        torch.testing.assert_close(lse[:, h:h + 1].cpu(), lse_ref, atol=ftol["lse"], rtol=0)
        assert_error_within_twice("S16384 causal:out", out[sl], theirs[sl].detach(), o_ref)
        assert_error_within_twice("S16384 causal:lse", lse[:, h:h + 1], their_lse[:, h:h + 1], lse_ref)
        gq, gk, gv, _ = attention_backward(q[sl], k[sl], v[sl], do[sl], causal=True, out=o_ref, lse=lse_ref)
        for name, got, ref, their in (("dq", dq, gq, qa.grad), ("dk", dk, gk, ka.grad), ("dv", dv, gv, va.grad)):
            torch.testing.assert_close(got[sl].float().cpu(), ref, atol=btol["atol"], rtol=btol["rtol"])
            assert_error_within_twice("S16384 causal:" + name, got[sl], their[sl], ref)
        del o_ref, lse_ref, gq, gk, gv
    del qa, ka, va, theirs, their_lse

    # The shard of rank 5 of 8: heads 20..23, as a strided view of the full tensors and as a copy.
    hq, hkv = shard_heads(H, H, 8, 5)
    assert (hq.start, hq.stop) == (20, 24) and hq == hkv
    views = [t[:, :, hq] for t in (qc, kc, vc, doc)]
    assert not views[0].is_contiguous()
    copies = [t.contiguous() for t in views]
    res = []
    for a, b, c, d_ in (views, copies):
        o, l = ops.fwd(a, b, c, causal=True)
        dl = ops.bwd_preprocess(d_, o)
        res.append((o, l, dl) + tuple(ops.bwd(a, b, c, d_, l, dl, causal=True)))
    assert ops.device_status() == 0
    (o1, l1, dl1, dq1, dk1, dv1), (o2, l2, dl2, dq2, dk2, dv2) = res
    assert torch.equal(o1, o2) and torch.equal(l1, l2) and torch.equal(dl1, dl2)
    assert torch.equal(dk1, dk2) and torch.equal(dv1, dv2)
    torch.testing.assert_close(dq1.float(), dq2.float(), atol=2e-2, rtol=2e-2)  # fp32 adds land in arrival order
    # ... and it is the same as those heads of the unsharded run
    assert torch.equal(o1, out[:, :, hq]) and torch.equal(l1, lse[:, hq])
    assert torch.equal(dk1, dk[:, :, hkv]) and torch.equal(dv1, dv[:, :, hkv])
