"""GPU (two or more devices): the operators run on the device of their tensors, not on the current one.
The reference binds the context of `q` before every launch
(flash-attn2-rs/src/host/forward/mod.rs:716-718); so do the C ABI calls here."""
import pytest
import torch

from tests._cases import BWD_TOL, FWD_TOL, make_qkv

pytestmark = pytest.mark.gpu


def test_operators_follow_the_tensors_device():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import flash_attn2_b200 as fa
    from oracle.attention_oracle import attention_backward, attention_forward

    q, k, v, do = make_qkv(21, 1, 4, 2, 300, 300, 128, torch.bfloat16, with_do=True)
    torch.cuda.set_device(0)
    q1, k1, v1, do1 = [t.to("cuda:1") for t in (q, k, v, do)]
    assert torch.cuda.current_device() == 0
    out, lse, _, _ = fa.fwd(q1, k1, v1, is_causal=True)
    dq, dk, dv, _ = fa.bwd(do1, q1, k1, v1, out, lse, is_causal=True)
    torch.cuda.synchronize(1)
    assert torch.cuda.current_device() == 0 and out.device.index == 1
    assert fa.cabi_ops.device_status(1) == 0
    o_ref, lse_ref = attention_forward(q, k, v, causal=True)
    ftol, btol = FWD_TOL[torch.bfloat16], BWD_TOL[torch.bfloat16]
    torch.testing.assert_close(out.float().cpu(), o_ref, atol=ftol["atol"], rtol=ftol["rtol"])
    torch.testing.assert_close(lse.cpu(), lse_ref, atol=ftol["lse"], rtol=0)
    refs = attention_backward(q, k, v, do, causal=True, out=out.float().cpu())
    for got, ref in zip((dq, dk, dv), refs):
        torch.testing.assert_close(got.float().cpu(), ref, atol=btol["atol"], rtol=btol["rtol"])
