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


def test_packed_sequences_split_by_cost_over_two_devices():
    """Packed sequences are independent units: split over two GPUs by causal cost (longest first), each GPU runs
    forward and backward on its own packed shard, and the assembled O, LSE, dK, dV equal the one-GPU run of the
    whole batch bit for bit (dQ, summed in arrival order, within tolerance)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from flash_attn2_b200 import cabi_ops as ops
    from flash_attn2_b200.sharding import pack_sequences, shard_sequences_by_cost

    g = torch.Generator().manual_seed(31)
    lengths = [int(x) for x in torch.randint(64, 1025, (12,), generator=g)]
    h, hk, d = 8, 2, 128
    seqs = [[torch.randn(n, heads, d, generator=g).to(torch.bfloat16) for n in lengths] for heads in (h, hk, hk, h)]
    everything = list(range(len(lengths)))

    def run(indices, dev):
        (q, cu), (k, _), (v, _), (do, _) = [pack_sequences(t, indices) for t in seqs]
        q, k, v, do, cu = [t.to(dev) for t in (q, k, v, do, cu)]
        mx = max(lengths[i] for i in indices)
        out, lse = ops.varlen_fwd(q, k, v, cu, cu, mx, mx, causal=True)
        delta = ops.bwd_preprocess(do, out, cu_seqlens_q=cu, max_seqlen_q=mx)
        dq, dk, dv = ops.bwd(q, k, v, do, lse, delta, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=mx,
                             max_seqlen_k=mx, causal=True)
        assert ops.device_status(dev) == 0
        cu = cu.cpu().tolist()
        return {i: [t[cu[n]:cu[n + 1]].cpu() for t in (out, dq, dk, dv)] + [lse[:, cu[n]:cu[n + 1]].cpu()]
                for n, i in enumerate(indices)}

    whole = run(everything, "cuda:0")
    shards = shard_sequences_by_cost(lengths, 2)
    assert sorted(shards[0] + shards[1]) == everything
    cost = [sum(lengths[i] ** 2 for i in s) for s in shards]
    assert max(cost) <= 1.25 * min(cost)
    parts = {}
    for rank, idx in enumerate(shards):
        parts.update(run(idx, f"cuda:{rank}"))
    for i in everything:
        o, dq, dk, dv, lse = parts[i]
        wo, wdq, wdk, wdv, wlse = whole[i]
        assert torch.equal(o, wo) and torch.equal(lse, wlse) and torch.equal(dk, wdk) and torch.equal(dv, wdv), i
        torch.testing.assert_close(dq.float(), wdq.float(), atol=2e-2, rtol=2e-2)
