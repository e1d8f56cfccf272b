"""GPU: nothing is written outside an output or a workspace.

Every tensor the C-ABI wrappers allocate (O, LSE, delta, dQ, dK, dV, the fp32 dQ accumulator) is placed inside
a larger buffer whose margins hold a bit pattern; after forward, delta preprocess and backward on ragged
shapes (dense and packed, head dims on both kernel families) the margins must be untouched. TMA stores are
clipped by the hardware; the predicated stores, the reductions and the conversion kernels are what this
watches. It stands in for the memory checker that cannot run on this pool.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

PAD = 4096  # elements on each side


class Canaries:
    def __init__(self):
        self.buffers = []

    def alloc(self, shape, dtype, device):
        n = 1
        for s in shape:
            n *= int(s)
        word = torch.int16 if dtype in (torch.float16, torch.bfloat16) else torch.int32
        raw = torch.full((n + 2 * PAD,), 0x5A5A if word == torch.int16 else 0x5A5A5A5A, dtype=word, device=device)
        self.buffers.append(raw)
        return raw[PAD:PAD + n].view(dtype).view(tuple(int(s) for s in shape))

    def check(self):
        torch.cuda.synchronize()
        for i, raw in enumerate(self.buffers):
            pattern = 0x5A5A if raw.dtype == torch.int16 else 0x5A5A5A5A
            assert (raw[:PAD] == pattern).all(), f"buffer {i}: written before its start"
            assert (raw[-PAD:] == pattern).all(), f"buffer {i}: written past its end"


DENSE = [(2, 4, 2, 333, 333, 128, True), (1, 3, 1, 200, 777, 64, False), (1, 2, 2, 130, 70, 96, True),
         (2, 4, 2, 333, 333, 256, True), (1, 3, 1, 200, 777, 192, False), (1, 2, 2, 130, 70, 136, True),
         (1, 2, 2, 1, 200, 128, False), (1, 2, 2, 65, 129, 256, False)]


@pytest.mark.parametrize("shape", DENSE, ids=[f"b{s[0]}-h{s[1]}/{s[2]}-sq{s[3]}-sk{s[4]}-d{s[5]}" for s in DENSE])
def test_dense_outputs_stay_inside_their_buffers(shape, monkeypatch):
    from flash_attn2_b200 import cabi_ops as ops
    from tests._cases import make_qkv

    b, h, hk, sq, sk, d, causal = shape
    q, k, v, do = [t.cuda() for t in make_qkv(21, b, h, hk, sq, sk, d, torch.bfloat16, with_do=True)]
    can = Canaries()
    monkeypatch.setattr(ops, "_alloc", can.alloc)
    out, lse = ops.fwd(q, k, v, causal=causal)
    delta = ops.bwd_preprocess(do, out)
    ops.bwd(q, k, v, do, lse, delta, causal=causal)
    assert ops.device_status() == 0
    assert len(can.buffers) == 7
    can.check()


@pytest.mark.parametrize("d", [64, 96, 128, 192, 256])
def test_packed_outputs_stay_inside_their_buffers(d, monkeypatch):
    from flash_attn2_b200 import cabi_ops as ops

    lengths = [130, 7, 257, 0, 64, 300]
    g = torch.Generator().manual_seed(22)
    total = sum(lengths)
    q = torch.randn(total, 4, d, generator=g).to(torch.float16).cuda()
    k = torch.randn(total, 2, d, generator=g).to(torch.float16).cuda()
    v = torch.randn(total, 2, d, generator=g).to(torch.float16).cuda()
    do = torch.randn(total, 4, d, generator=g).to(torch.float16).cuda()
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32).cuda()
    can = Canaries()
    monkeypatch.setattr(ops, "_alloc", can.alloc)
    out, lse = ops.varlen_fwd(q, k, v, cu, cu, max(lengths), max(lengths), causal=True)
    delta = ops.bwd_preprocess(do, out, cu_seqlens_q=cu, max_seqlen_q=max(lengths))
    ops.bwd(q, k, v, do, lse, delta, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lengths),
            max_seqlen_k=max(lengths), causal=True)
    assert ops.device_status() == 0
    can.check()
