"""Run by tests/test_dropin_gpu.py in a child pytest whose import path is the prepared copy of the reference's
Python package (baseline/_ref): its six autograd wrappers and its torch custom-op registration, on top of this
repository's operator library, against the gold kernel. The cases follow the reference's own
flash-attn2-rs/tests/test_gold.py:366-424 (test_autograd: head size 63, which the wrappers pad; GQA; an empty
second sequence in the packed forms) with dropout off, which that test does not cover and this library does
not build, and add a compiled forward + backward through the registered custom ops.
"""
import kernels
import pytest
import torch

rs = kernels.get_kernel("kernels-community-rs/flash-attn2-rs", version=1)
gold = kernels.get_kernel("kernels-community/flash-attn2", version=4)

FUNCTIONS = ["flash_attn_func", "flash_attn_qkvpacked_func", "flash_attn_kvpacked_func", "flash_attn_varlen_func",
             "flash_attn_varlen_qkvpacked_func", "flash_attn_varlen_kvpacked_func"]


def _inputs(function, head_dim):
    torch.manual_seed(0)
    q = torch.randn(1, 17, 4, head_dim, device="cuda", dtype=torch.float16)
    k = torch.randn(1, 23, 2, head_dim, device="cuda", dtype=q.dtype)
    v = torch.randn_like(k)
    cu_q = torch.tensor([0, 17, 17], device="cuda", dtype=torch.int32)
    cu_k = torch.tensor([0, 23, 23], device="cuda", dtype=torch.int32)
    qv, kv, vv = q[0], k[0], v[0]
    return {
        "flash_attn_func": ((q, k, v), ()),
        "flash_attn_qkvpacked_func": ((torch.stack((q, q, q), 2),), ()),
        "flash_attn_kvpacked_func": ((q, torch.stack((k, v), 2)), ()),
        "flash_attn_varlen_func": ((qv, kv, vv), (cu_q, cu_k, 17, 23)),
        "flash_attn_varlen_qkvpacked_func": ((torch.stack((qv, qv, qv), 1),), (cu_q, 17)),
        "flash_attn_varlen_kvpacked_func": ((qv, torch.stack((kv, vv), 1)), (cu_q, cu_k, 17, 23)),
    }[function]


@pytest.mark.parametrize("head_dim", [63, 128, 200])
@pytest.mark.parametrize("function", FUNCTIONS)
def test_wrappers_forward_and_gradients(function, head_dim):
    inputs, metadata = _inputs(function, head_dim)
    ours = [x.detach().requires_grad_() for x in inputs]
    theirs = [x.detach().requires_grad_() for x in inputs]
    actual = getattr(rs, function)(*ours, *metadata, dropout_p=0.0, causal=True)
    expected = getattr(gold, function)(*theirs, *metadata, dropout_p=0.0, causal=True)
    torch.testing.assert_close(actual, expected, atol=0.005, rtol=0.03)
    got = torch.autograd.grad(actual.sum(), ours)
    want = torch.autograd.grad(expected.sum(), theirs)
    for g, w in zip(got, want):
        torch.testing.assert_close(g, w, atol=0.008, rtol=0.04)


def test_compiled_forward_and_backward():
    """torch.compile traces through the package's registered custom ops (fake implementations, autograd)."""
    torch.manual_seed(1)
    q = torch.randn(2, 96, 4, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(2, 96, 2, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(2, 96, 2, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)

    def f(q, k, v):
        return rs.flash_attn_func(q, k, v, causal=True).float().square().sum()

    eager = f(q, k, v)
    eager_grads = torch.autograd.grad(eager, (q, k, v))
    compiled = torch.compile(f, fullgraph=True)
    out = compiled(q, k, v)
    grads = torch.autograd.grad(out, (q, k, v))
    torch.testing.assert_close(out, eager, atol=1e-2, rtol=1e-3)
    for g, e in zip(grads, eager_grads):
        torch.testing.assert_close(g, e, atol=2e-2, rtol=2e-2)
