"""Seeded inputs shared by the parity tests (CPU tensors; the reference benchmark's fixture
convention: torch.Generator().manual_seed(seed), randn in the order q, k, v[, dO], cast, copy)."""
import torch


def make_qkv(seed, b, h, hk, sq, sk, d, dtype, with_do=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, sq, h, d, generator=g).to(dtype)
    k = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    v = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    if with_do:
        return q, k, v, torch.randn(b, sq, h, d, generator=g).to(dtype)
    return q, k, v


def alibi_slopes(h):
    return 2.0 ** (-8.0 * (torch.arange(h).float() + 1) / h)


# Absolute tolerances of the reference's own tests for this path
# (flash-attn2-rs/tests/test_fwd.py:160-168, tests/test_gold.py:275,363,1264-1267).
FWD_TOL = {torch.float16: dict(atol=2e-3, rtol=2.5e-2, mean=2e-3, lse=3e-2),
           torch.bfloat16: dict(atol=1e-2, rtol=5e-2, mean=8e-3, lse=8e-2)}
BWD_TOL = {torch.float16: dict(atol=0.008, rtol=0.04), torch.bfloat16: dict(atol=0.06, rtol=0.08)}
