"""Generates tests/golden/reference_attention.pt from the reference's own test oracle.

Runs only where the reference checkout is mounted (its path is the one argument). It imports `reference_attention` from flash-attn2-rs/tests/test_fwd.py — the
crate's test-harness naive attention — with a stub for the `kernels` loader that module needs at
import time, evaluates it on small seeded CPU inputs that cover the mask / GQA / softcap / ALiBi /
ragged cases of that file's PARITY_CASES, and stores inputs' seeds and the outputs. The oracle in
oracle/attention_oracle.py is pinned against these vectors by tests/test_oracle.py.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import torch

# (name, batch, heads, heads_k, seqlen_q, seqlen_k, head_dim, options)
CASES = [
    ("full-mha", 2, 4, 4, 64, 64, 32, {}),
    ("causal-mha", 2, 4, 4, 64, 64, 32, {"causal": True}),
    ("causal-gqa-h8-hk2", 1, 8, 2, 96, 96, 32, {"causal": True}),
    ("full-mqa-h4-hk1", 1, 4, 1, 48, 48, 32, {}),
    ("causal-sq80-sk64", 1, 4, 4, 80, 64, 32, {"causal": True}),
    ("full-sq32-sk64", 1, 4, 4, 32, 64, 32, {}),
    ("custom-scale", 1, 4, 4, 64, 64, 32, {"causal": True, "softmax_scale": 0.05}),
    ("local-causal-wl16", 1, 4, 4, 64, 64, 32, {"causal": True, "window_left": 16}),
    ("window-wl16-wr16", 1, 4, 4, 64, 64, 32, {"window_left": 16, "window_right": 16}),
    ("softcap30-causal", 1, 4, 4, 64, 64, 32, {"causal": True, "softcap": 30.0}),
    ("alibi-causal", 1, 4, 4, 64, 64, 32, {"causal": True, "alibi": True}),
    ("alibi-full", 1, 4, 4, 48, 48, 32, {"alibi": True}),
    ("alibi-local-wl16", 1, 4, 4, 64, 64, 32, {"causal": True, "window_left": 16, "alibi": True}),
    ("odd-causal-s83", 2, 4, 4, 83, 83, 32, {"causal": True}),
    ("cfg1-b1-h4-s128-d64", 1, 4, 4, 128, 128, 64, {}),
]


def make_inputs(seed, b, h, hk, sq, sk, d, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, sq, h, d, generator=g).to(dtype)
    k = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    v = torch.randn(b, sk, hk, d, generator=g).to(dtype)
    return q, k, v


def main(ref_root: str) -> None:
    sys.modules.setdefault("kernels", types.SimpleNamespace(get_kernel=lambda *a, **k: None))
    path = Path(ref_root) / "flash-attn2-rs" / "tests" / "test_fwd.py"
    spec = importlib.util.spec_from_file_location("ref_test_fwd", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {}
    for i, (name, b, h, hk, sq, sk, d, opt) in enumerate(CASES):
        opt = dict(opt)
        q, k, v = make_inputs(i, b, h, hk, sq, sk, d)
        if opt.pop("alibi", False):
            opt["alibi_slopes"] = 2.0 ** (-8.0 * (torch.arange(h).float() + 1) / h)
        o, lse = mod.reference_attention(q, k, v, **opt)
        out[name] = {"seed": i, "out": o.contiguous().half(), "lse": lse.contiguous()}
    dst = Path(__file__).resolve().parent / "reference_attention.pt"
    torch.save(out, dst)
    print(f"wrote {dst} ({dst.stat().st_size} bytes, {len(out)} cases)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
