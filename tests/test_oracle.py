"""CPU: the oracle against the golden vectors made from the reference's own test oracle, and
internal consistency of its backward (explicit formulas == autograd through the forward)."""
from pathlib import Path

import pytest
import torch

from oracle.attention_oracle import attention_backward, attention_forward, varlen_forward
from tests._cases import alibi_slopes, make_qkv
from tests.golden.make_golden import CASES, make_inputs

GOLDEN = torch.load(Path(__file__).parent / "golden" / "reference_attention.pt")


@pytest.mark.parametrize("idx", range(len(CASES)), ids=[c[0] for c in CASES])
def test_oracle_matches_reference_golden(idx):
    name, b, h, hk, sq, sk, d, opt = CASES[idx]
    opt = dict(opt)
    q, k, v = make_inputs(idx, b, h, hk, sq, sk, d)
    if opt.pop("alibi", False):
        opt["alibi_slopes"] = alibi_slopes(h)
    out, lse = attention_forward(q, k, v, **opt)
    gold = GOLDEN[name]
    assert gold["seed"] == idx
    g_out, g_lse = gold["out"].float(), gold["lse"]
    # The naive reference yields NaN rows / -inf LSE where no key is visible; the kernels (and the
    # oracle) define O = 0 and LSE = +inf there (tests/test_fwd.py:164-168 of the reference).
    empty = torch.isneginf(g_lse)
    assert (torch.isposinf(lse) == empty).all()
    fin = ~empty
    torch.testing.assert_close(lse[fin], g_lse[fin], atol=1e-5, rtol=1e-5)
    fin_o = fin.transpose(1, 2).unsqueeze(-1).expand_as(out)
    torch.testing.assert_close(out[fin_o], g_out[fin_o], atol=1e-3, rtol=1e-3)  # golden O stored as fp16
    assert (out[~fin_o] == 0).all()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("hk", [4, 2])
def test_oracle_backward_matches_autograd(causal, hk):
    q, k, v, do = make_qkv(5, 2, 4, hk, 70, 70, 32, torch.float32, with_do=True)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    # autograd through plain softmax attention
    g = 4 // hk
    s = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(g, 2)) / (32 ** 0.5)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(70, 70, dtype=torch.bool), 1), float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v.repeat_interleave(g, 2))
    o.backward(do)
    dq, dk, dv, delta = attention_backward(q.detach(), k.detach(), v.detach(), do, causal=causal)
    torch.testing.assert_close(dq, q.grad, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(dk, k.grad, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(dv, v.grad, atol=2e-5, rtol=1e-4)
    assert delta.shape == (2, 4, 128) and (delta[:, :, 70:] == 0).all()
    torch.testing.assert_close(delta[:, :, :70], (do * o.detach()).sum(-1).transpose(1, 2), atol=1e-5, rtol=1e-5)


def test_oracle_empty_rows_and_varlen_layout():
    # causal with more queries than keys: the first Sq - Sk rows see nothing
    q, k, v = make_qkv(6, 1, 2, 2, 12, 8, 16, torch.float32)
    out, lse = attention_forward(q, k, v, causal=True)
    assert torch.isposinf(lse[:, :, :4]).all() and (out[:, :4] == 0).all()
    assert torch.isfinite(lse[:, :, 4:]).all()
    # packed: an empty sequence in the middle
    cu = [0, 5, 5, 12]
    qp, kp, vp = q[0], k[0].repeat(2, 1, 1)[:12], v[0].repeat(2, 1, 1)[:12]
    o2, l2 = varlen_forward(qp, kp, vp, cu, cu, causal=True)
    assert o2.shape == qp.shape and l2.shape == (2, 12)
    ref, ref_l = attention_forward(qp[5:12].unsqueeze(0), kp[5:12].unsqueeze(0), vp[5:12].unsqueeze(0), causal=True)
    torch.testing.assert_close(o2[5:12], ref[0])
    torch.testing.assert_close(l2[:, 5:12], ref_l[0])


def test_backward_formulas_with_softcap_and_alibi_match_autograd():
    """The explicit backward (P * (dP - delta) times the derivative of the softcap) against autograd
    through the oracle's own forward, which the golden vectors pin."""
    from oracle.attention_oracle import attention_backward, attention_forward

    g = torch.Generator().manual_seed(5)
    q, k, v, do = [torch.randn(1, 37, 4, 16, generator=g) for _ in range(4)]
    k, v = k[:, :, :2].contiguous(), v[:, :, :2].contiguous()
    slopes = torch.tensor([0.1, 0.2, 0.3, 0.4])
    for opt in (dict(causal=True, softcap=5.0), dict(softcap=3.0, window_left=8, window_right=4), dict(causal=True)):
        qa, ka, va = [t.clone().requires_grad_() for t in (q, k, v)]
        out, _ = attention_forward(qa, ka, va, alibi_slopes=slopes, **opt)
        out.backward(do)
        dq, dk, dv, _ = attention_backward(q, k, v, do, alibi_slopes=slopes, **opt)
        torch.testing.assert_close(dq, qa.grad, atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(dk, ka.grad, atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(dv, va.grad, atol=1e-5, rtol=1e-4)


def test_window_normalisation_follows_the_reference_host_layer():
    """flash-attn2-rs/src/host/forward/mod.rs:310-320: sides of at least seqlen_k are open, causal sets right = 0,
    ALiBi takes its key-position-only form when left is open and right is 0. Where the clamp changes the mask
    (Sq > Sk, right window >= Sk) the rows before the first key see every key instead of none."""
    from oracle.attention_oracle import attention_forward, normalise_windows

    assert normalise_windows(False, 200, 130, 31) == (-1, -1, False)
    assert normalise_windows(True, 300, -1, 256) == (-1, 0, True)
    assert normalise_windows(False, 0, 5, 1) == (0, -1, False)
    assert normalise_windows(False, -1, 0, 100) == (-1, 0, True)
    assert normalise_windows(True, 64, 7, 100) == (64, 0, False)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 40, 2, 16, generator=g)
    k = torch.randn(1, 8, 2, 16, generator=g)
    v = torch.randn(1, 8, 2, 16, generator=g)
    clamped = attention_forward(q, k, v, window_left=3, window_right=8)    # right >= Sk: open
    open_right = attention_forward(q, k, v, window_left=3, window_right=-1)
    assert torch.equal(clamped[0], open_right[0]) and torch.equal(clamped[1], open_right[1])
    kept = attention_forward(q, k, v, window_left=3, window_right=7)       # right < Sk: rows 0..23 see no key
    assert torch.isposinf(kept[1][:, :, :24]).all() and not torch.isposinf(kept[1][:, :, 25:]).any()
