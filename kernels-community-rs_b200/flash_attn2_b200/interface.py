"""Python surface of the operators, mirroring the reference package for the paths this library
builds (flash-attn2-rs/tvm-ffi-ext/flash_attn2_rs/flash_attn_interface.py): the same function
names, argument meaning, return lists and error behaviour for `fwd_explicit`, `fwd`, `bwd`,
`varlen_fwd`, `varlen_bwd`, `flash_attn_func` and `flash_attn_varlen_func`. Every call goes through
the tvm-ffi operators in `_ops`; there is no CPU implementation (CPU tensors raise
NotImplementedError like the reference's CPU dispatch does).
"""
from __future__ import annotations

import operator

import torch

from ._ops import ops


def _torch_tensors(values):
    # tvm-ffi converts a returned tensor to torch, but not tensors inside a returned Array.
    return [torch.from_dlpack(v) for v in values]


def _float_arg(value, name):
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise RuntimeError(f"{name} must be a float")
    return float(value)


def _bool_arg(value, name):
    if not isinstance(value, (bool, int)) or isinstance(value, float):
        raise RuntimeError(f"{name} must be a bool")
    return bool(value)


def _int_arg(value, name):
    if isinstance(value, bool):
        return int(value)
    try:
        return operator.index(value)
    except TypeError:
        raise RuntimeError(f"{name} must be an int") from None


def _require_cuda(op, *tensors):
    for t in tensors:
        if isinstance(t, torch.Tensor) and not t.is_cuda:
            raise NotImplementedError(f"{op}: no CPU implementation; tensors must be on a CUDA device")


def _no_dropout(p):
    if p != 0:
        raise RuntimeError("dropout is not built in the sm_100a library (p_dropout must be 0)")


def fwd_explicit(*args):
    """Positional tvm-ffi forward: (q, k, v, alibi_slopes, softmax_scale, is_causal, window_left,
    window_right, softcap[, out]) -> [out, lse]."""
    return _torch_tensors(ops.fwd(*args))


def fwd(q, k, v, out=None, alibi_slopes=None, p_dropout=0.0, softmax_scale=None, is_causal=False,
        window_size_left=-1, window_size_right=-1, softcap=0.0, return_softmax=False, gen=None):
    """Returns [output, LSE, probabilities (empty), RNG state (unused)]."""
    _require_cuda("fwd", q, k, v, out, alibi_slopes)
    p = _float_arg(p_dropout, "p_dropout")
    scale = None if softmax_scale is None else _float_arg(softmax_scale, "softmax_scale")
    causal = _bool_arg(is_causal, "is_causal")
    left, right = _int_arg(window_size_left, "window_size_left"), _int_arg(window_size_right, "window_size_right")
    cap = _float_arg(softcap, "softcap")
    if _bool_arg(return_softmax, "return_softmax"):
        raise RuntimeError("return_softmax requires dropout, which is not built in the sm_100a library")
    _no_dropout(p)
    if not -(2 ** 31) <= left < 2 ** 31 or not -(2 ** 31) <= right < 2 ** 31:
        raise RuntimeError("window sizes must fit int32")
    if q.shape[1] == 1 and alibi_slopes is None:
        causal = False  # single-query convention of the reference
    if alibi_slopes is not None:
        alibi_slopes = alibi_slopes.contiguous()
    if out is None:
        out = torch.empty_like(q, memory_format=torch.contiguous_format)
    lse = ops.fwd_lse(q, k, v, alibi_slopes, scale, causal, left, right, cap, out)
    probabilities = torch.empty(0, device=q.device, dtype=q.dtype)
    state = torch.empty(2, device=q.device, dtype=torch.int64)
    return [out, lse, probabilities, state]


def _finish(grads, buffers):
    out = []
    for g, buf in zip(grads, buffers):
        if buf is not None:
            buf.copy_(g.view(buf.shape))
            g = buf
        out.append(g)
    return out


def bwd(dout, q, k, v, out, softmax_lse, dq=None, dk=None, dv=None, alibi_slopes=None, p_dropout=0.0,
        softmax_scale=None, is_causal=False, window_size_left=-1, window_size_right=-1, softcap=0.0,
        deterministic=False, gen=None, rng_state=None):
    """Returns [dQ, dK, dV, softmax_d] (softmax_d = rowsum(dO * O), padded to 128 rows)."""
    _require_cuda("bwd", dout, q, k, v, out, softmax_lse, dq, dk, dv)
    p = _float_arg(p_dropout, "p_dropout")
    scale = None if softmax_scale is None else _float_arg(softmax_scale, "softmax_scale")
    causal = _bool_arg(is_causal, "is_causal")
    left, right = _int_arg(window_size_left, "window_size_left"), _int_arg(window_size_right, "window_size_right")
    cap = _float_arg(softcap, "softcap")
    deterministic = _bool_arg(deterministic, "deterministic")
    _no_dropout(p)
    for name, t in (("dout", dout), ("out", out)):
        if not isinstance(t, torch.Tensor) or t.shape != q.shape or t.device != q.device or t.dtype != q.dtype:
            raise RuntimeError(f"{name} must match q's shape, dtype and device")
    if (softmax_lse.shape != (q.shape[0], q.shape[2], q.shape[1]) or softmax_lse.dtype != torch.float32
            or not softmax_lse.is_contiguous()):
        raise RuntimeError("softmax_lse must be contiguous float32 [B, H, Sq] on q's device")
    if q.shape[1] == 1 and alibi_slopes is None:
        causal = False
    delta = ops.bwd_preprocess(dout, out, p)
    args = (q, k, v, dout, softmax_lse, delta, alibi_slopes, scale, causal, left, right, cap, p, None)
    if deterministic:
        grad_q = ops.bwd_dq(*args)
        grad_k, grad_v = _torch_tensors(ops.bwd_dkv(*args))
    else:
        grad_q, grad_k, grad_v = _torch_tensors(ops.bwd_all(*args))
    return [*_finish((grad_q, grad_k, grad_v), (dq, dk, dv)), delta]


def varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, out=None, seqused_k=None, leftpad_k=None, block_table=None,
               alibi_slopes=None, max_seqlen_q=0, max_seqlen_k=0, p_dropout=0.0, softmax_scale=None,
               zero_tensors=False, is_causal=False, window_size_left=-1, window_size_right=-1, softcap=0.0,
               return_softmax=False, gen=None):
    """Packed-sequence forward, returning [out, LSE [H, total_q], probabilities (empty), RNG state]."""
    _require_cuda("varlen_fwd", q, k, v, cu_seqlens_q, cu_seqlens_k, out)
    max_q, max_k = _int_arg(max_seqlen_q, "max_seqlen_q"), _int_arg(max_seqlen_k, "max_seqlen_k")
    p = _float_arg(p_dropout, "p_dropout")
    scale = None if softmax_scale is None else _float_arg(softmax_scale, "softmax_scale")
    causal = _bool_arg(is_causal, "is_causal")
    left, right = _int_arg(window_size_left, "window_size_left"), _int_arg(window_size_right, "window_size_right")
    cap = _float_arg(softcap, "softcap")
    _no_dropout(p)
    if block_table is not None:
        raise RuntimeError("paged K/V (block_table) is not built in the sm_100a library")
    values = ops.varlen_fwd_explicit(q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, alibi_slopes, scale,
                                     causal, left, right, cap, p, None, max_q, max_k,
                                     _bool_arg(return_softmax, "return_softmax"), _bool_arg(zero_tensors, "zero_tensors"))
    output, lse, probabilities = _torch_tensors(values)
    if output.ndim == 4:
        output = output.squeeze(0)
    if out is not None:
        out.copy_(output)
        output = out
    state = torch.empty(2, device=q.device, dtype=torch.int64)
    return [output, lse, probabilities, state]


def varlen_bwd(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, dq=None, dk=None, dv=None,
               alibi_slopes=None, max_seqlen_q=0, max_seqlen_k=0, p_dropout=0.0, softmax_scale=None,
               zero_tensors=False, is_causal=False, window_size_left=-1, window_size_right=-1, softcap=0.0,
               deterministic=False, gen=None, rng_state=None):
    """Packed backward returning [dQ, dK, dV, softmax_d [H, total_q + 128*batch]]."""
    _require_cuda("varlen_bwd", dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k)
    max_q, max_k = _int_arg(max_seqlen_q, "max_seqlen_q"), _int_arg(max_seqlen_k, "max_seqlen_k")
    p = _float_arg(p_dropout, "p_dropout")
    scale = None if softmax_scale is None else _float_arg(softmax_scale, "softmax_scale")
    causal = _bool_arg(is_causal, "is_causal")
    left, right = _int_arg(window_size_left, "window_size_left"), _int_arg(window_size_right, "window_size_right")
    cap = _float_arg(softcap, "softcap")
    _no_dropout(p)
    if max_q == 1 and alibi_slopes is None:
        causal = False
    values = ops.varlen_bwd_explicit(q, k, v, dout, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, alibi_slopes, scale,
                                     causal, left, right, cap, p, None, max_q, max_k,
                                     _bool_arg(zero_tensors, "zero_tensors"))
    grad_q, grad_k, grad_v, delta = _torch_tensors(values)
    return [*_finish((grad_q, grad_k, grad_v), (dq, dk, dv)), delta]


class _DenseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic):
        out, lse, _, _ = fwd(q, k, v, alibi_slopes=alibi_slopes, softmax_scale=softmax_scale, is_causal=causal,
                             window_size_left=window_size[0], window_size_right=window_size[1], softcap=softcap)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic = ctx.meta
        dq, dk, dv, _ = bwd(dout.contiguous(), q, k, v, out, lse, alibi_slopes=alibi_slopes,
                            softmax_scale=softmax_scale, is_causal=causal, window_size_left=window_size[0],
                            window_size_right=window_size[1], softcap=softcap, deterministic=deterministic)
        return dq, dk, dv, None, None, None, None, None, None


class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, softmax_scale, causal, window_size, softcap, deterministic):
        out, lse, _, _ = varlen_fwd(q, k, v, cu_q, cu_k, max_seqlen_q=max_q, max_seqlen_k=max_k,
                                    softmax_scale=softmax_scale, is_causal=causal, window_size_left=window_size[0],
                                    window_size_right=window_size[1], softcap=softcap)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.meta = (max_q, max_k, softmax_scale, causal, window_size, softcap, deterministic)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, softmax_scale, causal, window_size, softcap, deterministic = ctx.meta
        dq, dk, dv, _ = varlen_bwd(dout.contiguous(), q, k, v, out, lse, cu_q, cu_k, max_seqlen_q=max_q,
                                   max_seqlen_k=max_k, softmax_scale=softmax_scale, is_causal=causal,
                                   window_size_left=window_size[0], window_size_right=window_size[1],
                                   softcap=softcap, deterministic=deterministic)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """Dense attention with Q/K/V autograd, including MQA/GQA."""
    _no_dropout(dropout_p)
    if return_attn_probs:
        raise RuntimeError("return_attn_probs requires dropout, which is not built in the sm_100a library")
    return _DenseAttention.apply(q, k, v, softmax_scale, causal, tuple(window_size), softcap, alibi_slopes, deterministic)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                           softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
                           deterministic=False, return_attn_probs=False, block_table=None):
    """Variable-length attention with autograd and GPU cumulative lengths."""
    _no_dropout(dropout_p)
    if alibi_slopes is not None or block_table is not None or return_attn_probs:
        raise RuntimeError("alibi_slopes / block_table / return_attn_probs are not built for the packed autograd path")
    return _VarlenAttention.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale,
                                  causal, tuple(window_size), softcap, deterministic)
