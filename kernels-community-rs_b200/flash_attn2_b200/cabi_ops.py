"""Torch-tensor front end of the C ABI (include/fa2_b200.h).

Device memory, streams and allocation come from torch; everything else is the C library. These
functions mirror the operator semantics of the reference crate's host layer for the same paths
(flash-attn2-rs/src/host/forward/mod.rs, backward.rs, varlen/mod.rs) and are what the GPU parity
tests call.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _cabi


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _cabi.FA2_F16
    if t.dtype == torch.bfloat16:
        return _cabi.FA2_BF16
    raise TypeError("q, k, v must be float16 or bfloat16")


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NotImplementedError("flash_attn2_b200 runs on CUDA tensors only (no CPU fallback)")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _strides3(t: torch.Tensor):
    if t.dim() == 4:
        return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    return (C.c_int64 * 3)(0, t.stride(0), t.stride(1))


def _check_last_stride(name, t):
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must have unit last stride")


def fwd(q, k, v, *, out=None, alibi_slopes=None, softmax_scale=None, causal=False, window_left=-1,
        window_right=-1, softcap=0.0):
    """Dense forward: returns (out [B,Sq,H,D], lse fp32 [B,H,Sq])."""
    _require_cuda(q, k, v, out, alibi_slopes)
    lib = _cabi.load()
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be rank-4 [B, S, H, D]")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share dtype (all f16 or all bf16)")
    b, sq, h, d = q.shape
    if k.shape[0] != b or k.shape[3] != d:
        raise ValueError("k must be [B, Sk, Hk, D] with q's batch and head dim")
    if v.shape != k.shape:
        raise ValueError("v must have k's shape [B, Sk, Hk, D]")
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check_last_stride(name, t)
    sk, hk = k.shape[1], k.shape[2]
    if out is None:
        out = torch.empty((b, sq, h, d), dtype=q.dtype, device=q.device)
    elif out.shape != q.shape or out.dtype != q.dtype or out.device != q.device:
        raise ValueError("out must match q's shape, dtype and device")
    lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
    a = _cabi.FwdArgs()
    a.q, a.k, a.v, a.out, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    if alibi_slopes is not None:
        if alibi_slopes.dtype != torch.float32:
            raise TypeError("alibi_slopes must be float32")
        alibi_slopes = alibi_slopes.contiguous()
        if tuple(alibi_slopes.shape) == (h,):
            a.alibi_batch_stride = 0
        elif tuple(alibi_slopes.shape) == (b, h):
            a.alibi_batch_stride = h
        else:
            raise ValueError(f"alibi_slopes must be [{h}] or [{b}, {h}]")
        a.alibi_slopes = alibi_slopes.data_ptr()
    a.dtype = _dtype_code(q)
    a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim = b, sq, sk, h, hk, d
    a.q_stride, a.k_stride, a.v_stride, a.o_stride = _strides3(q), _strides3(k), _strides3(v), _strides3(out)
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / (d ** 0.5)
    a.causal = int(bool(causal))
    a.window_left, a.window_right = int(window_left), int(window_right)
    a.softcap = float(softcap)
    with torch.cuda.device(q.device):
        _cabi.check(lib.fa2_fwd(C.byref(a), _stream(q)))
    return out, lse


def varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, *, softmax_scale=None,
               causal=False, window_left=-1, window_right=-1, softcap=0.0, alibi_slopes=None):
    """Packed forward: q [total_q,H,D], k/v [total_k,Hk,D]; returns (out, lse fp32 [H,total_q])."""
    _require_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k)
    lib = _cabi.load()
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("packed q, k, v must be rank-3 [total, H, D]")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share dtype (all f16 or all bf16)")
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k)):
        if t.dtype != torch.int32 or t.dim() != 1 or not t.is_contiguous() or t.numel() < 2:
            raise ValueError(f"{name} must be a contiguous int32 vector of batch + 1 entries")
    if cu_seqlens_k.numel() != cu_seqlens_q.numel():
        raise ValueError("cu_seqlens_q and cu_seqlens_k must have the same length")
    total_q, h, d = q.shape
    total_k, hk = k.shape[0], k.shape[1]
    if v.shape != k.shape or k.shape[2] != d:
        raise ValueError("k and v must be [total_k, Hk, D] with q's head dim")
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check_last_stride(name, t)
    batch = cu_seqlens_q.numel() - 1
    out = torch.empty_like(q, memory_format=torch.contiguous_format)
    lse = torch.full((h, total_q), float("inf"), dtype=torch.float32, device=q.device)
    a = _cabi.FwdArgs()
    a.q, a.k, a.v, a.out, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    if alibi_slopes is not None:
        alibi_slopes = alibi_slopes.contiguous()
        a.alibi_slopes = alibi_slopes.data_ptr()
        a.alibi_batch_stride = 0 if alibi_slopes.dim() == 1 else h
    a.dtype = _dtype_code(q)
    a.batch, a.seqlen_q, a.seqlen_k = batch, int(max_seqlen_q), int(max_seqlen_k)
    a.heads, a.heads_k, a.head_dim = h, hk, d
    a.q_stride, a.k_stride, a.v_stride, a.o_stride = _strides3(q), _strides3(k), _strides3(v), _strides3(out)
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / (d ** 0.5)
    a.causal = int(bool(causal))
    a.window_left, a.window_right = int(window_left), int(window_right)
    a.softcap = float(softcap)
    a.cu_seqlens_q, a.cu_seqlens_k = cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr()
    a.total_q, a.total_k = total_q, total_k
    with torch.cuda.device(q.device):
        _cabi.check(lib.fa2_varlen_fwd(C.byref(a), _stream(q)))
    return out, lse


def device_status(device=None) -> int:
    """Synchronises and returns the kernels' status word (0 = ok); see fa2_device_status."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    return _cabi.load().fa2_device_status(idx)
