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


def _alloc(shape, dtype, device):
    """Every output and workspace of this module is allocated here (a test substitutes a canary-padded one)."""
    return torch.empty(tuple(shape), dtype=dtype, device=device)


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
        out = _alloc((b, sq, h, d), q.dtype, q.device)
    elif out.shape != q.shape or out.dtype != q.dtype or out.device != q.device:
        raise ValueError("out must match q's shape, dtype and device")
    lse = _alloc((b, h, sq), torch.float32, q.device)
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
    out = _alloc(q.shape, q.dtype, q.device)
    lse = _alloc((h, total_q), torch.float32, q.device).fill_(float("inf"))
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


def bwd_preprocess(dout, out, *, cu_seqlens_q=None, max_seqlen_q=None):
    """delta = rowsum(dO * O) in fp32: [B, H, ceil(Sq/128)*128], or packed [H, total_q + 128*batch]."""
    _require_cuda(dout, out)
    lib = _cabi.load()
    if dout.shape != out.shape or dout.dtype != out.dtype or dout.device != out.device:
        raise ValueError("dout and out must share shape, dtype and device")
    _check_last_stride("dout", dout)
    _check_last_stride("out", out)
    a = _cabi.BwdPreprocessArgs()
    a.dout, a.out = dout.data_ptr(), out.data_ptr()
    a.dtype = _dtype_code(dout)
    if cu_seqlens_q is None:
        b, sq, h, d = out.shape
        delta = _alloc((b, h, (sq + 127) // 128 * 128), torch.float32, out.device)
        a.batch, a.seqlen_q = b, sq
    else:
        total_q, h, d = out.shape
        b = cu_seqlens_q.numel() - 1
        delta = _alloc((h, total_q + 128 * b), torch.float32, out.device).zero_()
        a.batch, a.seqlen_q = b, int(max_seqlen_q)
        a.cu_seqlens_q, a.total_q = cu_seqlens_q.data_ptr(), total_q
    a.delta = delta.data_ptr()
    a.heads, a.head_dim = h, d
    a.do_stride, a.o_stride = _strides3(dout), _strides3(out)
    with torch.cuda.device(out.device):
        _cabi.check(lib.fa2_bwd_preprocess(C.byref(a), _stream(out)))
    return delta


def bwd(q, k, v, dout, lse, delta, *, softmax_scale=None, causal=False, window_left=-1, window_right=-1,
        which=3, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None, max_seqlen_k=None, dq_accum=None,
        kernel_events=None, alibi_slopes=None, softcap=0.0):
    """dQ, dK, dV (input dtype, contiguous). `which`: bit 0 = dQ, bit 1 = dK and dV.

    `kernel_events`: optional pair of torch.cuda.Event recorded around the main kernel only."""
    _require_cuda(q, k, v, dout, lse, delta)
    lib = _cabi.load()
    if k.dtype != q.dtype or v.dtype != q.dtype or dout.dtype != q.dtype:
        raise TypeError("q, k, v, dout must share dtype (all f16 or all bf16)")
    if dout.shape != q.shape or v.shape != k.shape:
        raise ValueError("dout must match q and v must match k")
    for name, t in (("q", q), ("k", k), ("v", v), ("dout", dout)):
        _check_last_stride(name, t)
    if lse.dtype != torch.float32 or delta.dtype != torch.float32 or not lse.is_contiguous() or not delta.is_contiguous():
        raise ValueError("lse and delta must be contiguous float32")
    a = _cabi.BwdArgs()
    packed = cu_seqlens_q is not None
    if packed:
        total_q, h, d = q.shape
        total_k, hk = k.shape[0], k.shape[1]
        b = cu_seqlens_q.numel() - 1
        a.batch, a.seqlen_q, a.seqlen_k = b, int(max_seqlen_q), int(max_seqlen_k)
        a.cu_seqlens_q, a.cu_seqlens_k = cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr()
        a.total_q, a.total_k = total_q, total_k
        if tuple(lse.shape) != (h, total_q) or tuple(delta.shape) != (h, total_q + 128 * b):
            raise ValueError("packed lse must be [H, total_q] and delta [H, total_q + 128*batch]")
    else:
        b, sq, h, d = q.shape
        sk, hk = k.shape[1], k.shape[2]
        a.batch, a.seqlen_q, a.seqlen_k = b, sq, sk
        if tuple(lse.shape) != (b, h, sq) or tuple(delta.shape) != (b, h, (sq + 127) // 128 * 128):
            raise ValueError("lse must be [B, H, Sq] and delta [B, H, ceil(Sq/128)*128]")
    dq = _alloc(q.shape, q.dtype, q.device)
    dk = _alloc(k.shape, k.dtype, k.device)
    dv = _alloc(v.shape, v.dtype, v.device)
    a.q, a.k, a.v, a.dout = q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr()
    a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dtype = _dtype_code(q)
    a.heads, a.heads_k, a.head_dim = h, hk, d
    a.q_stride, a.k_stride, a.v_stride, a.do_stride = _strides3(q), _strides3(k), _strides3(v), _strides3(dout)
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / (d ** 0.5)
    a.causal = int(bool(causal))
    a.window_left, a.window_right = int(window_left), int(window_right)
    a.which = int(which)
    if kernel_events is not None:
        a.ev_kernel_start, a.ev_kernel_stop = kernel_events[0].cuda_event, kernel_events[1].cuda_event
    if alibi_slopes is not None:
        if alibi_slopes.dtype != torch.float32 or not alibi_slopes.is_contiguous() or not alibi_slopes.is_cuda:
            raise ValueError("alibi_slopes must be a contiguous float32 CUDA tensor")
        if tuple(alibi_slopes.shape) == (h,):
            a.alibi_batch_stride = 0
        elif tuple(alibi_slopes.shape) == (b, h):
            a.alibi_batch_stride = h
        else:
            raise ValueError("alibi_slopes must be [H] or [B, H]")
        a.alibi_slopes = alibi_slopes.data_ptr()
    a.softcap = float(softcap)
    need = lib.fa2_bwd_workspace_bytes(C.byref(a))
    if need > 0:
        if dq_accum is None:
            dq_accum = _alloc((need // 4,), torch.float32, q.device)
        a.dq_accum, a.dq_accum_bytes = dq_accum.data_ptr(), dq_accum.numel() * 4
    with torch.cuda.device(q.device):
        _cabi.check(lib.fa2_bwd(C.byref(a), _stream(q)))
    return dq, dk, dv
