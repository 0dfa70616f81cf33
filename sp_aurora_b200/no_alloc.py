"""Backward pass for callers that must not allocate device memory.

`flash_attn_backward_noalloc` wraps the C entry point spa_attn_bwd_noalloc: the
caller hands in every tensor, outputs included, and the library keeps its
scratch (the delta row sums, rowsum(dO * O)) in a fixed 16 MiB array that is
part of the library image on each GPU. It exists for code that runs where all
GPU memory is already spoken for (a pool that owns the device, a fixed-budget
service) or that may not enter the CUDA allocator. Limits: the problem must
satisfy B*Sq*Hq*4 bytes <= scratch_bytes(); calls share the one array, so two
calls must not overlap on the same GPU; the first call on a device performs a
one-time address lookup and should happen before any stream capture. It has no
counterpart in the reference.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import BwdNoallocArgs, check, lib, stream_ptr
from .local_attn import _check_tensor, check_qkv


def scratch_bytes() -> int:
    return int(lib.spa_noalloc_scratch_bytes())


def flash_attn_backward_noalloc(dout, q, k, v, out, lse, dq, dk, dv, softmax_scale=None,
                                causal=False, causal_off=0):
    """Writes dq [B,Sq,Hq,D], dk, dv [B,Sk,Hkv,D] (caller-allocated, contiguous,
    q.dtype). Nothing is allocated, here or in the library."""
    B, Sq, Sk, Hq, Hkv, D = check_qkv(q, k, v)
    _check_tensor("out", out, q.dtype, q.device)
    _check_tensor("dout", dout, q.dtype, q.device)
    for name, t, shape in (("dq", dq, (B, Sq, Hq, D)), ("dk", dk, (B, Sk, Hkv, D)),
                           ("dv", dv, (B, Sk, Hkv, D))):
        if tuple(t.shape) != shape or t.dtype != q.dtype or not t.is_contiguous() or t.device != q.device:
            raise ValueError(f"{name} must be contiguous {shape} {q.dtype} on {q.device}")
    if lse.dtype != torch.float32 or not lse.is_contiguous() or tuple(lse.shape) != (B, Hq, Sq):
        raise ValueError("lse must be contiguous fp32 [B,Hq,Sq]")
    a = BwdNoallocArgs()
    a.q, a.q_sb, a.q_ss, a.q_sh = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    a.k, a.k_sb, a.k_ss, a.k_sh = k.data_ptr(), k.stride(0), k.stride(1), k.stride(2)
    a.v, a.v_sb, a.v_ss, a.v_sh = v.data_ptr(), v.stride(0), v.stride(1), v.stride(2)
    a.out, a.o_sb, a.o_ss, a.o_sh = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    a.dout, a.do_sb, a.do_ss, a.do_sh = dout.data_ptr(), dout.stride(0), dout.stride(1), dout.stride(2)
    a.lse, a.dq, a.dk, a.dv = lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.D = B, Sq, Sk, Hq, Hkv, D
    a.dtype = _lib.DTYPE_CODE[q.dtype]
    a.causal, a.causal_off = int(bool(causal)), int(causal_off)
    a.scale = float(D ** -0.5 if softmax_scale is None else softmax_scale)
    a.stream = stream_ptr(q.device)
    check(lib.spa_attn_bwd_noalloc(C.byref(a)), "spa_attn_bwd_noalloc")
    return dq, dk, dv
