"""Per-device attention steps over the C-ABI: forward (+ fused out/lse merge),
backward, delta, stand-alone merge and the fp32 -> dtype cast.

Mirrors the reference's local-attention layer
(sp_aurora/intel_flash_attn.py:18 intel_flash_attn_forward, :129
intel_flash_attn_backward, :161-168 _flash_attn_forward/_backward) and its merge
(sp_aurora/utils.py:109 update_out_and_lse), but on `[B, S, H, D]` tensors -- the
layout the public API documents -- and with a real backward.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import BwdArgs, FwdArgs, check, lib, stream_ptr

_SUPPORTED_D = (32, 64, 128)

# Optional per-kernel timing: when set to a dict, every forward/backward kernel
# call appends (start event, end event, algorithmic FLOPs of the call), the events
# recorded on the launching stream, under "fwd" / "bwd". Used by the benchmark;
# None (default) records nothing.
KERNEL_TIMERS = None


class _Timed:
    def __init__(self, name, device, flops=0.0):
        self.name, self.device, self.flops = name, device, flops

    def __enter__(self):
        if KERNEL_TIMERS is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.device))
        return self

    def __exit__(self, *exc):
        if KERNEL_TIMERS is not None:
            self.end.record(torch.cuda.current_stream(self.device))
            KERNEL_TIMERS.setdefault(self.name, []).append((self.start, self.end, self.flops))
        return False


def attn_flops(B, Sq, Sk, Hq, D, causal, causal_off=0) -> float:
    """Algorithmic forward FLOPs of one call: 4*B*Hq*D*(visible query-key pairs)."""
    if not causal:
        pairs = float(Sq) * Sk
    else:   # query i sees clamp(i + off + 1, 0, Sk) keys
        i_a = min(Sq, max(0, -causal_off))                 # first row with at least one key
        i_b = min(Sq, max(i_a, Sk - causal_off - 1))       # first row that sees all Sk keys
        n = i_b - i_a                                      # rows on the ramp
        first = i_a + causal_off + 1
        pairs = n * first + n * (n - 1) / 2.0 + (Sq - i_b) * float(Sk)
    return 4.0 * B * Hq * D * pairs


def check_unsupported_kwargs(dropout_p=0.0, window_size=(-1, -1), alibi_slopes=None, softcap=0.0):
    """The reference accepts and silently ignores these
    (sp_aurora/intel_flash_attn.py:25-28); here they are rejected loudly."""
    if dropout_p and dropout_p > 0.0:
        raise NotImplementedError("dropout_p > 0 is not supported")
    if alibi_slopes is not None:
        raise NotImplementedError("alibi_slopes is not supported")
    if tuple(window_size) != (-1, -1):
        raise NotImplementedError("sliding-window attention is not supported")
    if softcap:
        raise NotImplementedError("softcap is not supported")


def _check_tensor(name: str, t: torch.Tensor, dtype=None, device=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this package has no CPU path)")
    if t.dim() != 4:
        raise ValueError(f"{name} must be [B, S, H, D], got shape {tuple(t.shape)}")
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must be contiguous in its last dimension")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if device is not None and t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")


def check_qkv(q, k, v):
    _check_tensor("q", q)
    if q.dtype not in _lib.DTYPE_CODE:
        raise ValueError(f"dtype {q.dtype} not supported (use bf16, fp16 or fp32)")
    _check_tensor("k", k, q.dtype, q.device)
    _check_tensor("v", v, q.dtype, q.device)
    B, Sq, Hq, D = q.shape
    if k.shape != v.shape:
        raise ValueError(f"k {tuple(k.shape)} and v {tuple(v.shape)} differ")
    if k.shape[0] != B or k.shape[3] != D:
        raise ValueError(f"q {tuple(q.shape)} and k {tuple(k.shape)} disagree on batch/head_dim")
    if D not in _SUPPORTED_D:
        raise ValueError(f"head_dim must be one of {_SUPPORTED_D}, got {D}")
    Hkv = k.shape[2]
    if Hq % Hkv != 0:
        raise ValueError(f"query heads ({Hq}) must be a multiple of kv heads ({Hkv})")
    return B, Sq, k.shape[1], Hq, Hkv, D


def _fill_qkv(a, q, k, v):
    a.q, a.q_sb, a.q_ss, a.q_sh = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    a.k, a.k_sb, a.k_ss, a.k_sh = k.data_ptr(), k.stride(0), k.stride(1), k.stride(2)
    a.v, a.v_sb, a.v_ss, a.v_sh = v.data_ptr(), v.stride(0), v.stride(1), v.stride(2)


def attn_fwd_step(q, k, v, softmax_scale: float, causal: bool, lse: torch.Tensor,
                  out: Optional[torch.Tensor] = None, out_acc: Optional[torch.Tensor] = None,
                  merge_prev: bool = False, causal_off: int = 0) -> None:
    """One spa_attn_fwd call. `lse` fp32 [B,Hq,Sq] is written (and read when
    merge_prev); `out` (q.dtype, strided) and/or `out_acc` (fp32 contiguous)
    receive the (merged) rows."""
    B, Sq, Sk, Hq, Hkv, D = check_qkv(q, k, v)
    a = FwdArgs()
    _fill_qkv(a, q, k, v)
    if out is not None:
        _check_tensor("out", out, q.dtype, q.device)
        a.out, a.o_sb, a.o_ss, a.o_sh = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    if out_acc is not None:
        if out_acc.dtype != torch.float32 or not out_acc.is_contiguous() or \
                tuple(out_acc.shape) != (B, Sq, Hq, D):
            raise ValueError("out_acc must be contiguous fp32 [B,Sq,Hq,D]")
        a.out_acc = out_acc.data_ptr()
    if lse.dtype != torch.float32 or not lse.is_contiguous() or tuple(lse.shape) != (B, Hq, Sq):
        raise ValueError("lse must be contiguous fp32 [B,Hq,Sq]")
    a.lse = lse.data_ptr()
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.D = B, Sq, Sk, Hq, Hkv, D
    a.dtype = _lib.DTYPE_CODE[q.dtype]
    a.causal, a.causal_off, a.merge_prev = int(bool(causal)), int(causal_off), int(bool(merge_prev))
    a.scale = float(softmax_scale)
    a.stream = stream_ptr(q.device)
    with _Timed("fwd", q.device, attn_flops(B, Sq, Sk, Hq, D, causal, causal_off)):
        check(lib.spa_attn_fwd(C.byref(a)), "spa_attn_fwd")


def flash_attn_forward(q, k, v, softmax_scale: Optional[float] = None, causal: bool = False,
                       dropout_p: float = 0.0, window_size=(-1, -1), alibi_slopes=None,
                       softcap: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Local attention: returns (out [B,Sq,Hq,D] in q.dtype, lse [B,Hq,Sq] fp32).
    Counterpart of sp_aurora/intel_flash_attn.py:18 intel_flash_attn_forward."""
    check_unsupported_kwargs(dropout_p, window_size, alibi_slopes, softcap)
    B, Sq, Sk, Hq, Hkv, D = check_qkv(q, k, v)
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    attn_fwd_step(q, k, v, softmax_scale, causal, lse, out=out)
    return out, lse


def bwd_delta(out: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    """delta[b,h,s] = sum_d out*dout, fp32 [B,H,S]."""
    _check_tensor("out", out)
    _check_tensor("dout", dout, out.dtype, out.device)
    B, S, H, D = out.shape
    delta = torch.empty((B, H, S), dtype=torch.float32, device=out.device)
    check(lib.spa_bwd_delta(out.data_ptr(), out.stride(0), out.stride(1), out.stride(2),
                            dout.data_ptr(), dout.stride(0), dout.stride(1), dout.stride(2),
                            delta.data_ptr(), B, S, H, D, _lib.DTYPE_CODE[out.dtype],
                            stream_ptr(out.device)), "spa_bwd_delta")
    return delta


def attn_bwd_step(q, k, v, dout, lse, delta, softmax_scale: float, causal: bool,
                  dq_acc: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor,
                  dkv_accumulate: bool = False, causal_off: int = 0) -> None:
    """One spa_attn_bwd call. dq_acc fp32 [B,Sq,Hq,D] is accumulated into;
    dk/dv [B,Sk,Hkv,D] contiguous (fp32 or q.dtype) are overwritten or added to."""
    B, Sq, Sk, Hq, Hkv, D = check_qkv(q, k, v)
    _check_tensor("dout", dout, q.dtype, q.device)
    a = BwdArgs()
    _fill_qkv(a, q, k, v)
    a.dout, a.do_sb, a.do_ss, a.do_sh = dout.data_ptr(), dout.stride(0), dout.stride(1), dout.stride(2)
    for name, t in (("lse", lse), ("delta", delta)):
        if t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != (B, Hq, Sq):
            raise ValueError(f"{name} must be contiguous fp32 [B,Hq,Sq]")
    if dq_acc.dtype != torch.float32 or not dq_acc.is_contiguous() or \
            tuple(dq_acc.shape) != (B, Sq, Hq, D):
        raise ValueError("dq_acc must be contiguous fp32 [B,Sq,Hq,D]")
    for name, t in (("dk", dk), ("dv", dv)):
        if not t.is_contiguous() or tuple(t.shape) != (B, Sk, Hkv, D):
            raise ValueError(f"{name} must be contiguous [B,Sk,Hkv,D]")
        if t.dtype not in (torch.float32, q.dtype) or t.dtype != dk.dtype:
            raise ValueError("dk/dv must both be fp32 or both q.dtype")
    a.lse, a.delta, a.dq_acc = lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr()
    a.dk, a.dv = dk.data_ptr(), dv.data_ptr()
    a.dkv_fp32 = int(dk.dtype == torch.float32)
    a.dkv_accumulate = int(bool(dkv_accumulate))
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.D = B, Sq, Sk, Hq, Hkv, D
    a.dtype = _lib.DTYPE_CODE[q.dtype]
    a.causal, a.causal_off = int(bool(causal)), int(causal_off)
    a.scale = float(softmax_scale)
    a.stream = stream_ptr(q.device)
    with _Timed("bwd", q.device, 2.5 * attn_flops(B, Sq, Sk, Hq, D, causal, causal_off)):
        check(lib.spa_attn_bwd(C.byref(a)), "spa_attn_bwd")


def cast_from_f32(src: torch.Tensor, dtype: torch.dtype, alpha: float = 1.0,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(dtype)(alpha * src) for a contiguous fp32 [B,S,H,D] accumulator."""
    if src.dtype != torch.float32 or not src.is_contiguous() or src.dim() != 4:
        raise ValueError("src must be contiguous fp32 [B,S,H,D]")
    B, S, H, D = src.shape
    if out is None:
        out = torch.empty((B, S, H, D), dtype=dtype, device=src.device)
    _check_tensor("out", out, dtype, src.device)
    check(lib.spa_cast_from_f32(src.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1),
                                out.stride(2), B, S, H, D, _lib.DTYPE_CODE[dtype], float(alpha),
                                stream_ptr(src.device)), "spa_cast_from_f32")
    return out


def flash_attn_backward(dout, q, k, v, out, lse, softmax_scale: Optional[float] = None,
                        causal: bool = False):
    """Local attention backward: returns (dq, dk, dv) in q.dtype.
    Counterpart of sp_aurora/intel_flash_attn.py:129 intel_flash_attn_backward."""
    B, Sq, Sk, Hq, Hkv, D = check_qkv(q, k, v)
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    delta = bwd_delta(out, dout)
    dq_acc = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=q.device)
    dk = torch.empty((B, Sk, Hkv, D), dtype=q.dtype, device=q.device)
    dv = torch.empty_like(dk)
    attn_bwd_step(q, k, v, dout, lse, delta, softmax_scale, causal, dq_acc, dk, dv)
    dq = dq_acc if q.dtype == torch.float32 else cast_from_f32(dq_acc, q.dtype)
    return dq, dk, dv


def update_out_and_lse(out: Optional[torch.Tensor], lse: Optional[torch.Tensor],
                       block_out: torch.Tensor, block_lse: torch.Tensor, slice_=None):
    """Merge a block result into the running (out, lse).

    Counterpart of sp_aurora/utils.py:109 update_out_and_lse with this package's
    layouts: out fp32 [B,S,H,D], lse fp32 [B,H,S], block_out [B,S,H,D] (any
    supported dtype), block_lse [B,H,S]. The first call (out is None) returns
    fp32 copies (sp_aurora/utils.py:116-122); later calls update in place."""
    if slice_ is not None:
        raise NotImplementedError("slice_ is only used by the varlen/zigzag variants")
    _check_tensor("block_out", block_out)
    B, S, H, D = block_out.shape
    if tuple(block_lse.shape) != (B, H, S):
        raise RuntimeError(
            f"Shape mismatch: block_lse.shape={tuple(block_lse.shape)}, expected {(B, H, S)}")
    if out is None:
        return block_out.to(torch.float32).contiguous(), block_lse.to(torch.float32).clone()
    if tuple(out.shape) != (B, S, H, D) or tuple(lse.shape) != (B, H, S):
        raise RuntimeError(
            f"Shape mismatch: out.shape={tuple(out.shape)}, block_out.shape={tuple(block_out.shape)}")
    if out.dtype != torch.float32 or not out.is_contiguous() or not lse.is_contiguous():
        raise ValueError("out must be contiguous fp32 and lse contiguous")
    block_lse = block_lse.to(torch.float32).contiguous()
    check(lib.spa_merge(out.data_ptr(), lse.data_ptr(), block_out.data_ptr(), block_out.stride(0),
                        block_out.stride(1), block_out.stride(2), block_lse.data_ptr(), B, S, H, D,
                        _lib.DTYPE_CODE[block_out.dtype], stream_ptr(out.device)), "spa_merge")
    return out, lse
