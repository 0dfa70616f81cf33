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
# recorded on the launching stream, under "fwd", "bwd_dq" (the dQ pass: 1.0x the
# forward's FLOPs of the 2.5x a backward counts), "bwd_dkv" (the dK/dV pass: 1.5x) or
# "bwd" (both passes in one call). Used by the benchmark; None (default) records nothing.
KERNEL_TIMERS = None


# Optional per-stage timing of the multi-GPU schedules: when set to a dict, the ring code
# brackets its stages (re-layout exchanges, per-step kernel groups, waits for transfers)
# with CUDA events on the compute stream and appends (start, end) under the stage's name.
# A "wait" stage is the time the compute stream stalls for a transfer, i.e. exposed
# communication. None (default) records nothing.
STAGE_TIMERS = None


class stage:
    def __init__(self, name, device):
        self.name, self.device = name, device

    def __enter__(self):
        if STAGE_TIMERS is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.device))
        return self

    def __exit__(self, *exc):
        if STAGE_TIMERS is not None:
            self.end.record(torch.cuda.current_stream(self.device))
            STAGE_TIMERS.setdefault(self.name, []).append((self.start, self.end))
        return False


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


def _check_rowstat(name: str, t: torch.Tensor, B: int, Hq: int, Sq: int):
    """lse / delta: fp32 [B,Hq,Sq] with contiguous rows (batch and head strides are free)."""
    if t.dtype != torch.float32 or tuple(t.shape) != (B, Hq, Sq) or (Sq > 1 and t.stride(2) != 1):
        raise ValueError(f"{name} must be fp32 [B,Hq,Sq] with contiguous rows")


def _fill_qkv(a, q, k, v):
    a.q, a.q_sb, a.q_ss, a.q_sh = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    a.k, a.k_sb, a.k_ss, a.k_sh = k.data_ptr(), k.stride(0), k.stride(1), k.stride(2)
    a.v, a.v_sb, a.v_ss, a.v_sh = v.data_ptr(), v.stride(0), v.stride(1), v.stride(2)


def attn_fwd_step(q, k, v, softmax_scale: float, causal: bool, lse: torch.Tensor,
                  out: Optional[torch.Tensor] = None, out_acc: Optional[torch.Tensor] = None,
                  merge_prev: bool = False, causal_off: int = 0) -> None:
    """One spa_attn_fwd call. `lse` fp32 [B,Hq,Sq] (rows contiguous) is written (and
    read when merge_prev); `out` (q.dtype, strided) and/or `out_acc` (fp32 contiguous)
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
    _check_rowstat("lse", lse, B, Hq, Sq)
    a.lse, a.lse_sb, a.lse_sh = lse.data_ptr(), lse.stride(0), lse.stride(1)
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
                  dq_acc: Optional[torch.Tensor], dk: Optional[torch.Tensor],
                  dv: Optional[torch.Tensor], dkv_accumulate: bool = False, causal_off: int = 0,
                  dq: Optional[torch.Tensor] = None, dq_overwrite: bool = False,
                  deterministic: bool = False, passes: int = _lib.SPA_BWD_BOTH) -> None:
    """One spa_attn_bwd call (see include/spa.h). The block's dQ plus the running sum in
    dq_acc (fp32 [B,Sq,Hq,D] contiguous; ignored on input when dq_overwrite) is written to
    dq (q.dtype, strided) and / or back to dq_acc. dk/dv [B,Sk,Hkv,D] are fp32 contiguous
    or q.dtype (strided), overwritten or added to. `passes` runs only the dQ kernel or only
    the dK/dV kernel of the pair."""
    B, Sq, Sk, Hq, Hkv, D = check_qkv(q, k, v)
    _check_tensor("dout", dout, q.dtype, q.device)
    a = BwdArgs()
    _fill_qkv(a, q, k, v)
    a.dout, a.do_sb, a.do_ss, a.do_sh = dout.data_ptr(), dout.stride(0), dout.stride(1), dout.stride(2)
    _check_rowstat("lse", lse, B, Hq, Sq)
    _check_rowstat("delta", delta, B, Hq, Sq)
    if lse.stride()[:2] != delta.stride()[:2]:
        raise ValueError("lse and delta must share their batch and head strides")
    a.lse, a.delta, a.lse_sb, a.lse_sh = lse.data_ptr(), delta.data_ptr(), lse.stride(0), lse.stride(1)
    if passes != _lib.SPA_BWD_DKV_ONLY:
        if dq_acc is not None:
            if dq_acc.dtype != torch.float32 or not dq_acc.is_contiguous() or \
                    tuple(dq_acc.shape) != (B, Sq, Hq, D):
                raise ValueError("dq_acc must be contiguous fp32 [B,Sq,Hq,D]")
            a.dq_acc = dq_acc.data_ptr()
        if dq is not None:
            _check_tensor("dq", dq, q.dtype, q.device)
            if tuple(dq.shape) != (B, Sq, Hq, D):
                raise ValueError("dq must be [B,Sq,Hq,D]")
            a.dq, a.dq_sb, a.dq_ss, a.dq_sh = dq.data_ptr(), dq.stride(0), dq.stride(1), dq.stride(2)
        if dq is None and dq_acc is None:
            raise ValueError("one of dq / dq_acc is required")
        if dq_acc is None and not dq_overwrite:
            raise ValueError("accumulating dq needs dq_acc")
        a.dq_overwrite = int(bool(dq_overwrite))
    if passes != _lib.SPA_BWD_DQ_ONLY:
        for name, t in (("dk", dk), ("dv", dv)):
            if t is None or tuple(t.shape) != (B, Sk, Hkv, D) or t.stride(-1) != 1:
                raise ValueError(f"{name} must be [B,Sk,Hkv,D] with a contiguous last dimension")
            if t.dtype not in (torch.float32, q.dtype) or t.dtype != dk.dtype or t.stride() != dk.stride():
                raise ValueError("dk/dv must both be fp32 or both q.dtype, with equal strides")
        fp32_grads = dk.dtype == torch.float32 and q.dtype != torch.float32
        if fp32_grads and not dk.is_contiguous():
            raise ValueError("fp32 dk/dv of a 16-bit problem must be contiguous")
        a.dk, a.dv = dk.data_ptr(), dv.data_ptr()
        a.dkv_sb, a.dkv_ss, a.dkv_sh = dk.stride(0), dk.stride(1), dk.stride(2)
        a.dkv_fp32 = int(fp32_grads)   # fp32 problems: fp32 is the element type
        a.dkv_accumulate = int(bool(dkv_accumulate))
    a.deterministic = int(bool(deterministic))
    a.passes = int(passes)
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.D = B, Sq, Sk, Hq, Hkv, D
    a.dtype = _lib.DTYPE_CODE[q.dtype]
    a.causal, a.causal_off = int(bool(causal)), int(causal_off)
    a.scale = float(softmax_scale)
    a.stream = stream_ptr(q.device)
    share = {_lib.SPA_BWD_BOTH: 2.5, _lib.SPA_BWD_DQ_ONLY: 1.0, _lib.SPA_BWD_DKV_ONLY: 1.5}[a.passes]
    name = {_lib.SPA_BWD_BOTH: "bwd", _lib.SPA_BWD_DQ_ONLY: "bwd_dq", _lib.SPA_BWD_DKV_ONLY: "bwd_dkv"}[a.passes]
    with _Timed(name, q.device, share * attn_flops(B, Sq, Sk, Hq, D, causal, causal_off)):
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
                        causal: bool = False, dq: Optional[torch.Tensor] = None,
                        dk: Optional[torch.Tensor] = None, dv: Optional[torch.Tensor] = None,
                        deterministic: bool = False):
    """Local attention backward: returns (dq, dk, dv) in q.dtype, written into the given
    tensors when provided (any strides with a contiguous last dimension).
    Counterpart of sp_aurora/intel_flash_attn.py:129 intel_flash_attn_backward."""
    B, Sq, Sk, Hq, Hkv, D = check_qkv(q, k, v)
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    delta = bwd_delta(out, dout)
    if dq is None:
        dq = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    if dk is None:
        dk = torch.empty((B, Sk, Hkv, D), dtype=q.dtype, device=q.device)
    if dv is None:
        dv = torch.empty((B, Sk, Hkv, D), dtype=q.dtype, device=q.device)
    # each dq row, dk row and dv row has one owning CTA: no accumulator, nothing to zero
    attn_bwd_step(q, k, v, dout, lse, delta, softmax_scale, causal, None, dk, dv,
                  dq=dq, dq_overwrite=True, deterministic=deterministic)
    return dq, dk, dv


class LocalFlashAttnFunc(torch.autograd.Function):
    """Differentiable single-device attention on [B, S, H, D] tensors; returns (out, lse).
    What sp_aurora/ulysses/attn_layer.py:34 select_flash_attn_impl hands to its callers."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** -0.5
        out, lse = flash_attn_forward(q, k, v, softmax_scale, causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.softmax_scale, ctx.causal = softmax_scale, causal
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dq, dk, dv = flash_attn_backward(dout, q, k, v, out, lse, ctx.softmax_scale, ctx.causal)
        return dq, dk, dv, None, None


def update_out_and_lse(out: Optional[torch.Tensor], lse: Optional[torch.Tensor],
                       block_out: torch.Tensor, block_lse: torch.Tensor, slice_=None):
    """Merge a block result into the running (out, lse).

    Counterpart of sp_aurora/utils.py:109 update_out_and_lse with this package's
    layouts: out fp32 [B,S,H,D], lse fp32 [B,H,S], block_out [B,S,H,D] (any
    supported dtype), block_lse [B,H,S]. The first call (out is None) returns
    fp32 copies (sp_aurora/utils.py:116-122); later calls update in place.

    `slice_` (sp_aurora/utils.py:123-128, used by zigzag-style callers that merge a block into
    part of the rows): a `slice` over the sequence dimension; the block is merged into
    out[:, slice_] and lse[:, :, slice_]. The reference indexes its [B,H,S,D] accumulator with
    a tuple; with this package's layouts out and lse order their dimensions differently, so
    only the sequence range is taken."""
    if slice_ is not None:
        if out is None:
            raise RuntimeError("first update_out_and_lse should not pass slice_ args")
        if isinstance(slice_, tuple):          # (..., seq_slice): keep the last entry
            slice_ = slice_[-1]
        if not isinstance(slice_, slice):
            raise ValueError("slice_ must be a slice over the sequence dimension")
        sub_out = out[:, slice_].contiguous()
        sub_lse = lse[:, :, slice_].contiguous()
        update_out_and_lse(sub_out, sub_lse, block_out, block_lse)
        out[:, slice_].copy_(sub_out)
        lse[:, :, slice_].copy_(sub_lse)
        return out, lse
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
