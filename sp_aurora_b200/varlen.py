"""Packed variable-length sequences and the public zigzag layout for ring attention.

The reference's tests import `sp_aurora_varlen_func` and `zigzag_sp_aurora_varlen_func`
(test/flash_attention/test_intel_ring_flash_attn_varlen.py:23-26,55-77) and its HF adapter calls
a varlen ring (sp_aurora/adapters/hf_adapter.py:141-155), but the package never defined them.
Here they exist with flash-attn's varlen calling convention:

    q, k, v: [total_tokens, H, D], the sequences of the batch packed back to back;
    cu_seqlens_q / cu_seqlens_k: int32 [n_seq + 1] cumulative LOCAL lengths (equal on all ranks).

Every sequence is sharded over the ring like a batch-1 tensor: rank r holds its r-th contiguous
chunk (`*_varlen_func`), or, in the zigzag layout, its half-chunks r and 2W-1-r back to back
(`zigzag_*`; the layout the balanced causal ring uses internally, here chosen by the caller, which
saves the two re-layout exchanges). Each sequence runs as its own ring over views of the packed
tensors (no copies; one set of kernel launches per sequence), so sequences never see each other.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib, local_attn, zigzag
from .local_attn import check_unsupported_kwargs
from .ring import RingFlashAttnFunc

__all__ = ["ring_flash_attn_varlen_func", "zigzag_ring_flash_attn_func",
           "zigzag_ring_flash_attn_varlen_func"]


def _bounds(cu: torch.Tensor, total: int) -> List[int]:
    b = [int(x) for x in cu.tolist()]
    if len(b) < 2 or b[0] != 0 or b[-1] != total or any(y < x for x, y in zip(b, b[1:])):
        raise ValueError(f"cu_seqlens {b} must rise from 0 to the number of packed tokens ({total})")
    return b


def _check_packed(q, k, v):
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dim() != 3:
            raise ValueError(f"{name} must be packed [total_tokens, H, D], got {tuple(t.shape)}")


def ring_flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k=None, max_seqlen_q=None,
                                max_seqlen_k=None, dropout_p=0.0, softmax_scale=None, causal=False,
                                window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                return_attn_probs=False, group=None, max_seqlen=None):
    """Ring attention over packed sequences; returns out [total_tokens, Hq, D] (and lse
    [Hq, total_tokens] fp32 with return_attn_probs). `max_seqlen*` are accepted for signature
    compatibility (tile counts come from cu_seqlens)."""
    check_unsupported_kwargs(dropout_p, window_size, alibi_slopes)
    _check_packed(q, k, v)
    cu_k = cu_seqlens_q if cu_seqlens_k is None else cu_seqlens_k
    bq, bk = _bounds(cu_seqlens_q, q.shape[0]), _bounds(cu_k, k.shape[0])
    if len(bq) != len(bk):
        raise ValueError("cu_seqlens_q and cu_seqlens_k describe different numbers of sequences")
    outs, lses = [], []
    for i in range(len(bq) - 1):
        qi, ki, vi = q[bq[i]:bq[i + 1]], k[bk[i]:bk[i + 1]], v[bk[i]:bk[i + 1]]
        if qi.shape[0] == 0:
            continue
        res = RingFlashAttnFunc.apply(qi.unsqueeze(0), ki.unsqueeze(0), vi.unsqueeze(0), 0.0,
                                      softmax_scale, causal, (-1, -1), None, deterministic, True, group)
        outs.append(res[0].squeeze(0))
        lses.append(res[1].squeeze(0))
    out = torch.cat(outs, dim=0) if outs else q.new_empty(q.shape)
    if not return_attn_probs:
        return out
    return out, torch.cat(lses, dim=1), None


class ZigzagRingFlashAttnFunc(torch.autograd.Function):
    """Causal ring attention on shards that already are in the zigzag layout."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, deterministic, return_softmax, group):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        local_attn.check_qkv(q, k, v)
        live = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        ctx.ring = live
        ctx.softmax_scale, ctx.group, ctx.deterministic = softmax_scale, group, bool(deterministic)
        if not live:      # one rank: the zigzag layout of one rank is the plain order
            out, lse = local_attn.flash_attn_forward(q, k, v, softmax_scale, True)
            ctx.save_for_backward(q, k, v, out, lse)
        else:
            out, lse, saved = zigzag.zigzag_ring_forward(group, q, k, v, softmax_scale,
                                                         need_lse=bool(return_softmax),
                                                         input_layout="zigzag")
            ctx.save_for_backward(*saved)
        return (out, lse, None) if return_softmax else out

    @staticmethod
    def backward(ctx, dout, *args):
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        if not ctx.ring:
            q, k, v, out, lse = ctx.saved_tensors
            dq, dk, dv = local_attn.flash_attn_backward(dout, q, k, v, out, lse, ctx.softmax_scale, True,
                                                        deterministic=ctx.deterministic)
        else:
            q_z, kv_z, out_z, lse_z = ctx.saved_tensors
            dq, dk, dv = zigzag.zigzag_ring_backward(ctx.group, dout, q_z, kv_z, out_z, lse_z,
                                                     ctx.softmax_scale, deterministic=ctx.deterministic,
                                                     input_layout="zigzag")
        _lib.maybe_check_status()
        return dq, dk, dv, None, None, None, None


def zigzag_ring_flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=True,
                                window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                return_attn_probs=False, group=None):
    """q, k, v: [B, S_local, H, D] in the zigzag layout: rank r of W holds half-chunks r and
    2W-1-r of the sequence, back to back. Causal only (the layout exists to balance the
    causal mask)."""
    check_unsupported_kwargs(dropout_p, window_size, alibi_slopes)
    if not causal:
        raise ValueError("the zigzag layout is defined for causal attention")
    return ZigzagRingFlashAttnFunc.apply(q, k, v, softmax_scale, deterministic, return_attn_probs, group)


def zigzag_ring_flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k=None, max_seqlen_q=None,
                                       max_seqlen_k=None, dropout_p=0.0, softmax_scale=None,
                                       causal=True, window_size=(-1, -1), alibi_slopes=None,
                                       deterministic=False, return_attn_probs=False, group=None,
                                       max_seqlen=None):
    """Packed sequences, each in the zigzag layout (see zigzag_ring_flash_attn_func)."""
    check_unsupported_kwargs(dropout_p, window_size, alibi_slopes)
    if not causal:
        raise ValueError("the zigzag layout is defined for causal attention")
    _check_packed(q, k, v)
    cu_k = cu_seqlens_q if cu_seqlens_k is None else cu_seqlens_k
    bq, bk = _bounds(cu_seqlens_q, q.shape[0]), _bounds(cu_k, k.shape[0])
    if bq != bk:
        raise ValueError("the zigzag layout needs equal query and key lengths per sequence")
    outs, lses = [], []
    for i in range(len(bq) - 1):
        if bq[i + 1] == bq[i]:
            continue
        sl = slice(bq[i], bq[i + 1])
        res = ZigzagRingFlashAttnFunc.apply(q[sl].unsqueeze(0), k[sl].unsqueeze(0), v[sl].unsqueeze(0),
                                            softmax_scale, deterministic, True, group)
        outs.append(res[0].squeeze(0))
        lses.append(res[1].squeeze(0))
    out = torch.cat(outs, dim=0) if outs else q.new_empty(q.shape)
    if not return_attn_probs:
        return out
    return out, torch.cat(lses, dim=1), None
