"""Rotary position embedding as a strided row copy (spa_rope_rows).

The reference has no position embedding on this path; a model that uses RoPE with Ulysses
attention would rotate q and k (one full read + write each) and then pack them for the
all-to-all (another read + write). `rope_copy` does both in one pass: it writes the rotated rows
straight into any strided destination, e.g. the head slices of the packed all-to-all message
(`all_to_all.heads_all_to_all_packed(..., rope=...)`), and `apply_rope` is the differentiable
in-layout form (its backward is the inverse rotation of the gradient).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib
from ._lib import check, lib

__all__ = ["rope_tables", "rope_copy", "apply_rope", "RopeFunction"]


def rope_tables(max_pos: int, head_dim: int, base: float = 10000.0, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos, sin fp32 [max_pos, head_dim/2] of the rotate-half convention (angle = pos * base^(-2i/D))."""
    inv = base ** (-torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def rope_copy(dst: torch.Tensor, src: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos_dim: int,
              pos_offset: int = 0, inverse: bool = False) -> torch.Tensor:
    """dst = rotate(src): equally shaped CUDA views [..., D] (up to four leading dims, last
    dim contiguous, strides multiples of 16 bytes); the token position of a row is
    pos_offset + its index along dimension `pos_dim`. dst may be src."""
    if dst.shape != src.shape or dst.dtype != src.dtype:
        raise ValueError("rope_copy needs equal shapes and dtypes")
    if not (dst.is_cuda and src.is_cuda and cos.is_cuda and sin.is_cuda):
        raise ValueError("rope_copy runs on CUDA tensors only (no CPU path)")
    if src.dtype not in _lib.DTYPE_CODE:
        raise ValueError(f"unsupported dtype {src.dtype}")
    D = src.shape[-1]
    nd = src.dim() - 1
    if nd < 1 or nd > 4 or src.stride(-1) != 1 or dst.stride(-1) != 1:
        raise ValueError("rope_copy needs 1-4 leading dimensions and a contiguous last dimension")
    if not 0 <= pos_dim < nd:
        raise ValueError("pos_dim must name a leading dimension")
    for t in (cos, sin):
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != D // 2 or not t.is_contiguous():
            raise ValueError("cos / sin must be contiguous fp32 [positions, D/2]")
    if dst.numel() == 0:
        return dst
    pad = 4 - nd
    n = [1] * pad + list(src.shape[:-1])
    ss = [0] * pad + list(src.stride()[:-1])
    ds = [0] * pad + list(dst.stride()[:-1])
    check(lib.spa_rope_rows(src.data_ptr(), dst.data_ptr(), _lib.i64x4(n), _lib.i64x4(ss), _lib.i64x4(ds),
                            D, _lib.DTYPE_CODE[src.dtype], cos.data_ptr(), sin.data_ptr(), cos.shape[0],
                            pos_dim + pad, int(pos_offset), int(bool(inverse)),
                            _lib.stream_ptr(src.device)), "spa_rope_rows")
    return dst


class RopeFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, pos_dim, pos_offset):
        ctx.save_for_backward(cos, sin)
        ctx.pos_dim, ctx.pos_offset = pos_dim, pos_offset
        return rope_copy(torch.empty_like(x), x, cos, sin, pos_dim, pos_offset)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        if g.stride(-1) != 1:
            g = g.contiguous()
        return rope_copy(torch.empty_like(g), g, cos, sin, ctx.pos_dim, ctx.pos_offset, inverse=True), \
            None, None, None, None


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos_offset: int = 0,
               pos_dim: int = 1) -> torch.Tensor:
    """Rotated copy of x [B, S, H, D] (positions along dim 1 by default); differentiable."""
    return RopeFunction.apply(x, cos, sin, pos_dim, pos_offset)
