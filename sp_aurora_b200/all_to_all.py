"""Sequence <-> head all-to-all reshards (Ulysses) for 4-D and qkv-packed 5-D
tensors: a pack kernel, one NCCL all_to_all_single, an unpack kernel.

Mirrors sp_aurora/comm/all_to_all.py (all_to_all_4D :17, SeqAllToAll4D :183,
seq_all_to_all_4d_inference :208, all_to_all_5D :228, SeqAllToAll5D :338) and
sp_aurora/intel_ulysses_attn.py:60 intel_all_to_all_4d. The result is the exact
permutation the reference produces; only the wire order differs: messages are
laid out (P, B, S_local, heads, D) so that for B == 1 the received buffer IS the
gathered tensor and the unpack pass disappears.

The pack/unpack copies run in the CUDA permutation kernel (spa_permute_rows);
`copy_fn` lets CPU tests of the index arithmetic substitute a host copy.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib

__all__ = ["all_to_all_4D", "all_to_all_5D", "SeqAllToAll4D", "SeqAllToAll5D",
           "seq_all_to_all_4d_inference", "strided_copy", "heads_all_to_all_packed",
           "seq_all_to_all_packed", "HeadsAllToAllPacked"]


def _coalesce(shape, sst, dst):
    """Merge adjacent dims that are contiguous in BOTH views; returns lists."""
    dims = [(n, a, b) for n, a, b in zip(shape, sst, dst) if n != 1]
    if not dims:
        return [1], [1], [1]
    out = [dims[-1]]
    for n, a, b in reversed(dims[:-1]):
        n0, a0, b0 = out[0]
        if a == a0 * n0 and b == b0 * n0:
            out[0] = (n * n0, a0, b0)
        else:
            out.insert(0, (n, a, b))
    return [d[0] for d in out], [d[1] for d in out], [d[2] for d in out]


def strided_copy(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """dst[...] = src[...] for two equally-shaped CUDA views whose innermost
    dimension is contiguous, through spa_permute_rows (16-byte vectors)."""
    if dst.shape != src.shape or dst.dtype != src.dtype:
        raise ValueError("strided_copy needs equal shapes and dtypes")
    if not (dst.is_cuda and src.is_cuda):
        raise ValueError("strided_copy runs on CUDA tensors only (no CPU path)")
    if dst.numel() == 0:
        return dst
    elt = src.element_size()
    shape, sst, dstst = _coalesce(list(src.shape), list(src.stride()), list(dst.stride()))
    if sst[-1] != 1 or dstst[-1] != 1:
        raise ValueError("innermost dimension must be contiguous in both views")
    row_bytes = shape[-1] * elt
    outer = shape[:-1]
    if len(outer) > 4:
        raise ValueError("too many non-mergeable dimensions for the permutation kernel")
    pad = 4 - len(outer)
    n = [1] * pad + outer
    ss = [16] * pad + [s * elt for s in sst[:-1]]
    ds = [16] * pad + [s * elt for s in dstst[:-1]]
    check(lib.spa_permute_rows(src.data_ptr(), dst.data_ptr(), _lib.i64x4(n), _lib.i64x4(ss),
                               _lib.i64x4(ds), row_bytes, _lib.stream_ptr(src.device)),
          "spa_permute_rows")
    return dst


def _world(group) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


def _exchange(send: torch.Tensor, group) -> torch.Tensor:
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def all_to_all_4D(input: torch.Tensor, scatter_idx: int = 2, gather_idx: int = 1, group=None,
                  use_sync: bool = False, copy_fn: Callable = strided_copy) -> torch.Tensor:
    """(2,1): [B, S/P, H, D] -> [B, S, H/P, D];  (1,2): [B, S, H/P, D] -> [B, S/P, H, D].
    Rank r of the group ends up with heads [r*H/P, (r+1)*H/P) of all sequence
    chunks in group-rank order (and the inverse)."""
    if input.dim() != 4:
        raise ValueError(f"input must be 4D tensor, got {input.dim()} and shape {tuple(input.shape)}")
    P = _world(group)
    if P == 1:
        return input
    if scatter_idx == 2 and gather_idx == 1:
        B, Sl, H, D = input.shape
        if H % P != 0:
            raise ValueError(f"number of heads ({H}) must be divisible by the group size ({P})")
        h = H // P
        send = torch.empty((P, B, Sl, h, D), dtype=input.dtype, device=input.device)
        copy_fn(send, input.unflatten(2, (P, h)).permute(2, 0, 1, 3, 4))
        recv = _exchange(send, group)                       # [P_src, B, Sl, h, D]
        if B == 1:
            out = recv.view(1, P * Sl, h, D)
        else:
            out = torch.empty((B, P * Sl, h, D), dtype=input.dtype, device=input.device)
            copy_fn(out.view(B, P, Sl, h, D), recv.permute(1, 0, 2, 3, 4))
    elif scatter_idx == 1 and gather_idx == 2:
        B, S, h, D = input.shape
        if S % P != 0:
            raise ValueError(f"sequence length ({S}) must be divisible by the group size ({P})")
        Sl = S // P
        if B == 1 and input.is_contiguous():
            send = input.view(P, 1, Sl, h, D)
        else:
            send = torch.empty((P, B, Sl, h, D), dtype=input.dtype, device=input.device)
            copy_fn(send, input.unflatten(1, (P, Sl)).permute(1, 0, 2, 3, 4))
        recv = _exchange(send, group)                       # [P_src(head group), B, Sl, h, D]
        out = torch.empty((B, Sl, P * h, D), dtype=input.dtype, device=input.device)
        copy_fn(out.view(B, Sl, P, h, D), recv.permute(1, 2, 0, 3, 4))
    else:
        raise ValueError(f"Unsupported scatter_idx={scatter_idx}, gather_idx={gather_idx}")
    if use_sync and out.is_cuda:
        torch.cuda.current_stream(out.device).synchronize()
    return out


def all_to_all_5D(input: torch.Tensor, scatter_idx: int = 3, gather_idx: int = 1, group=None,
                  use_sync: bool = False, copy_fn: Callable = strided_copy) -> torch.Tensor:
    """qkv-packed: (3,1): [B, S/P, 3, H, D] -> [B, S, 3, H/P, D]; (1,3) is the inverse.
    The middle dimension may be any size T (3 for qkv, 2 for kv)."""
    if input.dim() != 5:
        raise ValueError(f"input must be 5D tensor, got {input.dim()} and shape {tuple(input.shape)}")
    P = _world(group)
    if P == 1:
        return input
    if scatter_idx == 3 and gather_idx == 1:
        B, Sl, T, H, D = input.shape
        if H % P != 0:
            raise ValueError(f"number of heads ({H}) must be divisible by the group size ({P})")
        h = H // P
        send = torch.empty((P, B, Sl, T, h, D), dtype=input.dtype, device=input.device)
        copy_fn(send, input.unflatten(3, (P, h)).permute(3, 0, 1, 2, 4, 5))
        recv = _exchange(send, group)                       # [P_src, B, Sl, T, h, D]
        if B == 1:
            out = recv.view(1, P * Sl, T, h, D)
        else:
            out = torch.empty((B, P * Sl, T, h, D), dtype=input.dtype, device=input.device)
            copy_fn(out.view(B, P, Sl, T, h, D), recv.permute(1, 0, 2, 3, 4, 5))
    elif scatter_idx == 1 and gather_idx == 3:
        B, S, T, h, D = input.shape
        if S % P != 0:
            raise ValueError(f"sequence length ({S}) must be divisible by the group size ({P})")
        Sl = S // P
        if B == 1 and input.is_contiguous():
            send = input.view(P, 1, Sl, T, h, D)
        else:
            send = torch.empty((P, B, Sl, T, h, D), dtype=input.dtype, device=input.device)
            copy_fn(send, input.unflatten(1, (P, Sl)).permute(1, 0, 2, 3, 4, 5))
        recv = _exchange(send, group)                       # [P_src(head group), B, Sl, T, h, D]
        out = torch.empty((B, Sl, T, P * h, D), dtype=input.dtype, device=input.device)
        copy_fn(out.view(B, Sl, T, P, h, D), recv.permute(1, 2, 3, 0, 4, 5))
    else:
        raise RuntimeError("scatter_idx must be 1 or 3 and gather_idx must be 1 or 3")
    if use_sync and out.is_cuda:
        torch.cuda.current_stream(out.device).synchronize()
    return out


def heads_all_to_all_packed(tensors, group=None, copy_fn: Callable = strided_copy, rope=None):
    """Sequence -> head reshard of several [B, S/P, H_i, D] tensors (q, k, v with their
    own head counts) as ONE all-to-all message instead of one per tensor
    (sp_aurora/intel_ulysses_attn.py:156-170 sends q, k and v separately).

    The message is laid out (P, B, S/P, sum_i H_i/P, D): every token row carries its q
    heads, then its k heads, then its v heads. Returns [B, S, H_i/P, D] views of the
    gathered buffer (last dimension contiguous, row stride sum_i H_i/P * D), which the
    attention kernels read in place.

    `rope` = (cos, sin, pos_offset, n_rotated): the first n_rotated tensors (q and k) are
    rotated by the rotary embedding while they are packed (one pass instead of two);
    pos_offset is the global position of this rank's first token."""
    P = _world(group)
    if P == 1:
        if rope is None:
            return list(tensors)
        from .rope import rope_copy
        cos, sin, pos_off, n_rot = rope
        return [rope_copy(torch.empty_like(t), t, cos, sin, 1, pos_off) if i < n_rot else t
                for i, t in enumerate(tensors)]
    B, Sl, _, D = tensors[0].shape
    hs = []
    for t in tensors:
        if t.dim() != 4 or t.shape[0] != B or t.shape[1] != Sl or t.shape[3] != D:
            raise ValueError("packed all-to-all needs [B, S_local, H_i, D] tensors of one B, S_local, D")
        if t.shape[2] % P:
            raise ValueError(f"number of heads ({t.shape[2]}) must be divisible by the group size ({P})")
        hs.append(t.shape[2] // P)
    hsum = sum(hs)
    send = torch.empty((P, B, Sl, hsum, D), dtype=tensors[0].dtype, device=tensors[0].device)
    o = 0
    for i, (t, h) in enumerate(zip(tensors, hs)):
        dst, src = send[:, :, :, o:o + h], t.unflatten(2, (P, h)).permute(2, 0, 1, 3, 4)
        if rope is not None and i < rope[3]:
            from .rope import rope_copy
            rope_copy(dst, src, rope[0], rope[1], 2, rope[2])    # dims (P, B, S_local, h): position = dim 2
        else:
            copy_fn(dst, src)
        o += h
    recv = _exchange(send, group)                           # [P_src, B, Sl, hsum, D]
    if B == 1:
        full = recv.view(1, P * Sl, hsum, D)
    else:
        full = torch.empty((B, P * Sl, hsum, D), dtype=recv.dtype, device=recv.device)
        copy_fn(full.view(B, P, Sl, hsum, D), recv.permute(1, 0, 2, 3, 4))
    outs, o = [], 0
    for h in hs:
        outs.append(full[:, :, o:o + h])
        o += h
    return outs


def seq_all_to_all_packed(tensors, group=None, copy_fn: Callable = strided_copy):
    """Head -> sequence reshard of several [B, S, H_i/P, D] tensors (dq, dk, dv) as ONE
    message; the inverse of heads_all_to_all_packed. Tensors that are adjacent head
    slices of one [1, S, sum h_i, D] buffer are sent from where they lie."""
    P = _world(group)
    if P == 1:
        return list(tensors)
    B, S, _, D = tensors[0].shape
    if S % P:
        raise ValueError(f"sequence length ({S}) must be divisible by the group size ({P})")
    Sl = S // P
    hs = [t.shape[2] for t in tensors]
    hsum = sum(hs)
    t0 = tensors[0]
    in_place = B == 1 and t0.stride() == (S * hsum * D, hsum * D, D, 1)
    o = 0
    for t, h in zip(tensors, hs):
        in_place = in_place and t.stride() == t0.stride() and \
            t.data_ptr() == t0.data_ptr() + o * D * t0.element_size()
        o += h
    if in_place:
        send = torch.as_strided(t0, (P, 1, Sl, hsum, D), (Sl * hsum * D, Sl * hsum * D, hsum * D, D, 1))
    else:
        send = torch.empty((P, B, Sl, hsum, D), dtype=t0.dtype, device=t0.device)
        o = 0
        for t, h in zip(tensors, hs):
            copy_fn(send[:, :, :, o:o + h], t.unflatten(1, (P, Sl)).permute(1, 0, 2, 3, 4))
            o += h
    recv = _exchange(send, group)                           # [P_src (head group), B, Sl, hsum, D]
    outs, o = [], 0
    for h in hs:
        out = torch.empty((B, Sl, P * h, D), dtype=t0.dtype, device=t0.device)
        copy_fn(out.view(B, Sl, P, h, D), recv[:, :, :, o:o + h].permute(1, 2, 0, 3, 4))
        outs.append(out)
        o += h
    return outs


class HeadsAllToAllPacked(torch.autograd.Function):
    """Autograd form of heads_all_to_all_packed: `apply(group, q, k, v)` reshards the
    tensors sequence -> heads as one message and returns views of the gathered buffer; the
    gradients go back head -> sequence as one message too."""

    @staticmethod
    def forward(ctx, group, *tensors):
        ctx.group = group
        outs = heads_all_to_all_packed(tensors, group=group)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        grads = [g if g.stride(-1) == 1 else g.contiguous() for g in grads]
        return (None, *seq_all_to_all_packed(grads, group=ctx.group))


class SeqAllToAll4D(torch.autograd.Function):
    """Counterpart of sp_aurora/comm/all_to_all.py:183 and
    sp_aurora/intel_ulysses_attn.py:25; the gradient is the inverse reshard
    (the reference's class-based backward raises, :203-205)."""

    @staticmethod
    def forward(ctx, group, input, scatter_idx, gather_idx, use_sync=False):
        ctx.group, ctx.scatter_idx, ctx.gather_idx, ctx.use_sync = group, scatter_idx, gather_idx, use_sync
        return all_to_all_4D(input, scatter_idx, gather_idx, group=group, use_sync=use_sync)

    @staticmethod
    def backward(ctx, grad_output):
        g = grad_output if grad_output.stride(-1) == 1 else grad_output.contiguous()
        return (None, all_to_all_4D(g, ctx.gather_idx, ctx.scatter_idx, group=ctx.group,
                                    use_sync=ctx.use_sync), None, None, None)


class SeqAllToAll5D(torch.autograd.Function):
    """Counterpart of sp_aurora/comm/all_to_all.py:338."""

    @staticmethod
    def forward(ctx, group, input, scatter_idx=3, gather_idx=1, use_sync=False):
        ctx.group, ctx.scatter_idx, ctx.gather_idx, ctx.use_sync = group, scatter_idx, gather_idx, use_sync
        return all_to_all_5D(input, scatter_idx, gather_idx, group=group, use_sync=use_sync)

    @staticmethod
    def backward(ctx, grad_output):
        g = grad_output if grad_output.stride(-1) == 1 else grad_output.contiguous()
        return (None, all_to_all_5D(g, ctx.gather_idx, ctx.scatter_idx, group=ctx.group,
                                    use_sync=ctx.use_sync), None, None, None)


def seq_all_to_all_4d_inference(group, input, scatter_idx, gather_idx, use_sync=False):
    """Forward-only helper, counterpart of sp_aurora/comm/all_to_all.py:208."""
    return all_to_all_4D(input, scatter_idx, gather_idx, group=group, use_sync=use_sync)


def reshard_lse(lse: torch.Tensor, group, to_seq_shard: bool = True) -> torch.Tensor:
    """lse [B, H/P, S] (local heads, full sequence) -> [B, H, S/P] (all heads,
    local sequence chunk). Tiny fp32 tensor (1/D of `out`): plain torch views
    around one all_to_all_single."""
    P = _world(group)
    if P == 1:
        return lse
    B, h, S = lse.shape
    Sl = S // P
    send = lse.view(B, h, P, Sl).permute(2, 0, 1, 3).contiguous()      # [P_dst, B, h, Sl]
    recv = _exchange(send, group)                                      # [P_src(head grp), B, h, Sl]
    return recv.permute(1, 0, 2, 3).reshape(B, P * h, Sl).contiguous()
