"""Packed-stream ("llama3") sequence parallelism: all-gather K/V, local varlen attention.

The reference's HF adapter imports `llama3_flash_attn_varlen_func` and
`llama3_flash_attn_prepare_cu_seqlens` (sp_aurora/adapters/hf_adapter.py:13-16,41-47,141-155) from
a module the package does not contain. Here they exist, with the calling convention the adapter
uses.

Layout: the sequences of a batch are packed back to back into one stream of T tokens
(`cu_seqlens`, global, int [n_seq + 1]); rank r of W holds the contiguous tokens
[r*T/W, (r+1)*T/W) of q, k and v as [T/W, H, D]. A sequence may start on one rank and end on
another. Each rank attends its own query tokens to the keys of the sequences they belong to:

  forward   all-gather K and V over the group, `heads_k_stride` kv heads at a time (the gather
            of the next group of heads runs while the current one is computed), then one kernel
            call per sequence segment held here: queries = the segment, keys = the sequence from
            its first token up to the segment's end (causal; bottom-right aligned through the
            kernels' `causal_off`) or to the sequence's end (non-causal);
  backward  the same gathers; dQ straight into the result; dK/dV of a head group into an fp32
            buffer over the gathered key range, reduce-scattered to the owning ranks.

Every query row and every key row of a head group is written by exactly one kernel call per
rank, so nothing is accumulated on a GPU and the result does not depend on scheduling.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib, local_attn
from .local_attn import check_unsupported_kwargs

__all__ = ["llama3_flash_attn_prepare_cu_seqlens", "llama3_flash_attn_varlen_func",
           "Llama3FlashAttnVarlenFunc"]


def _as_list(cu) -> List[int]:
    return [int(x) for x in (cu.tolist() if isinstance(cu, torch.Tensor) else cu)]


def llama3_flash_attn_prepare_cu_seqlens(cu_seqlens, causal: bool, rank: int, world_size: int):
    """Per-rank segment tables for a packed stream split evenly over `world_size` ranks.

    Returns (cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, local_k_slice):
    cu_seqlens_q  int32 [m + 1]: the rank's query tokens cut at sequence boundaries (local
                  offsets, 0 .. T/W);
    cu_seqlens_k  int32 [m + 1]: the keys of the same m segments, as offsets into the gathered
                  key stream restricted to `local_k_slice`;
    local_k_slice slice of the global key stream that this rank needs at all.
    The tensors live on cu_seqlens' device (CPU for a list)."""
    cu = _as_list(cu_seqlens)
    if len(cu) < 2 or cu[0] != 0 or any(b < a for a, b in zip(cu, cu[1:])):
        raise ValueError(f"cu_seqlens {cu} must rise from 0")
    total = cu[-1]
    if world_size <= 0 or total % world_size:
        raise ValueError(f"{total} packed tokens do not split evenly over {world_size} ranks")
    per = total // world_size
    lo, hi = rank * per, (rank + 1) * per
    q_bounds, k_bounds = [0], [0]
    k_start = None
    k_end = lo
    for s0, s1 in zip(cu, cu[1:]):
        a, b = max(s0, lo), min(s1, hi)
        if b <= a:
            continue
        if k_start is None:
            k_start = s0
        k_end = b if causal else s1
        q_bounds.append(b - lo)
        k_bounds.append(k_end - k_start)
    if k_start is None:           # no tokens on this rank (T == 0)
        k_start = lo
    dev = cu_seqlens.device if isinstance(cu_seqlens, torch.Tensor) else None
    cq = torch.tensor(q_bounds, dtype=torch.int32, device=dev)
    ck = torch.tensor(k_bounds, dtype=torch.int32, device=dev)
    max_q = max((b - a for a, b in zip(q_bounds, q_bounds[1:])), default=0)
    max_k = max((b - a for a, b in zip(k_bounds, k_bounds[1:])), default=0)
    return cq, ck, max_q, max_k, slice(k_start, k_end)


def _segments(cu_q, cu_k) -> List[Tuple[int, int, int, int]]:
    bq, bk = _as_list(cu_q), _as_list(cu_k)
    if len(bq) != len(bk):
        raise ValueError("cu_seqlens_q and cu_seqlens_k describe different numbers of segments")
    segs = []
    for i in range(len(bq) - 1):
        if bq[i + 1] > bq[i]:
            if bk[i + 1] - bk[i] < bq[i + 1] - bq[i]:
                raise ValueError("a segment has fewer keys than queries")
            segs.append((bq[i], bq[i + 1], bk[i], bk[i + 1]))
    return segs


class _Gather:
    """All-gather of one head group of K and of V: [T/W, hs, D] per rank -> [T, hs, D] each
    (rank-major along the token axis, which is the stream order)."""

    def __init__(self, group, world: int):
        self.group, self.world = group, world

    def start(self, k, v, h0: int, h1: int):
        if self.world == 1:
            return (k[:, h0:h1], v[:, h0:h1]), ()
        outs, works = [], []
        for t in (k, v):
            local = t[:, h0:h1].contiguous()
            full = torch.empty((self.world * local.shape[0],) + tuple(local.shape[1:]),
                               dtype=local.dtype, device=local.device)
            works.append(dist.all_gather_into_tensor(full, local, group=self.group, async_op=True))
            outs.append(full)
        return tuple(outs), tuple(works)

    @staticmethod
    def finish(tensors, works):
        for w in works:
            w.wait()
        return tensors


def _reduce_scatter_rows(full: torch.Tensor, group, world: int) -> torch.Tensor:
    """Sum a [T, hs, D] tensor over the ranks and keep this rank's [T/W, hs, D] rows."""
    if world == 1:
        return full
    mine = torch.empty((full.shape[0] // world,) + tuple(full.shape[1:]), dtype=full.dtype,
                       device=full.device)
    dist.reduce_scatter_tensor(mine, full, group=group)
    return mine


def llama3_forward(group, q, k, v, segs, k_slice: slice, heads_k_stride: int, softmax_scale: float,
                   causal: bool, fwd_step: Callable = local_attn.attn_fwd_step):
    """out [T/W, Hq, D] (q.dtype) and lse [Hq, T/W] fp32 for the rank's packed queries."""
    W = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
    Tl, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    out = torch.empty_like(q)
    lse = torch.empty((Hq, Tl), dtype=torch.float32, device=q.device)
    gather = _Gather(group, W)
    groups = [(h0, min(h0 + heads_k_stride, Hkv)) for h0 in range(0, Hkv, heads_k_stride)]
    pending = gather.start(k, v, *groups[0])
    for gi, (h0, h1) in enumerate(groups):
        kfull, vfull = gather.finish(*pending)
        if gi + 1 < len(groups):
            pending = gather.start(k, v, *groups[gi + 1])
        kg, vg = kfull[k_slice], vfull[k_slice]
        for qa, qb, ka, kb in segs:
            fwd_step(q[qa:qb, h0 * g:h1 * g].unsqueeze(0), kg[ka:kb].unsqueeze(0), vg[ka:kb].unsqueeze(0),
                     softmax_scale, causal, lse[h0 * g:h1 * g, qa:qb].unsqueeze(0),
                     out=out[qa:qb, h0 * g:h1 * g].unsqueeze(0),
                     causal_off=(kb - ka) - (qb - qa))
    return out, lse


def llama3_backward(group, dout, q, k, v, out, lse, segs, k_slice: slice, heads_k_stride: int,
                    softmax_scale: float, causal: bool, deterministic: bool = False,
                    bwd_step: Callable = local_attn.attn_bwd_step,
                    delta_fn: Callable = local_attn.bwd_delta,
                    cast_fn: Callable = local_attn.cast_from_f32,
                    reduce_scatter: Callable = _reduce_scatter_rows):
    """dq, dk, dv [T/W, H, D] in q.dtype."""
    W = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
    Tl, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    dt = q.dtype
    acc_dt = torch.float32
    delta = delta_fn(out.unsqueeze(0), dout.unsqueeze(0))[0]          # [Hq, T/W]
    dq = torch.zeros_like(q) if not segs else torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    gather = _Gather(group, W)
    groups = [(h0, min(h0 + heads_k_stride, Hkv)) for h0 in range(0, Hkv, heads_k_stride)]
    pending = gather.start(k, v, *groups[0])
    T = Tl * W
    for gi, (h0, h1) in enumerate(groups):
        kfull, vfull = gather.finish(*pending)
        if gi + 1 < len(groups):
            pending = gather.start(k, v, *groups[gi + 1])
        kg, vg = kfull[k_slice], vfull[k_slice]
        hs = h1 - h0
        # fp32 gradients over the whole key stream of this head group: rows outside the keys
        # this rank touched stay zero and the reduce-scatter sums the ranks' shares
        dk_full = torch.zeros((T, hs, D), dtype=acc_dt, device=q.device)
        dv_full = torch.zeros((T, hs, D), dtype=acc_dt, device=q.device)
        dkg, dvg = dk_full[k_slice], dv_full[k_slice]
        for qa, qb, ka, kb in segs:
            hq = slice(h0 * g, h1 * g)
            bwd_step(q[qa:qb, hq].unsqueeze(0), kg[ka:kb].unsqueeze(0), vg[ka:kb].unsqueeze(0),
                     dout[qa:qb, hq].unsqueeze(0), lse[hq, qa:qb].unsqueeze(0),
                     delta[hq, qa:qb].unsqueeze(0), softmax_scale, causal, None,
                     dkg[ka:kb].unsqueeze(0), dvg[ka:kb].unsqueeze(0),
                     causal_off=(kb - ka) - (qb - qa), dq=dq[qa:qb, hq].unsqueeze(0),
                     dq_overwrite=True, deterministic=deterministic)
        for full, dst in ((dk_full, dk), (dv_full, dv)):
            mine = reduce_scatter(full, group, W)                     # [T/W, hs, D] fp32
            if dt == torch.float32:
                dst[:, h0:h1].copy_(mine)
            else:
                dst[:, h0:h1].copy_(cast_fn(mine.unsqueeze(0), dt)[0])
    return dq, dk, dv


class Llama3FlashAttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, heads_k_stride, local_k_slice,
                softmax_scale, causal, deterministic, return_softmax, group):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        local_attn.check_qkv(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0))
        segs = _segments(cu_seqlens_q, cu_seqlens_k)
        if segs and segs[-1][1] != q.shape[0]:
            raise ValueError("cu_seqlens_q must end at the number of local query tokens")
        stride = int(heads_k_stride) if heads_k_stride else k.shape[1]
        if stride <= 0 or k.shape[1] % stride:
            raise ValueError(f"heads_k_stride {heads_k_stride} must divide the {k.shape[1]} kv heads")
        out, lse = llama3_forward(group, q, k, v, segs, local_k_slice, stride, softmax_scale, causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.segs, ctx.k_slice, ctx.stride = segs, local_k_slice, stride
        ctx.softmax_scale, ctx.causal, ctx.group = softmax_scale, bool(causal), group
        ctx.deterministic = bool(deterministic)
        return (out, lse, None) if return_softmax else out

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, out, lse = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dq, dk, dv = llama3_backward(ctx.group, dout, q, k, v, out, lse, ctx.segs, ctx.k_slice,
                                     ctx.stride, ctx.softmax_scale, ctx.causal, ctx.deterministic)
        _lib.maybe_check_status()
        return (dq, dk, dv) + (None,) * 9


def llama3_flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q=None,
                                  max_seqlen_k=None, heads_k_stride: Optional[int] = None,
                                  local_k_slice: Optional[slice] = None, dropout_p=0.0,
                                  softmax_scale=None, causal=False, window_size=(-1, -1),
                                  alibi_slopes=None, deterministic=False, return_attn_probs=False,
                                  group=None):
    """Attention over a packed stream split evenly over the ranks of `group`.

    q, k, v [T/W, H, D]: the rank's tokens; `cu_seqlens_q`, `cu_seqlens_k`, `local_k_slice` as
    returned by `llama3_flash_attn_prepare_cu_seqlens`; `heads_k_stride` kv heads are gathered
    and processed at a time (default: all), which bounds the gathered K/V and the fp32 dK/dV
    buffers to T * heads_k_stride * D elements each. Returns out [T/W, Hq, D], or
    (out, lse [Hq, T/W] fp32, None) with return_attn_probs. `max_seqlen_*` are accepted for
    signature compatibility."""
    check_unsupported_kwargs(dropout_p, window_size, alibi_slopes)
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dim() != 3:
            raise ValueError(f"{name} must be packed [tokens, H, D], got {tuple(t.shape)}")
    if local_k_slice is None:
        raise ValueError("local_k_slice is required (llama3_flash_attn_prepare_cu_seqlens returns it)")
    return Llama3FlashAttnVarlenFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, heads_k_stride,
                                           local_k_slice, softmax_scale, causal, deterministic,
                                           return_attn_probs, group)
