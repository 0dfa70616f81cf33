"""Load-balanced causal ring: internal zigzag re-layout of contiguous shards.

With contiguous shards (the reference's layout, sp_aurora/intel_ring_flash_attn.py:72-134)
rank r of a causal ring computes r+1 blocks while rank 0 computes one, so the
slowest rank does (2W)/(W+1) times the average work. Here the public functions
still take and return contiguous shards, but inside a causal ring of W > 1 ranks
the sequence is cut into 2W half-chunks and rank r works on half-chunks
(r, 2W-1-r): one cheap exchange in, one out. Every ring step then costs every
rank the same (two half-by-half blocks), and the results are the same numbers.

Per step, with the K|V pair that started on rank src = (r - step) mod W
(half-chunks src and 2W-1-src) and local query halves q0 (chunk r), q1 (chunk 2W-1-r):
  step 0  : (q0,k0) causal, (q1,k0) full, (q1,k1) causal
  src < r : (q0,k0) full,   (q1,k0) full          (k1 is later than both)
  src > r : (q1,k0) full,   (q1,k1) full          (q0 is earlier than both)
For batch size 1 the two halves of a tensor are adjacent rows of one [1, 2h, H, D]
tensor, and calls that share a query or key operand are merged into one launch:
  step 0  : (q1,[k0;k1]) causal with offset h,  (q0,k0) causal
  src < r : ([q0;q1],k0) full
  src > r : (q1,[k0;k1]) full
Internal layouts: q_z, out_z, accumulators [2(half),B,h,Hq,D]; K|V message
[2(k|v),2(half),B,h,Hkv,D]; lse_z, delta_z [B,Hq,2(half),h].
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib, local_attn


def _group_info(group):
    return dist.get_rank(group), dist.get_world_size(group)


def _global(group, r):
    return r if group is None else dist.get_global_rank(group, r)


def half_owner(c: int, W: int) -> Tuple[int, int]:
    """(rank, slot) that works on half-chunk c in the zigzag layout."""
    return (c, 0) if c < W else (2 * W - 1 - c, 1)


def exchange_halves(pairs: Sequence[Tuple[List[torch.Tensor], List[torch.Tensor]]], group,
                    to_zigzag: bool, shift: int = 0, defer: bool = False):
    """Move half-chunks between the contiguous layout (rank r holds half-chunks
    2r, 2r+1) and the zigzag layout (rank r holds the pair b, 2W-1-b of block
    b = (r - shift) mod W; shift = 0 is the resting layout, shift = s is where a block
    sits after s ring hops).

    `pairs` is a list of (src_halves, dst_halves): two tensors each; sources must be
    contiguous, destinations may be strided views (received through a staging tensor).
    to_zigzag=True : src_halves[i] is half-chunk 2r+i, dst_halves[j] receives slot j.
    to_zigzag=False: src_halves[j] is slot j, dst_halves[i] receives half-chunk 2r+i.
    All transfers of all pairs go out as one batched group (ordered per peer).
    With defer=True the transfers are posted and a function is returned that makes the
    current stream wait for them (and finishes staged copies); otherwise that happens
    before returning."""
    from .ring import RingComm
    if RingComm.FAKE:          # measurement aid: local copies only, no transfers
        for src, dst in pairs:
            for i in range(2):
                dst[i].copy_(src[i])
        return (lambda: None) if defer else None
    r, W = _group_info(group)
    blk = (r - shift) % W      # the block whose pair this rank holds in the zigzag layout
    ops = []
    local = []       # (dst, src) copies that can run at once
    after = []       # (dst, staging) copies that wait for their receive

    def recv_into(view, peer):
        tgt = view
        if not view.is_contiguous():
            tgt = torch.empty(view.shape, dtype=view.dtype, device=view.device)
            after.append((view, tgt))
        ops.append(dist.P2POp(dist.irecv, tgt, _global(group, peer), group=group))

    for src, dst in pairs:
        for i in range(2):
            c = 2 * r + i                      # half-chunk living here in contiguous layout
            zb, zs = half_owner(c, W)          # its block and slot in the zigzag layout
            zr = (zb + shift) % W              # the rank holding that block
            if to_zigzag:
                if zr == r:
                    local.append((dst[zs], src[i]))
                else:
                    ops.append(dist.P2POp(dist.isend, src[i], _global(group, zr), group=group))
            else:
                if zr == r:
                    local.append((dst[i], src[zs]))
                else:
                    recv_into(dst[i], zr)
        for j in range(2):
            c = blk if j == 0 else 2 * W - 1 - blk   # half-chunk living here in zigzag layout
            cr = c // 2                              # its rank in contiguous layout
            if cr == r:
                continue                             # handled as a local copy above
            if to_zigzag:
                recv_into(dst[j], cr)
            else:
                ops.append(dist.P2POp(dist.isend, src[j], _global(group, cr), group=group))
    reqs = dist.batch_isend_irecv(ops) if ops else []
    for d, s in local:
        d.copy_(s)

    def finish():
        for req in reqs:
            req.wait()
        for d, s in after:
            d.copy_(s)

    if defer:
        return finish
    finish()


def _halves(x: torch.Tensor) -> List[torch.Tensor]:
    """The two [B, S/2, ...] halves of a [B, S, ...] tensor, contiguous (views when the
    batch size is 1, copies otherwise)."""
    h = x.shape[1] // 2
    return [x[:, :h].contiguous(), x[:, h:].contiguous()]


def _step_calls(step: int, r: int, W: int):
    """(q_half, k_half, causal) blocks of one ring step (see module docstring)."""
    src = (r - step) % W
    if step == 0:
        return [(0, 0, True), (1, 0, False), (1, 1, True)]
    if src < r:
        return [(0, 0, False), (1, 0, False)]
    return [(1, 0, False), (1, 1, False)]


def _plan(step: int, r: int, W: int, merged: bool):
    """Kernel calls of one ring step as (q_lo, q_n, k_lo, k_n, causal, offset_halves):
    query halves [q_lo, q_lo+q_n) against key halves [k_lo, k_lo+k_n); a causal call
    lets query i see key j <= i + offset_halves*h. Within a step, a call that overwrites
    the dK/dV of a key half precedes the calls that add to it."""
    src = (r - step) % W
    if merged:
        if step == 0:
            return [(1, 1, 0, 2, True, 1), (0, 1, 0, 1, True, 0)]
        if src < r:
            return [(0, 2, 0, 1, False, 0)]
        return [(1, 1, 0, 2, False, 0)]
    if step == 0:
        return [(1, 1, 0, 1, False, 0), (1, 1, 1, 1, True, 0), (0, 1, 0, 1, True, 0)]
    if src < r:
        return [(0, 1, 0, 1, False, 0), (1, 1, 0, 1, False, 0)]
    return [(1, 1, 0, 1, False, 0), (1, 1, 1, 1, False, 0)]


def _rows(x_z: torch.Tensor, lo: int, n: int) -> torch.Tensor:
    """Halves [lo, lo+n) of a [2, B, h, H, D] tensor as one [B, n*h, H, D] tensor
    (n == 2 only for batch size 1, where the halves are adjacent rows)."""
    if n == 1:
        return x_z[lo]
    _, B, h, H, D = x_z.shape
    return x_z.view(B, 2 * h, H, D)


def _stat_rows(s_z: torch.Tensor, lo: int, n: int) -> torch.Tensor:
    """Halves [lo, lo+n) of a [B, Hq, 2, h] row-statistics tensor as [B, Hq, n*h]."""
    if n == 1:
        return s_z[:, :, lo]
    B, Hq, _, h = s_z.shape
    return s_z.view(B, Hq, 2 * h)


def _zigzag_layout_relayout(pairs, group, to_zigzag: bool, shift: int = 0, defer: bool = False):
    """exchange_halves for a caller whose shard already is in the zigzag layout: halves
    at rest are copied; a block that sits `shift` hops from home is sent there."""
    from .ring import RingComm
    r, W = _group_info(group)
    reqs, after = [], []
    if shift % W and not RingComm.FAKE:
        ops = []
        for src, dst in pairs:
            for j in range(2):
                tgt = dst[j]
                if not tgt.is_contiguous():
                    tgt = torch.empty(tgt.shape, dtype=tgt.dtype, device=tgt.device)
                    after.append((dst[j], tgt))
                ops.append(dist.P2POp(dist.isend, src[j], _global(group, (r - shift) % W), group=group))
                ops.append(dist.P2POp(dist.irecv, tgt, _global(group, (r + shift) % W), group=group))
        reqs = dist.batch_isend_irecv(ops)
    else:
        for src, dst in pairs:
            for i in range(2):
                dst[i].copy_(src[i])

    def finish():
        for req in reqs:
            req.wait()
        for d, s in after:
            d.copy_(s)

    if defer:
        return finish
    finish()


def zigzag_ring_forward(group, q, k, v, softmax_scale: float,
                        fwd_step: Callable = local_attn.attn_fwd_step,
                        cast_fn: Callable = local_attn.cast_from_f32, need_lse: bool = True,
                        input_layout: str = "contiguous"):
    """Causal ring forward with zigzag balance. `input_layout` "contiguous": rank r holds
    chunk r, re-laid out internally (one exchange in, one out); "zigzag": the shard already
    holds half-chunks r and 2W-1-r back to back and the result comes back in that layout.
    Returns (out [B,S,Hq,D], lse [B,Hq,S], saved) with `saved` = zigzag-layout
    tensors for the backward (q_z, kv_z, out_z, lse_z)."""
    from .ring import RingComm
    comm = RingComm(group)
    W, r = comm.world_size, comm.rank
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    if S % 2:
        raise ValueError("the balanced causal ring needs an even local sequence length")
    h = S // 2
    dev, dt = q.device, q.dtype
    stage = local_attn.stage
    q_z = torch.empty((2, B, h, Hq, D), dtype=dt, device=dev)
    kv_z = torch.empty((2, 2, B, h, Hkv, D), dtype=dt, device=dev)      # [k|v][half]
    relayout = exchange_halves if input_layout == "contiguous" else _zigzag_layout_relayout
    with stage("fwd.relayout_in", dev):
        relayout([(_halves(q), [q_z[0], q_z[1]]),
                  (_halves(k), [kv_z[0, 0], kv_z[0, 1]]),
                  (_halves(v), [kv_z[1, 0], kv_z[1, 1]])], group, to_zigzag=True)

    out_z = torch.empty((2, B, h, Hq, D), dtype=dt, device=dev)
    acc_z = torch.empty((2, B, h, Hq, D), dtype=torch.float32, device=dev)
    lse_z = torch.empty((B, Hq, 2, h), dtype=torch.float32, device=dev)
    merged = B == 1
    plan = [_plan(s, r, W, merged) for s in range(W)]
    n_calls = [sum(1 for st in plan for c in st if c[0] <= qh < c[0] + c[1]) for qh in (0, 1)]
    done = [0, 0]
    bufs = [torch.empty_like(kv_z), torch.empty_like(kv_z)]
    cur = kv_z
    for step in range(W):
        nxt = None
        if step + 1 != W:
            nxt = comm.send_recv(cur, bufs[step % 2])
            comm.commit()
        with stage("fwd.kernels", dev):
            for q_lo, q_n, k_lo, k_n, causal, off in plan[step]:
                halves = range(q_lo, q_lo + q_n)
                first = done[q_lo] == 0                       # the same for every half of a call
                last_any = any(done[i] + 1 == n_calls[i] for i in halves)
                last_all = all(done[i] + 1 == n_calls[i] for i in halves)
                fwd_step(_rows(q_z, q_lo, q_n), _rows(cur[0], k_lo, k_n), _rows(cur[1], k_lo, k_n),
                         softmax_scale, causal, _stat_rows(lse_z, q_lo, q_n),
                         out=_rows(out_z, q_lo, q_n) if last_any else None,
                         out_acc=None if (first and last_all) else _rows(acc_z, q_lo, q_n),
                         merge_prev=not first, causal_off=off * h)
                for i in halves:
                    done[i] += 1
        if nxt is not None:
            with stage("fwd.wait_kv", dev):
                comm.wait()
            cur = nxt

    out = torch.empty((B, S, Hq, D), dtype=dt, device=dev)
    pairs = [([out_z[0], out_z[1]], [out[:, :h], out[:, h:]])]
    lse = None
    if need_lse:     # the backward uses lse_z; the contiguous lse is only for the caller
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
        pairs.append(([lse_z[:, :, 0].contiguous(), lse_z[:, :, 1].contiguous()],
                      [lse[:, :, :h], lse[:, :, h:]]))
    with stage("fwd.relayout_out", dev):
        relayout(pairs, group, to_zigzag=False)
    return out, lse, (q_z, kv_z, out_z, lse_z)


def zigzag_ring_backward(group, dout, q_z, kv_z, out_z, lse_z, softmax_scale: float,
                         bwd_step: Callable = local_attn.attn_bwd_step,
                         delta_fn: Callable = local_attn.bwd_delta,
                         cast_fn: Callable = local_attn.cast_from_f32,
                         deterministic: bool = False, input_layout: str = "contiguous"):
    """Backward of zigzag_ring_forward. `dout` is the shard in the forward's `input_layout`;
    returns (dq, dk, dv) as shards of the same layout in q's dtype.

    Each step runs its dQ passes first and its dK/dV passes second: the travelling dK|dV
    partial of the current block is still in flight during the dQ passes, and the dK/dV
    passes then add straight into the received buffer, which is sent on."""
    from .ring import RingComm
    kv_comm = RingComm(group)
    d_kv_comm = RingComm(group)
    W, r = kv_comm.world_size, kv_comm.rank
    _, B, h, Hq, D = q_z.shape
    Hkv = kv_z.shape[4]
    dev, dt = q_z.device, q_z.dtype
    DQ, DKV = _lib.SPA_BWD_DQ_ONLY, _lib.SPA_BWD_DKV_ONLY
    stage = local_attn.stage
    do_z = torch.empty((2, B, h, Hq, D), dtype=dt, device=dev)
    relayout = exchange_halves if input_layout == "contiguous" else _zigzag_layout_relayout
    with stage("bwd.relayout_in", dev):
        relayout([(_halves(dout), [do_z[0], do_z[1]])], group, to_zigzag=True)
    merged = B == 1
    with stage("bwd.delta", dev):
        if merged:
            delta_z = delta_fn(_rows(out_z, 0, 2), _rows(do_z, 0, 2)).view(B, Hq, 2, h)
        else:
            delta_z = torch.empty((B, Hq, 2, h), dtype=torch.float32, device=dev)
            for i in range(2):
                delta_z[:, :, i].copy_(delta_fn(out_z[i], do_z[i]))
    dq_acc = torch.empty((2, B, h, Hq, D), dtype=torch.float32, device=dev)
    dq_z = torch.empty((2, B, h, Hq, D), dtype=dt, device=dev)
    plan = [_plan(s, r, W, merged) for s in range(W)]
    n_calls = [sum(1 for st in plan for c in st if c[0] <= qh < c[0] + c[1]) for qh in (0, 1)]
    done = [0, 0]
    # fp32 travelling partials [2(k|v), 2(half), B, h, Hkv, D], one message
    dkv_bufs = [torch.empty((2, 2, B, h, Hkv, D), dtype=torch.float32, device=dev) for _ in range(2)]
    kv_bufs = [torch.empty_like(kv_z), torch.empty_like(kv_z)]
    S = 2 * h
    dq = torch.empty((B, S, Hq, D), dtype=dt, device=dev)
    dk = torch.empty((B, S, Hkv, D), dtype=dt, device=dev)
    dv = torch.empty((B, S, Hkv, D), dtype=dt, device=dev)
    finish_dq = None
    cur = kv_z
    for step in range(W):
        nxt = None
        if step + 1 != W:
            nxt = kv_comm.send_recv(cur, kv_bufs[step % 2])
            kv_comm.commit()
        with stage("bwd.dq_kernels", dev):
            for q_lo, q_n, k_lo, k_n, causal, off in plan[step]:
                halves = range(q_lo, q_lo + q_n)
                first = done[q_lo] == 0
                last_any = any(done[i] + 1 == n_calls[i] for i in halves)
                bwd_step(_rows(q_z, q_lo, q_n), _rows(cur[0], k_lo, k_n), _rows(cur[1], k_lo, k_n),
                         _rows(do_z, q_lo, q_n), _stat_rows(lse_z, q_lo, q_n),
                         _stat_rows(delta_z, q_lo, q_n), softmax_scale, causal,
                         _rows(dq_acc, q_lo, q_n), None, None, causal_off=off * h,
                         dq=_rows(dq_z, q_lo, q_n) if last_any else None, dq_overwrite=first,
                         deterministic=deterministic, passes=DQ)
                for i in halves:
                    done[i] += 1
        if step + 1 == W:
            # dq is complete: its way back to the contiguous layout overlaps the last dK/dV pass
            with stage("bwd.relayout_out", dev):
                finish_dq = relayout([([dq_z[0], dq_z[1]], [dq[:, :h], dq[:, h:]])], group,
                                     to_zigzag=False, defer=True)
        tgt = dkv_bufs[step % 2]
        if step > 0:
            with stage("bwd.wait_dkv", dev):
                d_kv_comm.wait()       # the partial that travels with this block has arrived in tgt
        written = [step > 0, step > 0]
        with stage("bwd.dkv_kernels", dev):
            for q_lo, q_n, k_lo, k_n, causal, off in plan[step]:
                khalves = range(k_lo, k_lo + k_n)
                bwd_step(_rows(q_z, q_lo, q_n), _rows(cur[0], k_lo, k_n), _rows(cur[1], k_lo, k_n),
                         _rows(do_z, q_lo, q_n), _stat_rows(lse_z, q_lo, q_n),
                         _stat_rows(delta_z, q_lo, q_n), softmax_scale, causal,
                         None, _rows(tgt[0], k_lo, k_n), _rows(tgt[1], k_lo, k_n),
                         dkv_accumulate=written[k_lo], causal_off=off * h,
                         deterministic=deterministic, passes=DKV)
                for i in khalves:
                    written[i] = True
        if nxt is not None:
            with stage("bwd.wait_kv", dev):
                kv_comm.wait()
            cur = nxt
        if step + 1 != W:
            d_kv_comm.send_recv(tgt, dkv_bufs[(step + 1) % 2])
            d_kv_comm.commit()

    # The block now here has collected every rank's share.  It leaves in the element type
    # (the same rounding the owner would apply, half the bytes) and, for contiguous shards,
    # goes straight to the ranks that own its two halves instead of home first.
    with stage("bwd.cast_dkv", dev):
        done_dkv = dkv_bufs[(W - 1) % 2]
        msg = done_dkv
        if dt != torch.float32:
            msg = cast_fn(done_dkv.view(4 * B, h, Hkv, D), dt).view(2, 2, B, h, Hkv, D)
    with stage("bwd.wait_last_dkv_hop", dev):
        relayout([([msg[0, 0], msg[0, 1]], [dk[:, :h], dk[:, h:]]),
                  ([msg[1, 0], msg[1, 1]], [dv[:, :h], dv[:, h:]])], group,
                 to_zigzag=False, shift=W - 1)
    with stage("bwd.relayout_out", dev):
        finish_dq()
    return dq, dk, dv
