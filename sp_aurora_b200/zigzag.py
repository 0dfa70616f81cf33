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
Internal layouts keep the half index outermost so every call sees contiguous
[B, S/2, H, D] operands: q_z [2,B,h,Hq,D]; K|V message [2(half),2(k|v),B,h,Hkv,D];
lse_z [2,B,Hq,h]; accumulators alike.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist

from . import local_attn


def _group_info(group):
    return dist.get_rank(group), dist.get_world_size(group)


def _global(group, r):
    return r if group is None else dist.get_global_rank(group, r)


def half_owner(c: int, W: int) -> Tuple[int, int]:
    """(rank, slot) that works on half-chunk c in the zigzag layout."""
    return (c, 0) if c < W else (2 * W - 1 - c, 1)


def exchange_halves(pairs: Sequence[Tuple[List[torch.Tensor], List[torch.Tensor]]], group,
                    to_zigzag: bool) -> None:
    """Move half-chunks between the contiguous layout (rank r holds half-chunks
    2r, 2r+1) and the zigzag layout (rank r holds r, 2W-1-r).

    `pairs` is a list of (src_halves, dst_halves): two contiguous tensors each.
    to_zigzag=True : src_halves[i] is half-chunk 2r+i, dst_halves[j] receives slot j.
    to_zigzag=False: src_halves[j] is slot j, dst_halves[i] receives half-chunk 2r+i.
    All transfers of all pairs go out as one batched group (ordered per peer)."""
    from .ring import RingComm
    if RingComm.FAKE:          # measurement aid: local copies only, no transfers
        for src, dst in pairs:
            for i in range(2):
                dst[i].copy_(src[i])
        return
    r, W = _group_info(group)
    ops = []
    local = []
    for src, dst in pairs:
        for i in range(2):
            c = 2 * r + i                      # half-chunk living here in contiguous layout
            zr, zs = half_owner(c, W)          # where it lives in zigzag layout
            if to_zigzag:
                if zr == r:
                    local.append((dst[zs], src[i]))
                else:
                    ops.append(dist.P2POp(dist.isend, src[i], _global(group, zr), group=group))
            else:
                if zr == r:
                    local.append((dst[i], src[zs]))
                else:
                    ops.append(dist.P2POp(dist.irecv, dst[i], _global(group, zr), group=group))
        for j in range(2):
            c = r if j == 0 else 2 * W - 1 - r  # half-chunk living here in zigzag layout
            cr = c // 2                         # its rank in contiguous layout
            if cr == r:
                continue                        # handled as a local copy above
            if to_zigzag:
                ops.append(dist.P2POp(dist.irecv, dst[j], _global(group, cr), group=group))
            else:
                ops.append(dist.P2POp(dist.isend, src[j], _global(group, cr), group=group))
    reqs = dist.batch_isend_irecv(ops) if ops else []
    for d, s in local:
        d.copy_(s)
    for req in reqs:
        req.wait()


def _halves(x: torch.Tensor) -> List[torch.Tensor]:
    """Two contiguous [B, S/2, ...] halves of a [B, S, ...] tensor."""
    h = x.shape[1] // 2
    return [x[:, :h].contiguous(), x[:, h:].contiguous()]


def _step_calls(step: int, r: int, W: int):
    """(q_half, k_half, causal) calls of one ring step (see module docstring)."""
    src = (r - step) % W
    if step == 0:
        return [(0, 0, True), (1, 0, False), (1, 1, True)]
    if src < r:
        return [(0, 0, False), (1, 0, False)]
    return [(1, 0, False), (1, 1, False)]


def zigzag_ring_forward(group, q, k, v, softmax_scale: float,
                        fwd_step: Callable = local_attn.attn_fwd_step,
                        cast_fn: Callable = local_attn.cast_from_f32, need_lse: bool = True):
    """Causal ring forward over contiguous shards with internal zigzag balance.
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
    q_z = torch.empty((2, B, h, Hq, D), dtype=dt, device=dev)
    kv_z = torch.empty((2, 2, B, h, Hkv, D), dtype=dt, device=dev)
    exchange_halves([(_halves(q), [q_z[0], q_z[1]]),
                     (_halves(k), [kv_z[0, 0], kv_z[1, 0]]),
                     (_halves(v), [kv_z[0, 1], kv_z[1, 1]])], group, to_zigzag=True)

    out_z = torch.empty((2, B, h, Hq, D), dtype=dt, device=dev)
    acc_z = torch.empty((2, B, h, Hq, D), dtype=torch.float32, device=dev)
    lse_z = torch.empty((2, B, Hq, h), dtype=torch.float32, device=dev)
    plan = [_step_calls(s, r, W) for s in range(W)]
    n_calls = [sum(1 for st in plan for c in st if c[0] == qh) for qh in (0, 1)]
    done = [0, 0]
    bufs = [torch.empty_like(kv_z), torch.empty_like(kv_z)]
    cur = kv_z
    for step in range(W):
        nxt = None
        if step + 1 != W:
            nxt = comm.send_recv(cur, bufs[step % 2])
            comm.commit()
        for qh, kh, causal in plan[step]:
            first, last = done[qh] == 0, done[qh] + 1 == n_calls[qh]
            fwd_step(q_z[qh], cur[kh, 0], cur[kh, 1], softmax_scale, causal, lse_z[qh],
                     out=out_z[qh] if last else None,
                     out_acc=None if (first and last) else acc_z[qh], merge_prev=not first)
            done[qh] += 1
        if nxt is not None:
            comm.wait()
            cur = nxt

    out = torch.empty((B, S, Hq, D), dtype=dt, device=dev)
    o_dst = [torch.empty((B, h, Hq, D), dtype=dt, device=dev) for _ in range(2)]
    pairs = [([out_z[0], out_z[1]], o_dst)]
    lse = None
    if need_lse:     # the backward uses lse_z; the contiguous lse is only for the caller
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
        l_dst = [torch.empty((B, Hq, h), dtype=torch.float32, device=dev) for _ in range(2)]
        pairs.append(([lse_z[0], lse_z[1]], l_dst))
    exchange_halves(pairs, group, to_zigzag=False)
    out[:, :h].copy_(o_dst[0])
    out[:, h:].copy_(o_dst[1])
    if need_lse:
        lse[:, :, :h].copy_(l_dst[0])
        lse[:, :, h:].copy_(l_dst[1])
    return out, lse, (q_z, kv_z, out_z, lse_z)


def zigzag_ring_backward(group, dout, q_z, kv_z, out_z, lse_z, softmax_scale: float,
                         bwd_step: Callable = local_attn.attn_bwd_step,
                         delta_fn: Callable = local_attn.bwd_delta,
                         cast_fn: Callable = local_attn.cast_from_f32):
    """Backward of zigzag_ring_forward. `dout` is the contiguous shard; returns
    (dq, dk, dv) as contiguous shards in q's dtype."""
    from .ring import RingComm
    kv_comm = RingComm(group)
    d_kv_comm = RingComm(group)
    W, r = kv_comm.world_size, kv_comm.rank
    _, B, h, Hq, D = q_z.shape
    Hkv = kv_z.shape[4]
    dev, dt = q_z.device, q_z.dtype
    do_z = torch.empty((2, B, h, Hq, D), dtype=dt, device=dev)
    exchange_halves([(_halves(dout), [do_z[0], do_z[1]])], group, to_zigzag=True)
    delta_z = [delta_fn(out_z[i], do_z[i]) for i in range(2)]
    dq_acc = torch.zeros((2, B, h, Hq, D), dtype=torch.float32, device=dev)
    # dK|dV: each step's kernels write into `local`; the partial that travelled here
    # with the K|V block is folded in AFTER the kernels (so its transfer overlaps
    # them) and the sum is sent on. Layout [2(half), 2(k|v), B, h, Hkv, D] fp32.
    local = torch.empty((2, 2, B, h, Hkv, D), dtype=torch.float32, device=dev)
    dkv_bufs = [torch.empty_like(local) for _ in range(3)]
    kv_bufs = [torch.empty_like(kv_z), torch.empty_like(kv_z)]
    cur = kv_z
    next_dkv = None
    for step in range(W):
        nxt = None
        if step + 1 != W:
            nxt = kv_comm.send_recv(cur, kv_bufs[step % 2])
            kv_comm.commit()
        written = [False, False]
        tgt = dkv_bufs[0] if step == 0 else local   # step 0 (both key halves) starts the sum
        for qh, kh, causal in _step_calls(step, r, W):
            bwd_step(q_z[qh], cur[kh, 0], cur[kh, 1], do_z[qh], lse_z[qh], delta_z[qh],
                     softmax_scale, causal, dq_acc[qh], tgt[kh, 0], tgt[kh, 1],
                     dkv_accumulate=written[kh])
            written[kh] = True
        if step == 0:
            send = dkv_bufs[0]
        else:
            d_kv_comm.wait()           # partial for this block, sent during the previous step
            send = next_dkv
            for kh in range(2):
                if written[kh]:
                    send[kh].add_(local[kh])
        if nxt is not None:
            kv_comm.wait()
            cur = nxt
        recv = dkv_bufs[(step + 1) % 3]
        next_dkv = d_kv_comm.send_recv(send, recv)
        d_kv_comm.commit()
    d_kv_comm.wait()

    def to_dt(x):  # fp32 [B,h,H,D] -> dt
        return x if dt == torch.float32 else cast_fn(x, dt)

    dq_h = [to_dt(dq_acc[i]) for i in range(2)]
    dk_h = [to_dt(next_dkv[i, 0]) for i in range(2)]
    dv_h = [to_dt(next_dkv[i, 1]) for i in range(2)]
    S = 2 * h
    dq = torch.empty((B, S, Hq, D), dtype=dt, device=dev)
    dk = torch.empty((B, S, Hkv, D), dtype=dt, device=dev)
    dv = torch.empty((B, S, Hkv, D), dtype=dt, device=dev)
    dst = [[torch.empty_like(t[0]), torch.empty_like(t[1])] for t in (dq_h, dk_h, dv_h)]
    exchange_halves([(dq_h, dst[0]), (dk_h, dst[1]), (dv_h, dst[2])], group, to_zigzag=False)
    for full, halves in ((dq, dst[0]), (dk, dst[1]), (dv, dst[2])):
        full[:, :h].copy_(halves[0])
        full[:, h:].copy_(halves[1])
    return dq, dk, dv
