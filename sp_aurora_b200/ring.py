"""Ring (context-parallel) attention over contiguous sequence shards.

Mirrors sp_aurora/intel_ring_flash_attn.py (forward ring :17-150, backward ring
:153-271, autograd function :274-341, public functions :344-456) and the ring
communicator sp_aurora/utils.py:172-274, with the semantics the reference
intends (upstream algorithm kept in sp_aurora/ring_flash_attn.py:7-154):

* rank r of the group holds sequence chunk r; every step K|V move r -> r+1, so
  at step s a rank holds the block that started on rank (r - s) mod W;
* causal: step 0 is the diagonal block (masked), steps 1..r are full blocks,
  later steps are skipped but still forwarded;
* the out/lse merge of each step is fused into the attention kernel's epilogue;
* backward uses the global out/lse; dK|dV travel with their block in fp32 and
  make W hops; dQ stays local in fp32.

K and V travel as ONE message, posted before the step's kernel is launched so
the NCCL transfer overlaps the attention of the current block.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

import os

from . import _lib, local_attn, zigzag
from .local_attn import check_unsupported_kwargs

__all__ = [
    "RingComm", "ring_flash_attn_forward", "ring_flash_attn_backward", "RingFlashAttnFunc",
    "ring_flash_attn_func", "ring_flash_attn_kvpacked_func", "ring_flash_attn_qkvpacked_func",
]


class RingComm:
    """Ring neighbour exchange: send to (r+1) % W, receive from (r-1) % W.

    Same surface as sp_aurora/utils.py:172 IntelRingComm (`send_recv`, `commit`,
    `wait`, `send_recv_kv`). All transfers queued by `send_recv` go out as one
    batched NCCL group at `commit()`; no even/odd ordering is needed."""

    # Measurement aid: when True, exchanges are replaced by a local hand-off of
    # the send buffer (results are wrong, kernel work and launch order are
    # unchanged), which gives the compute-only time of a step.
    FAKE = False

    def __init__(self, process_group: Optional[dist.ProcessGroup] = None):
        self._process_group = process_group
        self._ops: List[dist.P2POp] = []
        self._reqs = None
        if dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank(process_group)
            self.world_size = dist.get_world_size(process_group)
        else:  # single process, no process group: plain local attention
            self.rank, self.world_size = 0, 1
        self.send_rank = (self.rank + 1) % self.world_size
        self.recv_rank = (self.rank - 1) % self.world_size
        if process_group is not None:
            self.send_rank = dist.get_global_rank(process_group, self.send_rank)
            self.recv_rank = dist.get_global_rank(process_group, self.recv_rank)

    def send_recv(self, to_send: torch.Tensor, recv_tensor: Optional[torch.Tensor] = None):
        if not to_send.is_contiguous():
            raise ValueError("RingComm.send_recv needs a contiguous tensor")
        res = torch.empty_like(to_send) if recv_tensor is None else recv_tensor
        if RingComm.FAKE:
            return to_send
        self._ops.append(dist.P2POp(dist.isend, to_send, self.send_rank, group=self._process_group))
        self._ops.append(dist.P2POp(dist.irecv, res, self.recv_rank, group=self._process_group))
        return res

    def commit(self):
        if self._reqs is not None:
            raise RuntimeError("commit called twice")
        self._reqs = dist.batch_isend_irecv(self._ops) if self._ops else []

    def wait(self):
        if self._reqs is None:
            raise RuntimeError("wait called before commit")
        for req in self._reqs:
            req.wait()
        self._reqs = None
        self._ops = []

    def send_recv_kv(self, k: torch.Tensor, v: torch.Tensor,
                     k_buffer: Optional[torch.Tensor] = None,
                     v_buffer: Optional[torch.Tensor] = None):
        next_k = self.send_recv(k.contiguous(), k_buffer)
        next_v = self.send_recv(v.contiguous(), v_buffer)
        self.commit()
        return next_k, next_v


def _pack_kv(k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """Return (message, axis): one contiguous tensor holding K and V, and the
    axis along which they sit. kv-packed views ([B,S,2,H,D] storage) are used in
    place; separate tensors are stacked once into [2,B,S,H,D]."""
    B, S, H, D = k.shape
    elt = k.element_size()
    packed_strides = (S * 2 * H * D, 2 * H * D, D, 1)
    if (k.stride() == packed_strides and v.stride() == packed_strides
            and v.data_ptr() == k.data_ptr() + H * D * elt
            and k.untyped_storage().data_ptr() == v.untyped_storage().data_ptr()):
        msg = torch.as_strided(k, (B, S, 2, H, D), (S * 2 * H * D, 2 * H * D, H * D, D, 1))
        return msg, 2
    return torch.stack((k, v)), 0


def _split_kv(msg: torch.Tensor, axis: int):
    return msg.select(axis, 0), msg.select(axis, 1)


def ring_flash_attn_forward(process_group, q, k, v, softmax_scale: float, causal: bool = True,
                            fwd_step: Callable = local_attn.attn_fwd_step):
    """W-step forward ring. Returns (out [B,S,Hq,D] q.dtype, lse [B,Hq,S] fp32).
    Counterpart of sp_aurora/intel_ring_flash_attn.py:17 intel_ring_flash_attn_forward.
    `fwd_step` is the per-block kernel call (tests substitute a CPU checker to
    exercise the schedule over gloo)."""
    comm = RingComm(process_group)
    W, r = comm.world_size, comm.rank
    B, S, Hq, D = q.shape
    out = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    last_step = r if causal else W - 1
    out_acc = None
    if last_step > 0:
        out_acc = torch.empty((B, S, Hq, D), dtype=torch.float32, device=q.device)
    if W == 1:
        fwd_step(q, k, v, softmax_scale, causal, lse, out=out)
        return out, lse

    cur, axis = _pack_kv(k, v)
    bufs = [torch.empty_like(cur), torch.empty_like(cur)]
    computed = 0
    for step in range(W):
        nxt = None
        if step + 1 != W:
            nxt = comm.send_recv(cur, bufs[step % 2])
            comm.commit()
        if (not causal) or step <= r:
            kc, vc = (k, v) if step == 0 else _split_kv(cur, axis)
            is_first, is_last = computed == 0, step == last_step
            fwd_step(q, kc, vc, softmax_scale, causal and step == 0, lse,
                     out=out if is_last else None,
                     out_acc=None if (is_first and is_last) else out_acc,
                     merge_prev=not is_first)
            computed += 1
        if nxt is not None:
            comm.wait()
            cur = nxt
    return out, lse


def ring_flash_attn_backward(process_group, dout, q, k, v, out, softmax_lse, softmax_scale: float,
                             causal: bool = True,
                             bwd_step: Callable = local_attn.attn_bwd_step,
                             delta_fn: Callable = local_attn.bwd_delta,
                             cast_fn: Callable = local_attn.cast_from_f32,
                             deterministic: bool = False):
    """W-step backward ring. Returns (dq, dk, dv) in q.dtype.
    Counterpart of sp_aurora/intel_ring_flash_attn.py:153; algorithm of
    sp_aurora/ring_flash_attn.py:70-154 (global out/lse, dK|dV ring of W hops).

    Each step runs the dQ pass first and the dK/dV pass second: the travelling dK|dV
    partial of the current block is still in flight during the dQ pass, and the dK/dV
    pass then adds straight into the received buffer (no separate fold), which is sent on."""
    kv_comm = RingComm(process_group)
    d_kv_comm = RingComm(process_group)
    W, r = kv_comm.world_size, kv_comm.rank
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    delta = delta_fn(out, dout)
    dq = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
    DQ, DKV = _lib.SPA_BWD_DQ_ONLY, _lib.SPA_BWD_DKV_ONLY

    if W == 1:
        dk = torch.empty((B, S, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty_like(dk)
        bwd_step(q, k, v, dout, softmax_lse, delta, softmax_scale, causal, None, None, None,
                 dq=dq, dq_overwrite=True, deterministic=deterministic, passes=DQ)
        bwd_step(q, k, v, dout, softmax_lse, delta, softmax_scale, causal, None, dk, dv,
                 deterministic=deterministic, passes=DKV)
        return dq, dk, dv

    dq_acc = torch.empty((B, S, Hq, D), dtype=torch.float32, device=q.device)
    last_step = r if causal else W - 1
    cur, axis = _pack_kv(k, v)
    kv_bufs = [torch.empty_like(cur), torch.empty_like(cur)]
    # fp32 travelling partials, K|V gradients as one message [2,B,S,Hkv,D]
    dkv_bufs = [torch.empty((2, B, S, Hkv, D), dtype=torch.float32, device=q.device)
                for _ in range(2)]
    for step in range(W):
        nxt = None
        if step + 1 != W:
            nxt = kv_comm.send_recv(cur, kv_bufs[step % 2])
            kv_comm.commit()
        computed = step <= r or not causal
        kc, vc = (k, v) if step == 0 else _split_kv(cur, axis)
        if computed:
            bwd_step(q, kc, vc, dout, softmax_lse, delta, softmax_scale, causal and step == 0,
                     dq_acc if last_step > 0 else None, None, None,
                     dq=dq if step == last_step else None, dq_overwrite=step == 0,
                     deterministic=deterministic, passes=DQ)
        tgt = dkv_bufs[step % 2]
        if step > 0:
            d_kv_comm.wait()           # the partial that travels with this block has arrived in tgt
        if computed:
            bwd_step(q, kc, vc, dout, softmax_lse, delta, softmax_scale, causal and step == 0,
                     None, tgt[0], tgt[1], dkv_accumulate=step > 0,
                     deterministic=deterministic, passes=DKV)
        if nxt is not None:
            kv_comm.wait()
            cur = nxt
        if step + 1 != W:
            d_kv_comm.send_recv(tgt, dkv_bufs[(step + 1) % 2])
            d_kv_comm.commit()
    # The block now here has every rank's share: it goes home in the element type (the rounding
    # its owner would apply, half the bytes of the fp32 partial).
    done = dkv_bufs[(W - 1) % 2]
    if q.dtype != torch.float32:
        done = cast_fn(done.view(2 * B, S, Hkv, D), q.dtype).view(2, B, S, Hkv, D)
    home = d_kv_comm.send_recv(done)
    d_kv_comm.commit()
    d_kv_comm.wait()
    return dq, home[0], home[1]


def _use_zigzag(group, q, causal) -> bool:
    """Causal rings of more than one rank run on the internally re-balanced
    (zigzag) layout; SPA_RING_ZIGZAG=0 keeps the plain contiguous schedule."""
    if not causal or not (dist.is_available() and dist.is_initialized()):
        return False
    if dist.get_world_size(group) == 1 or q.shape[1] % 2:
        return False
    return os.environ.get("SPA_RING_ZIGZAG", "1") != "0"


class RingFlashAttnFunc(torch.autograd.Function):
    """Counterpart of sp_aurora/intel_ring_flash_attn.py:274 IntelRingFlashAttnFunc."""

    @staticmethod
    def forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                deterministic, return_softmax, group):
        check_unsupported_kwargs(dropout_p, window_size, alibi_slopes)
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        local_attn.check_qkv(q, k, v)
        ctx.zigzag = _use_zigzag(group, q, causal)
        if ctx.zigzag:
            out, lse, saved = zigzag.zigzag_ring_forward(group, q, k, v, softmax_scale,
                                                         need_lse=bool(return_softmax))
            ctx.save_for_backward(*saved)
        else:
            out, lse = ring_flash_attn_forward(group, q, k, v, softmax_scale, causal)
            ctx.save_for_backward(q, k, v, out, lse)
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal
        ctx.group = group
        ctx.deterministic = bool(deterministic)
        return out if not return_softmax else (out, lse, None)

    @staticmethod
    def backward(ctx, dout, *args):
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        if ctx.zigzag:
            q_z, kv_z, out_z, lse_z = ctx.saved_tensors
            dq, dk, dv = zigzag.zigzag_ring_backward(ctx.group, dout, q_z, kv_z, out_z, lse_z,
                                                     ctx.softmax_scale,
                                                     deterministic=ctx.deterministic)
            _lib.maybe_check_status()
            return dq, dk, dv, None, None, None, None, None, None, None, None
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = ring_flash_attn_backward(ctx.group, dout, q, k, v, out, lse,
                                              ctx.softmax_scale, ctx.causal,
                                              deterministic=ctx.deterministic)
        _lib.maybe_check_status()
        return dq, dk, dv, None, None, None, None, None, None, None, None


def ring_flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                         window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                         return_attn_probs=False, group=None):
    """q,k,v: [B, S_local, H, D] (rank r of `group` holds sequence chunk r).
    Returns out, or (out, lse [B,Hq,S_local] fp32, None) with return_attn_probs.
    Counterpart of sp_aurora/intel_ring_flash_attn.py:399."""
    return RingFlashAttnFunc.apply(q, k, v, dropout_p, softmax_scale, causal, window_size,
                                   alibi_slopes, deterministic, return_attn_probs, group)


def ring_flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False,
                                  window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                  return_attn_probs=False, group=None):
    """kv: [B, S_local, 2, Hkv, D]. Counterpart of
    sp_aurora/intel_ring_flash_attn.py:371."""
    if kv.dim() != 5 or kv.shape[2] != 2:
        raise ValueError(f"kv must be [B, S, 2, H, D], got {tuple(kv.shape)}")
    return RingFlashAttnFunc.apply(q, kv[:, :, 0], kv[:, :, 1], dropout_p, softmax_scale, causal,
                                   window_size, alibi_slopes, deterministic, return_attn_probs,
                                   group)


def ring_flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False,
                                   window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                   return_attn_probs=False, group=None):
    """qkv: [B, S_local, 3, H, D]. Counterpart of
    sp_aurora/intel_ring_flash_attn.py:344."""
    if qkv.dim() != 5 or qkv.shape[2] != 3:
        raise ValueError(f"qkv must be [B, S, 3, H, D], got {tuple(qkv.shape)}")
    return RingFlashAttnFunc.apply(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], dropout_p,
                                   softmax_scale, causal, window_size, alibi_slopes, deterministic,
                                   return_attn_probs, group)
