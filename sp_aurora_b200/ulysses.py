"""Ulysses sequence-parallel attention: all-to-all (sequence -> heads), local
attention over the full sequence on H/P heads, all-to-all back.

Mirrors sp_aurora/intel_ulysses_attn.py (forward :184, backward :290, autograd
function :436, public functions :501/:549/:587) and the module
sp_aurora/ulysses/attn_layer.py:129 UlyssesAttention (+ AttnType :20).
Differences kept on purpose: lse IS resharded back and returned
(`(out, lse, None)` with return_attn_probs; the reference returns `(out, None)`,
sp_aurora/intel_ulysses_attn.py:478), and backward reuses the resharded q/k/v/out
saved by forward instead of re-communicating them (:376-379).
"""
from __future__ import annotations

from enum import Enum
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib, local_attn
from .all_to_all import (SeqAllToAll4D, all_to_all_4D, heads_all_to_all_packed, reshard_lse,
                         seq_all_to_all_packed)
from .local_attn import check_unsupported_kwargs

__all__ = [
    "ulysses_flash_attn_forward", "ulysses_flash_attn_backward", "UlyssesFlashAttnFunc",
    "ulysses_flash_attn_func", "ulysses_flash_attn_kvpacked_func",
    "ulysses_flash_attn_qkvpacked_func", "UlyssesAttention", "AttnType", "UlyssesComm",
    "select_flash_attn_impl",
]


def _group_size(group) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


def ulysses_flash_attn_forward(process_group, q, k, v, softmax_scale: float, causal: bool = False):
    """Returns (out [B,S_loc,Hq,D], lse [B,Hq,S_loc], saved) where `saved` holds
    the head-sharded q, k, v, out, lse for backward. q, k and v travel as one
    all-to-all message (the reference sends three, sp_aurora/intel_ulysses_attn.py:156-170)
    and are read by the attention kernel where they land."""
    P = _group_size(process_group)
    if P > 1 and (q.shape[2] % P or k.shape[2] % P):
        raise ValueError(
            f"q heads ({q.shape[2]}) and kv heads ({k.shape[2]}) must be divisible by the "
            f"Ulysses group size ({P})")
    q_r, k_r, v_r = heads_all_to_all_packed((q, k, v), group=process_group)
    out_r, lse_r = local_attn.flash_attn_forward(q_r, k_r, v_r, softmax_scale, causal)
    out = all_to_all_4D(out_r, 1, 2, group=process_group)
    lse = reshard_lse(lse_r, process_group)
    return out, lse, (q_r, k_r, v_r, out_r, lse_r)


def ulysses_flash_attn_backward(process_group, dout, q_r, k_r, v_r, out_r, lse_r,
                                softmax_scale: float, causal: bool = False):
    """Returns (dq, dk, dv) sharded on sequence like the inputs of forward. The three
    gradients are written by the kernels into one [B, S, hq+2*hkv, D] buffer and go back
    as one all-to-all message."""
    dout_r = all_to_all_4D(dout, 2, 1, group=process_group)
    B, S, hq, D = q_r.shape
    hkv = k_r.shape[2]
    grads = torch.empty((B, S, hq + 2 * hkv, D), dtype=q_r.dtype, device=q_r.device)
    dq_r, dk_r, dv_r = grads[:, :, :hq], grads[:, :, hq:hq + hkv], grads[:, :, hq + hkv:]
    local_attn.flash_attn_backward(dout_r, q_r, k_r, v_r, out_r, lse_r, softmax_scale, causal,
                                   dq=dq_r, dk=dk_r, dv=dv_r)
    dq, dk, dv = seq_all_to_all_packed((dq_r, dk_r, dv_r), group=process_group)
    return dq, dk, dv


class UlyssesFlashAttnFunc(torch.autograd.Function):
    """Counterpart of sp_aurora/intel_ulysses_attn.py:436 IntelUlyssesFlashAttnFunc."""

    @staticmethod
    def forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                deterministic, return_softmax, group):
        check_unsupported_kwargs(dropout_p, window_size, alibi_slopes)
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        local_attn.check_qkv(q, k, v)
        out, lse, saved = ulysses_flash_attn_forward(group, q, k, v, softmax_scale, causal)
        ctx.save_for_backward(*saved)
        ctx.softmax_scale, ctx.causal, ctx.group = softmax_scale, causal, group
        return out if not return_softmax else (out, lse, None)

    @staticmethod
    def backward(ctx, dout, *args):
        q_r, k_r, v_r, out_r, lse_r = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dq, dk, dv = ulysses_flash_attn_backward(ctx.group, dout, q_r, k_r, v_r, out_r, lse_r,
                                                 ctx.softmax_scale, ctx.causal)
        _lib.maybe_check_status()
        return dq, dk, dv, None, None, None, None, None, None, None, None


def ulysses_flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                            window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                            return_attn_probs=False, group=None):
    """q,k,v: [B, S_local, H, D]. Counterpart of sp_aurora/intel_ulysses_attn.py:501."""
    return UlyssesFlashAttnFunc.apply(q, k, v, dropout_p, softmax_scale, causal, window_size,
                                      alibi_slopes, deterministic, return_attn_probs, group)


def ulysses_flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False,
                                     window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                     return_attn_probs=False, group=None):
    """kv: [B, S_local, 2, Hkv, D]. Counterpart of sp_aurora/intel_ulysses_attn.py:587."""
    if kv.dim() != 5 or kv.shape[2] != 2:
        raise ValueError(f"kv must be [B, S, 2, H, D], got {tuple(kv.shape)}")
    return UlyssesFlashAttnFunc.apply(q, kv[:, :, 0], kv[:, :, 1], dropout_p, softmax_scale,
                                      causal, window_size, alibi_slopes, deterministic,
                                      return_attn_probs, group)


def ulysses_flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False,
                                      window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                      return_attn_probs=False, group=None):
    """qkv: [B, S_local, 3, H, D]. Counterpart of sp_aurora/intel_ulysses_attn.py:549."""
    if qkv.dim() != 5 or qkv.shape[2] != 3:
        raise ValueError(f"qkv must be [B, S, 3, H, D], got {tuple(qkv.shape)}")
    return UlyssesFlashAttnFunc.apply(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], dropout_p,
                                      softmax_scale, causal, window_size, alibi_slopes,
                                      deterministic, return_attn_probs, group)


class AttnType(str, Enum):
    """Attention backend names of sp_aurora/ulysses/attn_layer.py:20-31 (a str enum with
    the same members and values). Every value runs the same sm_100a kernels: there is no
    backend selection here, the argument is accepted and ignored. The yunchang spellings
    ("fa", "fa3", "sage_*", "sparse_sage") are accepted as aliases of FA."""
    TORCH = "torch"
    INTEL_SYCL = "intel_sycl"
    INTEL_ONEDNN = "intel_onednn"
    FA = "flash_attn"
    FA3 = "flash_attn_3"

    @classmethod
    def _missing_(cls, value):
        aliases = {"fa": cls.FA, "fa3": cls.FA3, "sage_auto": cls.FA, "sage_fp16": cls.FA,
                   "sage_fp8": cls.FA, "sparse_sage": cls.FA}
        if isinstance(value, str) and value.lower() in aliases:
            return aliases[value.lower()]
        return None

    @classmethod
    def from_string(cls, s: str):
        return cls(s)


def select_flash_attn_impl(attn_type: "AttnType" = AttnType.FA):
    """Counterpart of sp_aurora/ulysses/attn_layer.py:34 select_flash_attn_impl: returns
    the local attention function `fn(q, k, v, dropout_p=0.0, softmax_scale=None,
    causal=False, window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
    deterministic=False, return_attn_probs=False)` on [B, S, H, D] tensors. Every
    `attn_type` selects the same sm_100a kernels; with return_attn_probs the second
    result is lse [B, H, S] fp32."""
    AttnType(attn_type)   # raises ValueError on an unknown name, like the enum lookup would

    def attn_fn(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
        check_unsupported_kwargs(dropout_p, window_size, alibi_slopes, softcap)
        out, lse = local_attn.LocalFlashAttnFunc.apply(q, k, v, softmax_scale, causal)
        return (out, lse) if return_attn_probs else out

    return attn_fn


class UlyssesComm:
    """Counterpart of sp_aurora/intel_ulysses_attn.py:146 IntelUlyssesComm: the two
    reshards of Ulysses attention as methods (autograd-aware)."""

    def __init__(self, process_group: Optional[dist.ProcessGroup] = None):
        self.process_group = process_group
        live = dist.is_available() and dist.is_initialized()
        self.world_size = dist.get_world_size(process_group) if live else 1
        self.rank = dist.get_rank(process_group) if live else 0

    def all_to_all_qkv(self, q, k, v, scatter_idx: int = 2, gather_idx: int = 1):
        return tuple(SeqAllToAll4D.apply(self.process_group, t, scatter_idx, gather_idx)
                     for t in (q, k, v))

    def all_to_all_output(self, output, scatter_idx: int = 1, gather_idx: int = 2):
        return SeqAllToAll4D.apply(self.process_group, output, scatter_idx, gather_idx)


class UlyssesAttention(torch.nn.Module):
    """Module form; counterpart of sp_aurora/ulysses/attn_layer.py:129.

    forward(query, key, value) with [B, S_local, H, D] shards; gradients flow
    through the autograd-aware all-to-all and the local attention function."""

    def __init__(self, sequence_process_group: Optional[dist.ProcessGroup] = None,
                 scatter_idx: int = 2, gather_idx: int = 1, use_sync: bool = False,
                 attn_type: AttnType = AttnType.FA) -> None:
        super().__init__()
        self.spg = sequence_process_group
        self.scatter_idx = scatter_idx
        self.gather_idx = gather_idx
        self.use_sync = use_sync
        self.attn_type = AttnType(attn_type)   # any reference or yunchang spelling; ignored

    def forward(self, query, key, value, dropout_p=0.0, softmax_scale=None, causal=False,
                window_size=(-1, -1), softcap=0.0, alibi_slopes=None, deterministic=False,
                return_attn_probs=False, *args):
        check_unsupported_kwargs(dropout_p, window_size, alibi_slopes, softcap)
        out = UlyssesFlashAttnFunc.apply(query, key, value, dropout_p, softmax_scale, causal,
                                         window_size, alibi_slopes, deterministic,
                                         return_attn_probs, self.spg)
        return out
