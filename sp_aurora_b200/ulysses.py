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

from . import local_attn
from .all_to_all import SeqAllToAll4D, all_to_all_4D, reshard_lse
from .local_attn import check_unsupported_kwargs

__all__ = [
    "ulysses_flash_attn_forward", "ulysses_flash_attn_backward", "UlyssesFlashAttnFunc",
    "ulysses_flash_attn_func", "ulysses_flash_attn_kvpacked_func",
    "ulysses_flash_attn_qkvpacked_func", "UlyssesAttention", "AttnType",
]


def _group_size(group) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


def ulysses_flash_attn_forward(process_group, q, k, v, softmax_scale: float, causal: bool = False):
    """Returns (out [B,S_loc,Hq,D], lse [B,Hq,S_loc], saved) where `saved` holds
    the head-sharded q, k, v, out, lse for backward."""
    P = _group_size(process_group)
    if P > 1 and (q.shape[2] % P or k.shape[2] % P):
        raise ValueError(
            f"q heads ({q.shape[2]}) and kv heads ({k.shape[2]}) must be divisible by the "
            f"Ulysses group size ({P})")
    q_r = all_to_all_4D(q, 2, 1, group=process_group)
    k_r = all_to_all_4D(k, 2, 1, group=process_group)
    v_r = all_to_all_4D(v, 2, 1, group=process_group)
    out_r, lse_r = local_attn.flash_attn_forward(q_r, k_r, v_r, softmax_scale, causal)
    out = all_to_all_4D(out_r, 1, 2, group=process_group)
    lse = reshard_lse(lse_r, process_group)
    return out, lse, (q_r, k_r, v_r, out_r, lse_r)


def ulysses_flash_attn_backward(process_group, dout, q_r, k_r, v_r, out_r, lse_r,
                                softmax_scale: float, causal: bool = False):
    """Returns (dq, dk, dv) sharded on sequence like the inputs of forward."""
    dout_r = all_to_all_4D(dout, 2, 1, group=process_group)
    dq_r, dk_r, dv_r = local_attn.flash_attn_backward(dout_r, q_r, k_r, v_r, out_r, lse_r,
                                                      softmax_scale, causal)
    dq = all_to_all_4D(dq_r, 1, 2, group=process_group)
    dk = all_to_all_4D(dk_r, 1, 2, group=process_group)
    dv = all_to_all_4D(dv_r, 1, 2, group=process_group)
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


class AttnType(Enum):
    """Accepted for signature compatibility with sp_aurora/ulysses/attn_layer.py:20;
    every value runs the same sm_100a kernels (there is no backend selection)."""
    FA = "fa"
    FA3 = "fa3"
    TORCH = "torch"
    SAGE_AUTO = "sage_auto"
    SAGE_FP16 = "sage_fp16"
    SAGE_FP8 = "sage_fp8"
    SPARSE_SAGE = "sparse_sage"

    @classmethod
    def from_string(cls, s: str):
        for member in cls:
            if member.value == s:
                return member
        raise ValueError(f"'{s}' is not a valid {cls.__name__}")


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
        self.attn_type = attn_type

    def forward(self, query, key, value, dropout_p=0.0, softmax_scale=None, causal=False,
                window_size=(-1, -1), softcap=0.0, alibi_slopes=None, deterministic=False,
                return_attn_probs=False, *args):
        check_unsupported_kwargs(dropout_p, window_size, alibi_slopes, softcap)
        out = UlyssesFlashAttnFunc.apply(query, key, value, dropout_p, softmax_scale, causal,
                                         window_size, alibi_slopes, deterministic,
                                         return_attn_probs, self.spg)
        return out
