"""Hugging Face transformers hook: flash-attention calls go through the sequence-parallel path.

Counterpart of sp_aurora/adapters/hf_adapter.py (update_ring_flash_attn_params :34,
use_ring_attn :57, create_ring_flash_attention_forward :62, flash_attention_forward :285,
substitute_hf_flash_attn :353), which cannot be imported in the reference because the varlen
function it builds on is missing there. Usage is the same:

    substitute_hf_flash_attn(process_group, heads_k_stride=1)      # once, after init_process_group
    update_ring_flash_attn_params(cu_seqlens, process_group)       # per batch: global cu_seqlens
    model(input_ids=local_chunk, position_ids=local_positions)     # attn_implementation="flash_attention_2"

Each rank feeds the model its contiguous 1/W of the packed token stream (batch size 1); the
attention layers then run `llama3_flash_attn_varlen_func` (all-gather K/V by kv-head groups, one
kernel call per sequence segment). Both hooks of transformers are covered: the function table
`ALL_ATTENTION_FUNCTIONS` used by current model code, and
`modeling_flash_attention_utils._flash_attention_forward`, whatever its signature in the installed
version (arguments are bound by name, not by position lists per version).
transformers is imported only when a hook is installed.
"""
from __future__ import annotations

import functools
import inspect
from typing import Optional

import torch
import torch.distributed as dist

from ..llama3_varlen import llama3_flash_attn_prepare_cu_seqlens, llama3_flash_attn_varlen_func

DATA_PARAMS: dict = {}
RING_ATTN_SWITCH = True


def update_ring_flash_attn_params(cu_seqlens: torch.Tensor, process_group=None) -> None:
    """Set the packed batch's global `cu_seqlens` (int [n_seq + 1], 0 .. total tokens) for the
    attention calls that follow on this rank."""
    world = dist.get_world_size(process_group) if dist.is_initialized() else 1
    rank = dist.get_rank(process_group) if dist.is_initialized() else 0
    cq, ck, mq, mk, ks = llama3_flash_attn_prepare_cu_seqlens(cu_seqlens, True, rank, world)
    DATA_PARAMS.update(cu_seqlens_q=cq, cu_seqlens_k=ck, max_seqlen_q=mq, max_seqlen_k=mk,
                       local_k_slice=ks)


update_sp_aurora_params = update_ring_flash_attn_params     # the name sp_aurora/__init__.py:81 exports


def use_ring_attn(flag: bool) -> None:
    """Switch the substituted hooks between the sequence-parallel path and the original."""
    global RING_ATTN_SWITCH
    RING_ATTN_SWITCH = bool(flag)


def _ring_attention(query, key, value, *, process_group, heads_k_stride, is_causal=True, dropout=0.0,
                    softmax_scale=None, sliding_window=None, softcap=None, deterministic=None):
    """query/key/value [1, S_local, H, D] -> [1, S_local, Hq, D]."""
    if not DATA_PARAMS:
        raise RuntimeError("call update_ring_flash_attn_params(cu_seqlens, group) before the model")
    if query.size(0) != 1:
        raise ValueError("varlen data should be packed into batch size 1 in advance")
    if not is_causal:
        raise NotImplementedError("only causal attention is supported by the packed-stream path")
    if dropout:
        raise NotImplementedError("attention dropout is not supported")
    if softcap:
        raise NotImplementedError("softcap is not supported")
    if sliding_window is not None and sliding_window < DATA_PARAMS["max_seqlen_k"]:
        raise NotImplementedError("sliding-window attention shorter than the sequences is not supported")
    out = llama3_flash_attn_varlen_func(
        query.squeeze(0), key.squeeze(0), value.squeeze(0),
        cu_seqlens_q=DATA_PARAMS["cu_seqlens_q"], cu_seqlens_k=DATA_PARAMS["cu_seqlens_k"],
        max_seqlen_q=DATA_PARAMS["max_seqlen_q"], max_seqlen_k=DATA_PARAMS["max_seqlen_k"],
        heads_k_stride=heads_k_stride, local_k_slice=DATA_PARAMS["local_k_slice"],
        softmax_scale=softmax_scale, causal=True, deterministic=bool(deterministic),
        group=process_group)
    return out.unsqueeze(0)


def create_ring_flash_attention_forward(process_group, heads_k_stride: int, like=None):
    """A replacement for transformers' `_flash_attention_forward` with the same signature as
    `like` (default: a (query_states, key_states, value_states, attention_mask, query_length,
    is_causal, dropout, position_ids, softmax_scale, sliding_window, use_top_left_mask, softcap,
    deterministic, **kwargs) function). Arguments this path has no use for (attention_mask,
    position_ids, cu_seq_lens_*, target_dtype, ...) are accepted and ignored: the segment tables
    come from update_ring_flash_attn_params."""

    def ring_forward(query_states, key_states, value_states, attention_mask=None, query_length=None,
                     is_causal=True, dropout=0.0, position_ids=None, softmax_scale=None,
                     sliding_window=None, use_top_left_mask=False, softcap=None, deterministic=None,
                     **kwargs):
        causal = is_causal and not (use_top_left_mask and query_length == 1)
        return _ring_attention(query_states, key_states, value_states, process_group=process_group,
                               heads_k_stride=heads_k_stride, is_causal=causal, dropout=dropout,
                               softmax_scale=softmax_scale, sliding_window=sliding_window,
                               softcap=softcap, deterministic=deterministic)

    if like is None:
        return ring_forward
    sig = inspect.signature(like)

    @functools.wraps(like)
    def bound_forward(*args, **kwargs):
        ba = sig.bind(*args, **kwargs)
        named = {k: v for k, v in ba.arguments.items()
                 if sig.parameters[k].kind not in (inspect.Parameter.VAR_KEYWORD,
                                                   inspect.Parameter.VAR_POSITIONAL)}
        return ring_forward(**named)

    return bound_forward


def flash_attention_forward(module, query, key, value, attention_mask=None, dropout: float = 0.0,
                            scaling: Optional[float] = None, sliding_window: Optional[int] = None,
                            softcap: Optional[float] = None, *, process_group=None,
                            heads_k_stride: int = 1, **kwargs):
    """Entry of transformers' attention-function table: query/key/value [B, H, S, D] (as the
    model's attention layer holds them), returns (attn_output [B, S, Hq, D], None). The
    transposes are views: the kernels read [B, S, H, D] tensors with any head / sequence
    strides. fp32 activations under autocast are run in the autocast dtype, as transformers'
    own flash path does."""
    q, k, v = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    original = q.dtype
    if q.dtype == torch.float32 and torch.is_autocast_enabled():
        target = torch.get_autocast_gpu_dtype()
        q, k, v = q.to(target), k.to(target), v.to(target)
    kwargs.pop("is_causal", None)
    out = _ring_attention(q, k, v, process_group=process_group, heads_k_stride=heads_k_stride,
                          is_causal=getattr(module, "is_causal", True), dropout=dropout,
                          softmax_scale=scaling, sliding_window=sliding_window, softcap=softcap,
                          deterministic=kwargs.get("deterministic"))
    return out.to(original), None


def substitute_hf_flash_attn(process_group, heads_k_stride: int = 1) -> None:
    """Route transformers' flash-attention implementation through the sequence-parallel path
    (`use_ring_attn(False)` switches back without undoing the substitution)."""
    try:
        import transformers
        import transformers.modeling_flash_attention_utils as fa_utils
    except ImportError as exc:        # pragma: no cover - transformers is optional
        raise ValueError("transformers is not installed") from exc
    old = getattr(fa_utils, "_flash_attention_forward", None)
    if old is None:
        raise ValueError(f"The current transformer version {transformers.__version__} is not supported: "
                         "modeling_flash_attention_utils._flash_attention_forward is missing")
    if not getattr(old, "_sp_aurora_substituted", False):
        new = create_ring_flash_attention_forward(process_group, heads_k_stride, like=old)

        @functools.wraps(old)
        def switched(*args, **kwargs):
            return (new if RING_ATTN_SWITCH else old)(*args, **kwargs)

        switched._sp_aurora_substituted = True
        fa_utils._flash_attention_forward = switched
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    except ImportError:
        ALL_ATTENTION_FUNCTIONS = None
    if ALL_ATTENTION_FUNCTIONS is not None:
        try:
            previous = ALL_ATTENTION_FUNCTIONS["flash_attention_2"]
        except KeyError:
            previous = None

        def table_entry(module, query, key, value, attention_mask=None, **kwargs):
            if RING_ATTN_SWITCH or previous is None:
                return flash_attention_forward(module, query, key, value, attention_mask,
                                               process_group=process_group,
                                               heads_k_stride=heads_k_stride, **kwargs)
            return previous(module, query, key, value, attention_mask, **kwargs)

        ALL_ATTENTION_FUNCTIONS["flash_attention_2"] = table_entry
        ALL_ATTENTION_FUNCTIONS["sp_aurora"] = table_entry
