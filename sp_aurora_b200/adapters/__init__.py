"""Adapters that put the sequence-parallel attention behind other libraries' hooks.

`hf_adapter` routes Hugging Face transformers' flash-attention calls (both the attention-function
table of current model code and the older `_flash_attention_forward` hook) through the
packed-stream varlen path of `llama3_varlen`. Nothing here imports transformers until a hook is
installed.
"""
from . import hf_adapter

substitute_hf_flash_attn = hf_adapter.substitute_hf_flash_attn
update_ring_flash_attn_params = hf_adapter.update_ring_flash_attn_params
update_sp_aurora_params = hf_adapter.update_sp_aurora_params
use_ring_attn = hf_adapter.use_ring_attn

__all__ = ["hf_adapter", "substitute_hf_flash_attn", "update_ring_flash_attn_params",
           "update_sp_aurora_params", "use_ring_attn"]
