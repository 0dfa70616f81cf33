"""Adapters that put the sequence-parallel attention behind other libraries' hooks."""
from .hf_adapter import (  # noqa: F401
    substitute_hf_flash_attn,
    update_ring_flash_attn_params,
    update_sp_aurora_params,
    use_ring_attn,
)
