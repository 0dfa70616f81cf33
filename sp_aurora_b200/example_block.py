"""A transformer attention block on top of the sequence-parallel attention functions:
QKV projection -> attention over the sharded sequence -> output projection.

The shape of the reference's example model (examples/example_mpi_integration.py:38-86,
`RingAttentionModel`: q/k/v/out projections around `ring_flash_attn_func`), with two changes
that the kernels make free: ONE projection GEMM writes a `[B, S_local, Hq + 2*Hkv, D]` buffer
whose head slices ARE q, k and v (the attention kernels and the packed all-to-all read strided
views in place, so there is no split or transpose copy), and grouped-query attention
(`n_kv_heads < nheads`) is supported. The projections are plain `torch.nn.Linear` (library
GEMMs); everything between them runs in this package's kernels. With `rope_base` set, q and k
(adjacent head slices of the projection output) are rotated together by one `apply_rope` call,
positions offset by the rank's first token.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .hybrid import LongContextAttention
from .ring import ring_flash_attn_func
from .rope import apply_rope, rope_tables
from .ulysses import ulysses_flash_attn_func

__all__ = ["SequenceParallelAttentionBlock"]


class SequenceParallelAttentionBlock(torch.nn.Module):
    """x [B, S_local, d_model] -> [B, S_local, d_model]; rank r of `group` holds sequence chunk r.

    mode: "ring" (ring_flash_attn_func), "ulysses" (ulysses_flash_attn_func) or "hybrid"
    (LongContextAttention over the groups of set_seq_parallel_pg)."""

    def __init__(self, d_model: int, nheads: int, n_kv_heads: Optional[int] = None,
                 mode: str = "ring", group: Optional[dist.ProcessGroup] = None,
                 dtype: torch.dtype = torch.bfloat16, device=None, rope_base: Optional[float] = None):
        super().__init__()
        if d_model % nheads:
            raise ValueError(f"d_model ({d_model}) must be a multiple of nheads ({nheads})")
        n_kv_heads = n_kv_heads or nheads
        if nheads % n_kv_heads:
            raise ValueError(f"nheads ({nheads}) must be a multiple of n_kv_heads ({n_kv_heads})")
        if mode not in ("ring", "ulysses", "hybrid"):
            raise ValueError(f"unknown mode '{mode}'")
        self.nheads, self.n_kv_heads, self.head_dim = nheads, n_kv_heads, d_model // nheads
        self.mode, self.group = mode, group
        self.qkv_proj = torch.nn.Linear(d_model, (nheads + 2 * n_kv_heads) * self.head_dim, bias=False,
                                        dtype=dtype, device=device)
        self.out_proj = torch.nn.Linear(d_model, d_model, bias=False, dtype=dtype, device=device)
        self.hybrid = LongContextAttention() if mode == "hybrid" else None
        self.rope_base = rope_base
        self._rope = None            # (positions, device) -> tables, built on first use

    def _rope_tables(self, S_local: int, device):
        live = dist.is_available() and dist.is_initialized()
        group = None if self.mode == "hybrid" else self.group      # hybrid shards over all ranks
        world = dist.get_world_size(group) if live else 1
        rank = dist.get_rank(group) if live else 0
        key = (world * S_local, device)
        if self._rope is None or self._rope[0] != key:
            self._rope = (key, rope_tables(world * S_local, self.head_dim, self.rope_base, device))
        return self._rope[1], rank * S_local

    def forward(self, x: torch.Tensor, causal: bool = True) -> torch.Tensor:
        B, S, _ = x.shape
        hq, hkv = self.nheads, self.n_kv_heads
        qkv = self.qkv_proj(x).view(B, S, hq + 2 * hkv, self.head_dim)
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
        if self.rope_base is not None:
            (cos, sin), offset = self._rope_tables(S, x.device)
            qk = apply_rope(qkv[:, :, :hq + hkv], cos, sin, pos_offset=offset)   # one pass for q and k
            q, k = qk[:, :, :hq], qk[:, :, hq:]
        if self.mode == "ring":
            out = ring_flash_attn_func(q, k, v, causal=causal, group=self.group)
        elif self.mode == "ulysses":
            out = ulysses_flash_attn_func(q, k, v, causal=causal, group=self.group)
        else:
            out = self.hybrid(q, k, v, causal=causal)
        return self.out_proj(out.reshape(B, S, hq * self.head_dim))
