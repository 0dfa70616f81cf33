"""Hybrid Ulysses x ring attention and the process-group singleton.

Mirrors sp_aurora/hybrid/long_ctx_attention.py:19 LongContextAttention and
sp_aurora/globals.py (ProcessGroupSingleton :13, PROCESS_GROUP :45,
set_seq_parallel_pg :48, destroy_seq_parallel_pg :154).

Group layout: Ulysses groups are CONSECUTIVE ranks and ring groups are strided
({i, i+U, i+2U, ...}). With rank-ordered contiguous sequence shards a Ulysses
all-to-all then gathers one contiguous span of the sequence per group, and the
ring's "rank j holds an earlier span than rank j+1" causal rule stays true. (The
reference builds the groups the other way round, sp_aurora/globals.py:102-124,
which interleaves chunks and breaks causal order.)
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
import torch.distributed as dist

from .all_to_all import HeadsAllToAllPacked, SeqAllToAll4D, SeqAllToAll5D, reshard_lse
from .local_attn import check_unsupported_kwargs
from .ring import ring_flash_attn_func, ring_flash_attn_qkvpacked_func
from .ulysses import AttnType

__all__ = ["ProcessGroupSingleton", "PROCESS_GROUP", "set_seq_parallel_pg",
           "destroy_seq_parallel_pg", "get_ulysses_pg", "get_ring_pg", "is_initialized",
           "seq_parallel_group_ranks", "LongContextAttention", "LongContextAttentionQKVPacked"]


class ProcessGroupSingleton:
    def __init__(self):
        self.ULYSSES_PG: Optional[dist.ProcessGroup] = None
        self.RING_PG: Optional[dist.ProcessGroup] = None
        self.initialized: bool = False
        self._ulysses_degree: int = 1
        self._ring_degree: int = 1
        self._rank: int = 0
        self._world_size: int = 1

    def __repr__(self):
        return (f"ProcessGroupSingleton(initialized={self.initialized}, "
                f"ulysses_degree={self._ulysses_degree}, ring_degree={self._ring_degree})")

    @property
    def ulysses_degree(self) -> int:
        return self._ulysses_degree

    @property
    def ring_degree(self) -> int:
        return self._ring_degree


PROCESS_GROUP = ProcessGroupSingleton()


def seq_parallel_group_ranks(sp_ulysses_degree: int, sp_ring_degree: int, world_size: int):
    """Rank lists of every Ulysses group and every ring group (pure function)."""
    if sp_ulysses_degree * sp_ring_degree != world_size:
        raise ValueError(
            f"Ulysses degree ({sp_ulysses_degree}) * Ring degree ({sp_ring_degree}) "
            f"must equal world size ({world_size})")
    U, R = sp_ulysses_degree, sp_ring_degree
    ulysses = [[j * U + i for i in range(U)] for j in range(R)]
    ring = [[i + j * U for j in range(R)] for i in range(U)]
    return ulysses, ring


def high_priority_nccl_options():
    """NCCL group options with high-priority streams, or None without the NCCL backend.

    The attention kernels keep every SM occupied, so a send/recv kernel of default priority is
    only scheduled once the attention kernel drains and the ring hop stops overlapping compute
    (measured on 4 B200s: 4.2 ms of dk|dv waits per cfg4 step at default priority, 0.01 ms with
    high-priority streams).  Pass the result as `pg_options` to `init_process_group` /
    `new_group`; `set_seq_parallel_pg` does so for the groups it creates.
    SPA_NCCL_HIGH_PRIORITY=0 makes this return None (default-priority streams)."""
    import os
    if os.environ.get("SPA_NCCL_HIGH_PRIORITY", "1") == "0":
        return None
    if not (dist.is_available() and dist.is_nccl_available()):
        return None
    return dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)


def _group_kwargs(backend: Optional[str]) -> dict:
    effective = backend or (dist.get_backend() if dist.is_initialized() else "nccl")
    if str(effective) == "nccl":
        opts = high_priority_nccl_options()
        if opts is not None:
            return {"pg_options": opts}
    return {}


def set_seq_parallel_pg(sp_ulysses_degree: int, sp_ring_degree: int, rank: int, world_size: int,
                        backend: Optional[str] = None) -> None:
    """Create the Ulysses and ring groups; same signature and errors as
    sp_aurora/globals.py:48 (backend defaults to the default group's, NCCL on GPUs)."""
    if PROCESS_GROUP.initialized:
        raise ValueError("Process groups already initialized")
    ulysses, ring = seq_parallel_group_ranks(sp_ulysses_degree, sp_ring_degree, world_size)
    if not dist.is_initialized():
        dist.init_process_group(backend=backend or "nccl", **_group_kwargs(backend))
    PROCESS_GROUP._ulysses_degree = sp_ulysses_degree
    PROCESS_GROUP._ring_degree = sp_ring_degree
    PROCESS_GROUP._rank = rank
    PROCESS_GROUP._world_size = world_size
    # new_group is collective over the default group: every rank creates every group.
    for ranks in ulysses:
        g = dist.new_group(ranks, backend=backend, **_group_kwargs(backend))
        if rank in ranks:
            PROCESS_GROUP.ULYSSES_PG = g
    for ranks in ring:
        g = dist.new_group(ranks, backend=backend, **_group_kwargs(backend))
        if rank in ranks:
            PROCESS_GROUP.RING_PG = g
    PROCESS_GROUP.initialized = True
    dist.barrier()


def get_ulysses_pg():
    return PROCESS_GROUP.ULYSSES_PG


def get_ring_pg():
    return PROCESS_GROUP.RING_PG


def is_initialized() -> bool:
    return PROCESS_GROUP.initialized


def destroy_seq_parallel_pg() -> None:
    if PROCESS_GROUP.initialized:
        PROCESS_GROUP.ULYSSES_PG = None
        PROCESS_GROUP.RING_PG = None
        PROCESS_GROUP.initialized = False
        PROCESS_GROUP._ulysses_degree = 1
        PROCESS_GROUP._ring_degree = 1
        PROCESS_GROUP._rank = 0
        PROCESS_GROUP._world_size = 1


def _resolve_groups(ulysses_pg, ring_pg, sp_ulysses_degree, sp_ring_degree):
    if ulysses_pg is None and PROCESS_GROUP.initialized:
        ulysses_pg = PROCESS_GROUP.ULYSSES_PG
    if ring_pg is None and PROCESS_GROUP.initialized:
        ring_pg = PROCESS_GROUP.RING_PG
    if sp_ulysses_degree is None and PROCESS_GROUP.initialized:
        sp_ulysses_degree = PROCESS_GROUP.ulysses_degree
    if sp_ring_degree is None and PROCESS_GROUP.initialized:
        sp_ring_degree = PROCESS_GROUP.ring_degree
    return ulysses_pg, ring_pg, sp_ulysses_degree or 1, sp_ring_degree or 1


class LongContextAttention(torch.nn.Module):
    """Ulysses all-to-all inside, ring attention across; ctor and forward
    signature of sp_aurora/hybrid/long_ctx_attention.py:30-43,:101-115."""

    def __init__(self, scatter_idx: int = 2, gather_idx: int = 1,
                 sp_ulysses_degree: Optional[int] = None, sp_ring_degree: Optional[int] = None,
                 use_ulysses: bool = True, use_ring: bool = True,
                 ulysses_pg: Optional[dist.ProcessGroup] = None,
                 ring_pg: Optional[dist.ProcessGroup] = None,
                 attn_type: Union[str, AttnType] = AttnType.FA, use_pack_qkv: bool = False,
                 use_sync: bool = False):
        super().__init__()
        self.attn_type = AttnType(attn_type)   # any reference or yunchang spelling; ignored
        ulysses_pg, ring_pg, u, r = _resolve_groups(ulysses_pg, ring_pg, sp_ulysses_degree,
                                                    sp_ring_degree)
        self.sp_ulysses_degree, self.sp_ring_degree = u, r
        self.use_ulysses = use_ulysses and u > 1
        self.use_ring = use_ring and r > 1
        self.ulysses_pg, self.ring_pg = ulysses_pg, ring_pg
        self.scatter_idx, self.gather_idx = scatter_idx, gather_idx
        self.use_pack_qkv = use_pack_qkv
        self.use_sync = use_sync

    def forward(self, query, key, value, dropout_p: float = 0.0,
                softmax_scale: Optional[float] = None, causal: bool = False,
                window_size: Tuple[int, int] = (-1, -1), softcap: float = 0.0,
                alibi_slopes=None, deterministic: bool = False, return_attn_probs: bool = False,
                joint_tensor_key_value: Optional[torch.Tensor] = None):
        check_unsupported_kwargs(dropout_p, window_size, alibi_slopes, softcap)
        if joint_tensor_key_value is not None:
            key = joint_tensor_key_value[:, :, 0]
            value = joint_tensor_key_value[:, :, 1]
        upg = self.ulysses_pg if self.use_ulysses else None
        if upg is not None:
            # q, k and v (equal or GQA head counts) travel as ONE all-to-all message and are
            # read where they land; `use_pack_qkv` therefore changes nothing here
            # (sp_aurora/hybrid/long_ctx_attention.py:136-153 stacks or sends three).
            if self.scatter_idx != 2 or self.gather_idx != 1:
                raise ValueError("LongContextAttention reshards heads (2) against sequence (1)")
            query, key, value = HeadsAllToAllPacked.apply(upg, query, key, value)
        res = ring_flash_attn_func(query, key, value, dropout_p=dropout_p,
                                   softmax_scale=softmax_scale, causal=causal,
                                   window_size=window_size, alibi_slopes=alibi_slopes,
                                   deterministic=deterministic, return_attn_probs=True,
                                   group=self.ring_pg if self.use_ring else _SelfGroup.get())
        out, lse = res[0], res[1]
        if upg is not None:
            out = SeqAllToAll4D.apply(upg, out, self.gather_idx, self.scatter_idx, self.use_sync)
            if return_attn_probs:
                lse = reshard_lse(lse.detach(), upg)
        return (out, lse, None) if return_attn_probs else out


class LongContextAttentionQKVPacked(torch.nn.Module):
    """qkv-packed hybrid: one 5-D all-to-all for q, k and v, then the ring.
    forward(qkv [B, S_local, 3, H, D]) -> out [B, S_local, H, D] (and lse)."""

    def __init__(self, scatter_idx: int = 3, gather_idx: int = 1,
                 sp_ulysses_degree: Optional[int] = None, sp_ring_degree: Optional[int] = None,
                 ulysses_pg=None, ring_pg=None, attn_type: Union[str, AttnType] = AttnType.FA,
                 use_sync: bool = False):
        super().__init__()
        self.attn_type = AttnType(attn_type)   # any reference or yunchang spelling; ignored
        ulysses_pg, ring_pg, u, r = _resolve_groups(ulysses_pg, ring_pg, sp_ulysses_degree,
                                                    sp_ring_degree)
        self.ulysses_pg, self.ring_pg = (ulysses_pg if u > 1 else None), ring_pg
        self.use_ring = r > 1
        self.scatter_idx, self.gather_idx, self.use_sync = scatter_idx, gather_idx, use_sync

    def forward(self, qkv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
        check_unsupported_kwargs(dropout_p, window_size, alibi_slopes, softcap)
        upg = self.ulysses_pg
        if upg is not None:
            qkv = SeqAllToAll5D.apply(upg, qkv, self.scatter_idx, self.gather_idx, self.use_sync)
        res = ring_flash_attn_qkvpacked_func(qkv, dropout_p=dropout_p, softmax_scale=softmax_scale,
                                             causal=causal, window_size=window_size,
                                             alibi_slopes=alibi_slopes, deterministic=deterministic,
                                             return_attn_probs=True,
                                             group=self.ring_pg if self.use_ring else _SelfGroup.get())
        out, lse = res[0], res[1]
        if upg is not None:
            out = SeqAllToAll4D.apply(upg, out, 1, 2, self.use_sync)
            if return_attn_probs:
                lse = reshard_lse(lse.detach(), upg)
        return (out, lse, None) if return_attn_probs else out


class _SelfGroup:
    """A one-rank group so that 'no ring' means plain local attention even
    when the default group spans several ranks."""
    _group = None

    @classmethod
    def get(cls):
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return None
        if cls._group is None:
            # new_group is collective: every rank builds every singleton group.
            me = dist.get_rank()
            for r in range(dist.get_world_size()):
                g = dist.new_group([r])
                if r == me:
                    cls._group = g
        return cls._group
