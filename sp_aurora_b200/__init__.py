"""sp_aurora_b200: the sequence-parallel attention hot path of sp-aurora (ring,
Ulysses and hybrid attention, forward and backward) on NVIDIA B200 (sm_100a).

The export list follows sp_aurora/__init__.py:59-122; the `sp_aurora_*` names
are the spellings the reference's documentation uses for the ring functions.
All compute goes through libspaurora_sm100.so (hand-written CUDA, C ABI in
include/spa.h); importing this package fails if that library is not built.
"""
from ._lib import SpaError, check_status, device_info, launch_count  # noqa: F401  (loads the .so)
from .local_attn import (  # noqa: F401
    flash_attn_backward,
    flash_attn_forward,
    update_out_and_lse,
)
from .ring import (  # noqa: F401
    RingComm,
    RingFlashAttnFunc,
    ring_flash_attn_backward,
    ring_flash_attn_forward,
    ring_flash_attn_func,
    ring_flash_attn_kvpacked_func,
    ring_flash_attn_qkvpacked_func,
)
from .all_to_all import (  # noqa: F401
    SeqAllToAll4D,
    SeqAllToAll5D,
    all_to_all_4D,
    all_to_all_5D,
    seq_all_to_all_4d_inference,
)
from .ulysses import (  # noqa: F401
    AttnType,
    UlyssesAttention,
    UlyssesComm,
    UlyssesFlashAttnFunc,
    select_flash_attn_impl,
    ulysses_flash_attn_func,
    ulysses_flash_attn_kvpacked_func,
    ulysses_flash_attn_qkvpacked_func,
)
from .hybrid import (  # noqa: F401
    PROCESS_GROUP,
    LongContextAttention,
    LongContextAttentionQKVPacked,
    destroy_seq_parallel_pg,
    set_seq_parallel_pg,
    high_priority_nccl_options,
)

from .example_block import SequenceParallelAttentionBlock  # noqa: F401
from .llama3_varlen import (  # noqa: F401
    llama3_flash_attn_prepare_cu_seqlens,
    llama3_flash_attn_varlen_func,
)
from .adapters import (  # noqa: F401
    substitute_hf_flash_attn,
    update_ring_flash_attn_params,
    update_sp_aurora_params,
    use_ring_attn,
)
from .rope import apply_rope, rope_copy, rope_tables  # noqa: F401
from .mpi_utils import (  # noqa: F401
    cleanup_distributed,
    detect_mpi_environment,
    get_device_for_rank,
    init_distributed_backend,
    setup_mpi_distributed,
)
from .varlen import (  # noqa: F401
    ring_flash_attn_varlen_func,
    zigzag_ring_flash_attn_func,
    zigzag_ring_flash_attn_varlen_func,
)

# Names used by the reference's README and tests for the ring entry points.
sp_aurora_func = ring_flash_attn_func
sp_aurora_kvpacked_func = ring_flash_attn_kvpacked_func
sp_aurora_qkvpacked_func = ring_flash_attn_qkvpacked_func
# Names the reference's varlen test imports
# (test/flash_attention/test_intel_ring_flash_attn_varlen.py:23-26).
sp_aurora_varlen_func = ring_flash_attn_varlen_func
zigzag_sp_aurora_func = zigzag_ring_flash_attn_func
zigzag_sp_aurora_varlen_func = zigzag_ring_flash_attn_varlen_func

# The reference's own spellings (sp_aurora/intel_ring_flash_attn.py:453-456,
# sp_aurora/intel_ulysses_attn.py:501-624, sp_aurora/__init__.py:59-72).
intel_ring_flash_attn_func = ring_flash_attn_func
intel_ring_flash_attn_kvpacked_func = ring_flash_attn_kvpacked_func
intel_ring_flash_attn_qkvpacked_func = ring_flash_attn_qkvpacked_func
IntelRingFlashAttnFunc = RingFlashAttnFunc
intel_ulysses_flash_attn_func = ulysses_flash_attn_func
intel_ulysses_flash_attn_kvpacked_func = ulysses_flash_attn_kvpacked_func
intel_ulysses_flash_attn_qkvpacked_func = ulysses_flash_attn_qkvpacked_func
IntelUlyssesComm = UlyssesComm
IntelSeqAllToAll4D = SeqAllToAll4D

# Feature flags of sp_aurora/globals.py:171-173.
HAS_LONG_CTX_ATTN = True
HAS_FLASH_ATTN = True
HAS_SPARSE_SAGE_ATTENTION = False


def is_available() -> bool:
    """True when a CUDA device of compute capability 10.x is present
    (counterpart of sp_aurora/sycl_bindings/bindings.cpp:362 is_available)."""
    import torch
    if not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability()[0] == 10


__version__ = "0.1.0"


# yunchang-style names the reference also exports (sp_aurora/kernels/attention.py:12-117,
# sp_aurora/ring_pytorch_attn.py:20-240, sp_aurora/__init__.py:75). They are the same CUDA path
# under the other spelling, not a PyTorch implementation.
SeqAllToAll4D_v2 = SeqAllToAll4D


def pytorch_attn_forward(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                         window_size=(-1, -1), softcap=0.0, alibi_slopes=None, deterministic=False,
                         return_attn_probs=False):
    """Single-device attention on [B, S, H, D] tensors: (out, lse or None). The reference
    returns the S x S probability matrix with `return_attn_probs`; here the second value is the
    fp32 log-sum-exp [B, H, S], which is what the ring and hybrid callers consume."""
    from .local_attn import LocalFlashAttnFunc, check_unsupported_kwargs
    check_unsupported_kwargs(dropout_p, window_size, alibi_slopes, softcap)
    out, lse = LocalFlashAttnFunc.apply(q, k, v, softmax_scale, causal)
    return out, (lse if return_attn_probs else None)


def pytorch_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                      softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
    return pytorch_attn_forward(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap,
                                alibi_slopes, deterministic, False)[0]


def ring_pytorch_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                           window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                           return_attn_probs=False, group=None):
    return ring_flash_attn_func(q, k, v, dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal,
                                window_size=window_size, alibi_slopes=alibi_slopes,
                                deterministic=deterministic, return_attn_probs=return_attn_probs,
                                group=group)


def ring_pytorch_attn_forward(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                              window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                              return_attn_probs=False, group=None):
    """(out, lse): the reference's version returns None for lse (sp_aurora/ring_pytorch_attn.py:236)."""
    res = ring_flash_attn_func(q, k, v, dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal,
                               window_size=window_size, alibi_slopes=alibi_slopes,
                               deterministic=deterministic, return_attn_probs=True, group=group)
    return res[0], res[1]
