"""ctypes binding of libspaurora_sm100.so (declared in include/spa.h).

The library is the only compute path of this package: if it is missing the
import raises, there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

import os

# SPA_LIB_PATH lets a developer load another build of the same library (A/B timing).
_LIB_PATH = Path(os.environ.get("SPA_LIB_PATH") or
                 Path(__file__).resolve().parent / "libspaurora_sm100.so")

SPA_OK = 0
SPA_BWD_BOTH, SPA_BWD_DQ_ONLY, SPA_BWD_DKV_ONLY = 0, 1, 2
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class SpaError(RuntimeError):
    """A C-ABI call returned a negative status."""


class FwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_sb", C.c_int64), ("q_ss", C.c_int64), ("q_sh", C.c_int64),
        ("k", C.c_void_p), ("k_sb", C.c_int64), ("k_ss", C.c_int64), ("k_sh", C.c_int64),
        ("v", C.c_void_p), ("v_sb", C.c_int64), ("v_ss", C.c_int64), ("v_sh", C.c_int64),
        ("out", C.c_void_p), ("o_sb", C.c_int64), ("o_ss", C.c_int64), ("o_sh", C.c_int64),
        ("out_acc", C.c_void_p),
        ("lse", C.c_void_p), ("lse_sb", C.c_int64), ("lse_sh", C.c_int64),
        ("B", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32),
        ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("causal_off", C.c_int32),
        ("merge_prev", C.c_int32),
        ("scale", C.c_float),
        ("stream", C.c_void_p),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_sb", C.c_int64), ("q_ss", C.c_int64), ("q_sh", C.c_int64),
        ("k", C.c_void_p), ("k_sb", C.c_int64), ("k_ss", C.c_int64), ("k_sh", C.c_int64),
        ("v", C.c_void_p), ("v_sb", C.c_int64), ("v_ss", C.c_int64), ("v_sh", C.c_int64),
        ("dout", C.c_void_p), ("do_sb", C.c_int64), ("do_ss", C.c_int64), ("do_sh", C.c_int64),
        ("lse", C.c_void_p), ("delta", C.c_void_p), ("lse_sb", C.c_int64), ("lse_sh", C.c_int64),
        ("dq_acc", C.c_void_p),
        ("dq", C.c_void_p), ("dq_sb", C.c_int64), ("dq_ss", C.c_int64), ("dq_sh", C.c_int64),
        ("dq_overwrite", C.c_int32),
        ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dkv_sb", C.c_int64), ("dkv_ss", C.c_int64), ("dkv_sh", C.c_int64),
        ("dkv_fp32", C.c_int32), ("dkv_accumulate", C.c_int32), ("deterministic", C.c_int32),
        ("passes", C.c_int32),
        ("B", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32),
        ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("causal_off", C.c_int32),
        ("scale", C.c_float),
        ("stream", C.c_void_p),
    ]


class BwdNoallocArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_sb", C.c_int64), ("q_ss", C.c_int64), ("q_sh", C.c_int64),
        ("k", C.c_void_p), ("k_sb", C.c_int64), ("k_ss", C.c_int64), ("k_sh", C.c_int64),
        ("v", C.c_void_p), ("v_sb", C.c_int64), ("v_ss", C.c_int64), ("v_sh", C.c_int64),
        ("out", C.c_void_p), ("o_sb", C.c_int64), ("o_ss", C.c_int64), ("o_sh", C.c_int64),
        ("dout", C.c_void_p), ("do_sb", C.c_int64), ("do_ss", C.c_int64), ("do_sh", C.c_int64),
        ("lse", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("B", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32),
        ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("causal_off", C.c_int32),
        ("scale", C.c_float),
        ("stream", C.c_void_p),
    ]


# Every symbol include/spa.h declares, with its ctypes signature.
_I64x4 = C.c_int64 * 4
_SIGNATURES = {
    "spa_attn_fwd": (C.c_int, [C.POINTER(FwdArgs)]),
    "spa_attn_bwd": (C.c_int, [C.POINTER(BwdArgs)]),
    "spa_attn_bwd_noalloc": (C.c_int, [C.POINTER(BwdNoallocArgs)]),
    "spa_noalloc_scratch_bytes": (C.c_int64, []),
    "spa_bwd_delta": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                C.c_void_p]),
    "spa_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                            C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                            C.c_void_p]),
    "spa_cast_from_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                    C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                    C.c_float, C.c_void_p]),
    "spa_permute_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64),
                                   C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int64,
                                   C.c_void_p]),
    "spa_rope_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                C.POINTER(C.c_int64), C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_void_p]),
    "spa_device_info": (C.c_int, [C.c_int32, C.POINTER(C.c_int64)]),
    "spa_check_status": (C.c_int, []),
    "spa_launch_count": (C.c_int64, []),
    "spa_last_error": (C.c_char_p, []),
}


def _rebuild_if_stale() -> str:
    """Developer convenience: when a compiler is present and a source file is
    newer than the library, recompile before loading (never a fallback: without
    nvcc a stale or missing library still fails below). Returns the build error
    text, if any, so that a missing library can be explained."""
    from . import build as _build   # plain build recipe, does not load the library
    if os.environ.get("SPA_LIB_PATH"):
        return ""
    try:
        stale = _build._stale(_LIB_PATH, [_build.CSRC / s for s in _build.SOURCES] + _build.HEADERS)
        if stale:
            _build.build()      # serialised across processes by a file lock; re-checks staleness
    except RuntimeError as e:
        return str(e)
    return ""


def _load() -> C.CDLL:
    build_error = _rebuild_if_stale()
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python sp_aurora_b200/build.py` "
            "(this package has no fallback path)" + (f"\nlast build attempt:\n{build_error}" if build_error else ""))
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the .so does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def exported_symbols():
    return sorted(_SIGNATURES)


def check(rc: int, what: str) -> None:
    if rc != SPA_OK:
        msg = lib.spa_last_error().decode(errors="replace")
        raise SpaError(f"{what} failed with status {rc}: {msg}")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def check_status() -> None:
    """Synchronise the current device and raise if a bounded device wait gave up."""
    check(lib.spa_check_status(), "spa_check_status")


def maybe_check_status() -> None:
    """With SPA_CHECK_STATUS=1 in the environment: check_status() (a device synchronise) at
    the end of every backward of the public attention functions, so that a bounded wait that
    gave up surfaces as an exception in the training loop instead of as wrong gradients."""
    if os.environ.get("SPA_CHECK_STATUS") == "1":
        check_status()


def launch_count() -> int:
    return int(lib.spa_launch_count())


def device_info(device: int = 0) -> dict:
    buf = (C.c_int64 * 6)()
    check(lib.spa_device_info(device, buf), "spa_device_info")
    keys = ["sm_count", "cc_major", "cc_minor", "smem_optin_bytes", "l2_bytes", "global_mem_mib"]
    return dict(zip(keys, [int(x) for x in buf]))


def i64x4(vals):
    return _I64x4(*[int(v) for v in vals])
