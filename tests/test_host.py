"""CPU-side tests: the C-ABI library loads and exports every declared symbol,
argument validation, group layout, and the ring / all-to-all schedules driven
over world_size-2 gloo ranks with the CPU oracle standing in for the kernels."""
import os
import re
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import ctypes

    from sp_aurora_b200 import _lib
    header = open(os.path.join(ROOT, "include", "spa.h")).read()
    declared = set(re.findall(r"\b(spa_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in include/spa.h"
    raw = ctypes.CDLL(str(_lib._LIB_PATH))
    for name in declared:
        assert hasattr(raw, name), f"{name} declared in spa.h but not exported"
    assert declared == set(_lib.exported_symbols())
    assert _lib.launch_count() >= 0
    assert isinstance(_lib.lib.spa_last_error(), bytes)


def test_struct_layout_matches_header_order():
    """Field order of the ctypes structs follows the header's struct members."""
    from sp_aurora_b200 import _lib
    header = open(os.path.join(ROOT, "include", "spa.h")).read()
    for cname, struct in (("spa_fwd_args", _lib.FwdArgs), ("spa_bwd_args", _lib.BwdArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            parts = decl.split(",")
            names.append(re.findall(r"(\w+)$", parts[0].strip())[0])
            names.extend(p.strip().lstrip("*") for p in parts[1:])
        assert names == [f[0] for f in struct._fields_], cname


def test_cpu_tensors_are_rejected_loudly():
    import sp_aurora_b200 as spa
    q = torch.randn(1, 16, 2, 64)
    with pytest.raises(ValueError, match="CUDA"):
        spa.flash_attn_forward(q, q, q)
    with pytest.raises(ValueError, match="CUDA"):
        spa.ring_flash_attn_func(q, q, q)
    with pytest.raises(ValueError, match="CUDA"):
        spa.all_to_all.strided_copy(torch.empty(4, 8), torch.empty(4, 8))


def test_unsupported_kwargs_raise():
    from sp_aurora_b200.local_attn import check_unsupported_kwargs
    check_unsupported_kwargs(0.0, (-1, -1), None, 0.0)
    for kw in (dict(dropout_p=0.1), dict(window_size=(128, 0)), dict(alibi_slopes=torch.ones(2)),
               dict(softcap=1.0)):
        with pytest.raises(NotImplementedError):
            check_unsupported_kwargs(**kw)


def test_bad_c_abi_arguments_return_error_codes():
    import ctypes as C

    from sp_aurora_b200 import _lib
    a = _lib.FwdArgs()
    assert _lib.lib.spa_attn_fwd(C.byref(a)) == -1          # null pointers
    assert b"null" in _lib.lib.spa_last_error()
    b = _lib.BwdArgs()
    assert _lib.lib.spa_attn_bwd(C.byref(b)) == -1
    n = _lib.i64x4([1, 1, 1, 1])
    assert _lib.lib.spa_permute_rows(None, None, n, n, n, 16, None) == -1


def test_group_layout_is_causal_safe():
    from sp_aurora_b200.hybrid import seq_parallel_group_ranks
    u, r = seq_parallel_group_ranks(4, 2, 8)
    assert u == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert r == [[0, 4], [1, 5], [2, 6], [3, 7]]
    with pytest.raises(ValueError):
        seq_parallel_group_ranks(3, 2, 8)


def test_coalesce_merges_contiguous_dims():
    from sp_aurora_b200.all_to_all import _coalesce
    src = torch.empty(2, 3, 4, 8)
    dst = torch.empty(2, 3, 4, 8)
    assert _coalesce(list(src.shape), list(src.stride()), list(dst.stride()))[0] == [192]
    s2 = src.permute(1, 0, 2, 3)
    shape, ss, ds = _coalesce(list(s2.shape), list(s2.stride()), list(dst.view(3, 2, 4, 8).stride()))
    assert shape == [3, 2, 32] and ss == [32, 96, 1] and ds == [64, 32, 1]


# ---------------------------------------------------------------------------
# world_size-2 gloo runs
# ---------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _host_copy(dst, src):
    dst.copy_(src)
    return dst


def _zigzag_errs(rank, world, orc):
    """Balanced causal ring (internal zigzag re-layout) vs the full-sequence oracle."""
    from sp_aurora_b200 import zigzag
    errs = {}
    for hq, hkv, B in ((4, 4, 2), (4, 2, 2), (4, 2, 1)):   # batch 1 takes the merged-launch plan
        g = torch.Generator().manual_seed(21)
        S, D = 32 * world, 16
        q = torch.randn(B, S, hq, D, generator=g)
        k = torch.randn(B, S, hkv, D, generator=g)
        v = torch.randn(B, S, hkv, D, generator=g)
        dout = torch.randn(B, S, hq, D, generator=g)
        full_out, full_lse = orc.attention_ref(q, k, v, None, True)
        fdq, fdk, fdv = orc.attention_bwd_ref(dout, q, k, v, full_out, full_lse, None, True)
        sl = S // world
        sli = slice(rank * sl, (rank + 1) * sl)
        qs, ks, vs, ds = (t[:, sli].contiguous() for t in (q, k, v, dout))
        out, lse, saved = zigzag.zigzag_ring_forward(None, qs, ks, vs, D ** -0.5,
                                                     fwd_step=orc.fwd_step_cpu, cast_fn=orc.cast_cpu)
        dq, dk, dv = zigzag.zigzag_ring_backward(None, ds, *saved, D ** -0.5,
                                                 bwd_step=orc.bwd_step_cpu, delta_fn=orc.delta_cpu,
                                                 cast_fn=orc.cast_cpu)
        errs[(hq, hkv, B)] = [
            float((out.double() - full_out[:, sli]).abs().max()),
            float((lse.double() - full_lse[:, :, sli]).abs().max()),
            float((dq.double() - fdq[:, sli]).abs().max()),
            float((dk.double() - fdk[:, sli]).abs().max()),
            float((dv.double() - fdv[:, sli]).abs().max())]
        # the same problem with the shards handed over in the zigzag layout (half-chunks r and
        # 2W-1-r back to back): no re-layout exchange, results come back in that layout
        hc = S // (2 * world)
        rows = torch.cat((torch.arange(rank * hc, (rank + 1) * hc),
                          torch.arange((2 * world - 1 - rank) * hc, (2 * world - rank) * hc)))
        qs, ks, vs, ds = (t[:, rows].contiguous() for t in (q, k, v, dout))
        out, lse, saved = zigzag.zigzag_ring_forward(None, qs, ks, vs, D ** -0.5, fwd_step=orc.fwd_step_cpu,
                                                     cast_fn=orc.cast_cpu, input_layout="zigzag")
        dq, dk, dv = zigzag.zigzag_ring_backward(None, ds, *saved, D ** -0.5, bwd_step=orc.bwd_step_cpu,
                                                 delta_fn=orc.delta_cpu, cast_fn=orc.cast_cpu,
                                                 input_layout="zigzag")
        errs[(hq, hkv, B, "zigzag-in")] = [
            float((out.double() - full_out[:, rows]).abs().max()),
            float((lse.double() - full_lse[:, :, rows]).abs().max()),
            float((dq.double() - fdq[:, rows]).abs().max()),
            float((dk.double() - fdk[:, rows]).abs().max()),
            float((dv.double() - fdv[:, rows]).abs().max())]
    return errs


def _worker4(rank, world, port, ret):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from oracle import attention_oracle as orc
    res = {}
    try:
        res["zigzag_errs"] = _zigzag_errs(rank, world, orc)
    except Exception:  # noqa: BLE001
        import traceback
        res["error"] = traceback.format_exc()
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


def _worker(rank, world, port, golden, ret):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from oracle import attention_oracle as orc
    from sp_aurora_b200 import all_to_all as a2a
    from sp_aurora_b200 import ring
    res = {}
    try:
        gd = np.load(os.path.join(golden, "distributed.npz"))
        # all-to-all index arithmetic vs the reference's outputs (bit exact)
        x = torch.from_numpy(gd[f"a4_in_rank{rank}"])
        y = a2a.all_to_all_4D(x, 2, 1, copy_fn=_host_copy)
        z = a2a.all_to_all_4D(y, 1, 2, copy_fn=_host_copy)
        res["a4"] = torch.equal(y, torch.from_numpy(gd[f"a4_fwd_rank{rank}"])) and torch.equal(z, x)
        x5 = torch.from_numpy(gd[f"a5_in_rank{rank}"])
        y5 = a2a.all_to_all_5D(x5, 3, 1, copy_fn=_host_copy)
        z5 = a2a.all_to_all_5D(y5, 1, 3, copy_fn=_host_copy)
        res["a5"] = torch.equal(y5, torch.from_numpy(gd[f"a5_fwd_rank{rank}"])) and torch.equal(z5, x5)
        x1 = x[:1].contiguous()                          # B == 1: views, no unpack pass
        y1 = a2a.all_to_all_4D(x1, 2, 1, copy_fn=_host_copy)
        z1 = a2a.all_to_all_4D(y1, 1, 2, copy_fn=_host_copy)
        res["a4_b1"] = torch.equal(z1, x1)
        # q, k, v (GQA head counts) as one packed message, both directions, batch 2 and 1
        for Bp in (2, 1):
            ins = [[torch.arange(Bp * 8 * H * 4, dtype=torch.float32).view(Bp, 8, H, 4) + 1000 * r + 7 * t
                    for t, H in enumerate((4, 2, 2))] for r in range(world)]
            got = a2a.heads_all_to_all_packed(ins[rank], None, copy_fn=_host_copy)
            want = [orc.all_to_all_4d_ref([ins[r][t] for r in range(world)], 2, 1)[rank] for t in range(3)]
            back = a2a.seq_all_to_all_packed(got, None, copy_fn=_host_copy)
            res[f"packed_b{Bp}"] = all(torch.equal(g, w) for g, w in zip(got, want)) and \
                all(torch.equal(b, x) for b, x in zip(back, ins[rank]))
        lse = torch.arange(2 * 3 * 8, dtype=torch.float32).view(2, 3, 8) + 100 * rank
        rl = a2a.reshard_lse(lse, None)
        res["lse_shape"] = tuple(rl.shape) == (2, 6, 4)

        # RingComm value check (cf. the reference's test_ring.py:288-314)
        comm = ring.RingComm(None)
        t = torch.full((4,), float(rank))
        got = comm.send_recv(t)
        comm.commit()
        comm.wait()
        res["ringcomm"] = bool((got == float((rank - 1) % world)).all())

        # ring forward + backward schedule, oracle standing in for the kernels
        errs = {}
        for causal, hq, hkv in ((True, 4, 4), (False, 4, 2), (True, 4, 1)):
            g = torch.Generator().manual_seed(11)
            B, S, D = 2, 64, 16
            q = torch.randn(B, S, hq, D, generator=g)
            kv = torch.randn(B, S, 2, hkv, D, generator=g)
            dout = torch.randn(B, S, hq, D, generator=g)
            k, v = kv[:, :, 0], kv[:, :, 1]
            full_out, full_lse = orc.attention_ref(q, k, v, None, causal)
            fdq, fdk, fdv = orc.attention_bwd_ref(dout, q, k, v, full_out, full_lse, None, causal)
            sl = S // world
            sli = slice(rank * sl, (rank + 1) * sl)
            kvs = kv[:, sli].contiguous()
            qs, ks, vs, ds = q[:, sli].contiguous(), kvs[:, :, 0], kvs[:, :, 1], dout[:, sli].contiguous()
            out, lse = ring.ring_flash_attn_forward(None, qs, ks, vs, D ** -0.5, causal,
                                                    fwd_step=orc.fwd_step_cpu)
            dq, dk, dv = ring.ring_flash_attn_backward(
                None, ds, qs, ks, vs, out, lse, D ** -0.5, causal, bwd_step=orc.bwd_step_cpu,
                delta_fn=orc.delta_cpu, cast_fn=orc.cast_cpu)
            errs[(causal, hq, hkv)] = [
                float((out.double() - full_out[:, sli]).abs().max()),
                float((lse.double() - full_lse[:, :, sli]).abs().max()),
                float((dq.double() - fdq[:, sli]).abs().max()),
                float((dk.double() - fdk[:, sli]).abs().max()),
                float((dv.double() - fdv[:, sli]).abs().max())]
        res["ring_errs"] = errs
        res["zigzag_errs"] = _zigzag_errs(rank, world, orc)
    except Exception as e:  # noqa: BLE001
        import traceback
        res["error"] = traceback.format_exc()
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.fixture(scope="module")
def gloo_results(golden_dir):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), golden_dir, ret), nprocs=2, join=True)
    out = {r: dict(ret[r]) for r in range(2)}
    for r in out:
        assert "error" not in out[r], out[r].get("error")
    return out


def test_gloo_all_to_all_bit_exact_vs_reference(gloo_results):
    for r in range(2):
        assert gloo_results[r]["a4"] and gloo_results[r]["a5"] and gloo_results[r]["a4_b1"]
        assert gloo_results[r]["packed_b2"] and gloo_results[r]["packed_b1"]
        assert gloo_results[r]["lse_shape"]


def test_gloo_ring_comm(gloo_results):
    assert all(gloo_results[r]["ringcomm"] for r in range(2))


def test_gloo_ring_schedule_forward_backward(gloo_results):
    for r in range(2):
        for key, errs in gloo_results[r]["ring_errs"].items():
            assert max(errs) < 2e-5, (r, key, errs)   # fp32 hand-off between steps


def test_gloo_zigzag_ring_two_ranks(gloo_results):
    for r in range(2):
        for key, errs in gloo_results[r]["zigzag_errs"].items():
            assert max(errs) < 2e-5, (r, key, errs)


@pytest.mark.parametrize("world", [3, 4])
def test_gloo_zigzag_ring_more_ranks(world):
    """Odd and even ring sizes: with W = 3 both halves of one rank's shard come from the same
    peer on the last dK|dV hop, which is the case where per-peer message order matters."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker4, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        res = dict(ret[r])
        assert "error" not in res, res.get("error")
        for key, errs in res["zigzag_errs"].items():
            assert max(errs) < 2e-5, (r, key, errs)


def test_zigzag_merged_plan_covers_the_same_blocks():
    """The merged-launch plan (batch size 1) covers exactly the half-blocks of the
    per-half plan, with the same masks."""
    from sp_aurora_b200.zigzag import _plan, _step_calls
    for W in (2, 4, 8):
        for r in range(W):
            for s in range(W):
                want = sorted(_step_calls(s, r, W))
                got = []
                for q_lo, q_n, k_lo, k_n, causal, off in _plan(s, r, W, True):
                    for qh in range(q_lo, q_lo + q_n):
                        for kh in range(k_lo, k_lo + k_n):
                            # causal call with offset `off` halves: half-block (qh-q_lo, kh-k_lo)
                            # is diagonal when kh-k_lo == qh-q_lo+off, full when below it
                            d = (kh - k_lo) - (qh - q_lo) - off
                            assert not causal or d <= 0
                            got.append((qh, kh, bool(causal and d == 0)))
                assert sorted(got) == want, (W, r, s)
                unmerged = sorted((c[0], c[2], c[4]) for c in _plan(s, r, W, False))
                assert unmerged == want


def test_attn_type_accepts_reference_and_yunchang_names():
    """sp_aurora/ulysses/attn_layer.py:20-31: a str enum with these five values; every one
    (and the yunchang spellings) must construct both hybrid modules."""
    import sp_aurora_b200 as spa
    ref = {"TORCH": "torch", "INTEL_SYCL": "intel_sycl", "INTEL_ONEDNN": "intel_onednn",
           "FA": "flash_attn", "FA3": "flash_attn_3"}
    assert {m.name: m.value for m in spa.AttnType} == ref
    assert isinstance(spa.AttnType.FA, str) and spa.AttnType.FA == "flash_attn"
    for value in list(ref.values()) + ["fa", "fa3", "sage_fp8", "sparse_sage"] + list(spa.AttnType):
        spa.LongContextAttention(attn_type=value)
        spa.LongContextAttentionQKVPacked(attn_type=value)
        spa.UlyssesAttention(attn_type=value)
        assert callable(spa.select_flash_attn_impl(value))
    with pytest.raises(ValueError):
        spa.LongContextAttention(attn_type="no_such_backend")


def test_reference_export_names_exist():
    """Names a caller of the reference imports from the package root
    (sp_aurora/__init__.py:59-122, sp_aurora/intel_ring_flash_attn.py:453-456)."""
    import sp_aurora_b200 as spa
    for name in ("ring_flash_attn_func", "ring_flash_attn_kvpacked_func", "ring_flash_attn_qkvpacked_func",
                 "ulysses_flash_attn_func", "ulysses_flash_attn_kvpacked_func",
                 "ulysses_flash_attn_qkvpacked_func", "UlyssesComm", "SeqAllToAll4D", "SeqAllToAll5D",
                 "UlyssesAttention", "PROCESS_GROUP", "set_seq_parallel_pg", "HAS_LONG_CTX_ATTN",
                 "HAS_FLASH_ATTN", "HAS_SPARSE_SAGE_ATTENTION", "AttnType", "select_flash_attn_impl",
                 "LongContextAttention", "RingFlashAttnFunc", "update_out_and_lse", "RingComm",
                 "intel_ring_flash_attn_func", "intel_ring_flash_attn_kvpacked_func",
                 "intel_ring_flash_attn_qkvpacked_func", "IntelRingFlashAttnFunc",
                 "intel_ulysses_flash_attn_func", "sp_aurora_func", "sp_aurora_kvpacked_func",
                 "sp_aurora_qkvpacked_func", "SeqAllToAll4D_v2", "pytorch_attn_forward", "pytorch_attn_func",
                 "ring_pytorch_attn_func", "ring_pytorch_attn_forward", "substitute_hf_flash_attn",
                 "update_sp_aurora_params", "setup_mpi_distributed", "init_distributed_backend",
                 "cleanup_distributed", "get_device_for_rank", "detect_mpi_environment"):
        assert hasattr(spa, name), name
    # CPU tensors are refused loudly: there is no PyTorch fallback behind the yunchang-style names
    import torch
    x = torch.zeros(1, 8, 2, 32)
    with pytest.raises(ValueError):
        spa.pytorch_attn_func(x, x, x)
    comm = spa.UlyssesComm(None)
    assert comm.world_size == 1 and comm.rank == 0
    assert spa.HAS_SPARSE_SAGE_ATTENTION is False


def test_rope_arguments_are_validated_before_any_launch():
    """spa_rope_rows refuses bad head dims, misaligned strides and positions beyond the cos/sin
    tables with SPA_EINVAL (checked without a GPU: validation comes first)."""
    from sp_aurora_b200 import _lib
    lib = _lib.lib
    EINVAL = -1                        # SPA_EINVAL of include/spa.h
    buf = 0x10000                      # never dereferenced: the call is refused first
    n, st = _lib.i64x4([1, 2, 8, 4]), _lib.i64x4([0, 8 * 4 * 64, 4 * 64, 64])
    ok_args = (buf, buf, n, st, st, 64, 1, buf, buf, 8, 2, 0, 0, None)

    def call(**kw):
        names = ("src", "dst", "n", "ss", "ds", "D", "dtype", "cos", "sin", "rows", "pos_dim", "off", "inv",
                 "stream")
        a = dict(zip(names, ok_args))
        a.update(kw)
        return lib.spa_rope_rows(*[a[k] for k in names])
    assert call(D=48) == EINVAL
    assert call(off=1) == EINVAL                      # 8 positions from 1 exceed 8 table rows
    assert call(pos_dim=4) == EINVAL
    assert call(src=buf + 2) == EINVAL
    assert call(ds=_lib.i64x4([0, 8 * 4 * 64, 4 * 64, 3])) == EINVAL
    assert call(cos=None) == EINVAL


def test_misaligned_arguments_are_refused_before_any_launch():
    """Vector loads need 16-byte aligned bases and strides: the C ABI answers
    SPA_EINVAL instead of faulting (checked without a GPU: validation comes first)."""
    import ctypes as C
    from sp_aurora_b200 import _lib
    lib = _lib.lib
    buf = 0x10000                      # never dereferenced: the call is refused first
    bad = buf + 2
    H, D, S = 2, 64, 8
    ss, sb = H * D, S * H * D
    rc = lib.spa_bwd_delta(bad, sb, ss, D, buf, sb, ss, D, buf, 1, S, H, D, 1, None)
    assert rc == -1 and b"16" in lib.spa_last_error()
    rc = lib.spa_bwd_delta(buf, sb, ss + 1, D, buf, sb, ss, D, buf, 1, S, H, D, 1, None)
    assert rc == -1
    rc = lib.spa_cast_from_f32(buf, bad, sb, ss, D, 1, S, H, D, 1, C.c_float(1.0), None)
    assert rc == -1
    rc = lib.spa_merge(buf, buf, bad, sb, ss, D, buf, 1, S, H, D, 1, None)
    assert rc == -1
    a = _lib.FwdArgs()
    a.q, a.k, a.v, a.out, a.lse = bad, buf, buf, buf, buf
    for f in ("q", "k", "v", "o"):
        setattr(a, f + "_sb", sb), setattr(a, f + "_ss", ss), setattr(a, f + "_sh", D)
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.D, a.dtype, a.scale = 1, S, S, H, H, D, 1, 0.125
    assert lib.spa_attn_fwd(C.byref(a)) == -1
    b = _lib.BwdArgs()
    b.q, b.k, b.v, b.dout, b.lse, b.delta, b.dq, b.dk, b.dv = buf, buf, buf, buf, buf, buf, buf, bad, buf
    for f in ("q", "k", "v", "do"):
        setattr(b, f + "_sb", sb), setattr(b, f + "_ss", ss), setattr(b, f + "_sh", D)
    b.dq_overwrite = 1
    b.B, b.Sq, b.Sk, b.Hq, b.Hkv, b.D, b.dtype, b.scale = 1, S, S, H, H, D, 1, 0.125
    assert lib.spa_attn_bwd(C.byref(b)) == -1


def test_shared_memory_attribute_cache_is_per_device():
    """The opt-in shared-memory size is a per-device kernel attribute: the cache behind
    it must treat (kernel, device) as the key."""
    import ctypes as C
    from sp_aurora_b200 import _lib
    seen = _lib.lib.spa_internal_smem_attr_seen
    seen.restype, seen.argtypes = C.c_int, [C.c_void_p, C.c_int, C.c_int]
    k1, k2 = 0x1234000, 0x5678000
    assert seen(k1, 0, 1000) == 0 and seen(k1, 0, 1000) == 1      # second time: cached
    assert seen(k1, 1, 1000) == 0 and seen(k1, 1, 1000) == 1      # another device: not cached
    assert seen(k2, 0, 1000) == 0
    assert seen(k1, 0, 2000) == 0 and seen(k1, 0, 1500) == 1      # larger size: set again


def test_zigzag_plan_is_balanced():
    from sp_aurora_b200.zigzag import _step_calls, half_owner
    for W in (2, 4, 8):
        owners = sorted(half_owner(c, W) for c in range(2 * W))
        assert owners == sorted((r, s) for r in range(W) for s in (0, 1))
        for r in range(W):
            work = [sum(0.5 if c[2] else 1.0 for c in _step_calls(s, r, W)) for s in range(W)]
            assert work == [2.0] * W          # every rank, every step: two half-blocks


def test_bench_reference_arm_prints_contract_line():
    """`bench.py --impl reference` runs on host cores only (the oracle port on a bounded
    sample) and prints one JSON line with the keys the bench contract names."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, res.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "ring_attn_fwd_bwd_tflops"
    assert d["unit"] == "TFLOP/s" and d["higher_is_better"] is True and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["e2e"]["value"] == d["value"]


@pytest.mark.parametrize("W", [2, 3, 4, 5, 8])
def test_exchange_halves_message_matching_simulated(W, monkeypatch):
    """exchange_halves for every rank of rings up to 8, simulated in one process: the posted
    sends and receives are matched per (sender, receiver) pair in posting order, as NCCL and gloo
    do, and the data must land in the right half-chunks -- to the zigzag layout and back, and
    from the layout after W-1 hops (shift = W-1: where a finished dK|dV block sits) straight to
    the contiguous owners."""
    import torch.distributed as tdist
    from sp_aurora_b200 import zigzag

    class Op:
        def __init__(self, fn, tensor, peer, group=None):
            self.send, self.tensor, self.peer = fn is tdist.isend, tensor, peer

    class Req:
        def wait(self):
            pass

    posted = {}
    current = {"rank": 0}
    monkeypatch.setattr(zigzag, "_group_info", lambda group: (current["rank"], W))
    monkeypatch.setattr(zigzag, "_global", lambda group, r: r)
    monkeypatch.setattr(tdist, "P2POp", Op)
    monkeypatch.setattr(tdist, "batch_isend_irecv",
                        lambda ops: posted.setdefault(current["rank"], []).extend(ops) or [Req()])

    def run(to_zigzag, shift, src_of, dst_of):
        posted.clear()
        finishers = []
        for r in range(W):
            current["rank"] = r
            finishers.append(zigzag.exchange_halves([(src_of[r], dst_of[r])], None, to_zigzag, shift=shift,
                                                    defer=True))
        for s in range(W):
            for d in range(W):
                sends = [o for o in posted.get(s, []) if o.send and o.peer == d]
                recvs = [o for o in posted.get(d, []) if not o.send and o.peer == s]
                assert len(sends) == len(recvs), (s, d)
                for a, b in zip(sends, recvs):
                    b.tensor.copy_(a.tensor)
        for f in finishers:
            f()

    h = 3
    val = lambda c: torch.full((1, h, 2), float(c))          # half-chunk c carries the value c
    contiguous = {r: [val(2 * r), val(2 * r + 1)] for r in range(W)}
    zz = {r: [torch.empty(1, h, 2), torch.empty(1, h, 2)] for r in range(W)}
    run(True, 0, contiguous, zz)
    for r in range(W):
        assert float(zz[r][0][0, 0, 0]) == r and float(zz[r][1][0, 0, 0]) == 2 * W - 1 - r
    for shift in (0, W - 1):
        held = {r: [val((r - shift) % W), val(2 * W - 1 - (r - shift) % W)] for r in range(W)}
        back = {r: [torch.empty(1, h, 2), torch.empty(1, h, 2)] for r in range(W)}
        run(False, shift, held, back)
        for r in range(W):
            assert float(back[r][0][0, 0, 0]) == 2 * r and float(back[r][1][0, 0, 0]) == 2 * r + 1, (shift, r)
