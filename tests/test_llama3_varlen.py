"""Packed-stream (llama3-style) sequence parallelism: segment tables and the all-gather /
reduce-scatter schedule on gloo ranks with the CPU oracle in place of the kernels
(counterpart of what sp_aurora/adapters/hf_adapter.py:34-55,141-155 expects to import)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_prepare_cu_seqlens_tables():
    from sp_aurora_b200.llama3_varlen import llama3_flash_attn_prepare_cu_seqlens as prep
    cu = torch.tensor([0, 5, 12, 12, 16], dtype=torch.int32)        # lengths 5, 7, 0, 4; T = 16
    # two ranks of 8 tokens: rank 0 holds seq0 and 3 tokens of seq1, rank 1 the rest
    cq, ck, mq, mk, ks = prep(cu, True, 0, 2)
    assert cq.tolist() == [0, 5, 8] and ck.tolist() == [0, 5, 8] and (mq, mk) == (5, 5) and ks == slice(0, 8)
    cq, ck, mq, mk, ks = prep(cu, True, 1, 2)
    # segment 1: 4 queries of seq1 (tokens 8..12) see its keys 5..12; segment 2: seq3 whole
    assert cq.tolist() == [0, 4, 8] and ck.tolist() == [0, 7, 11] and (mq, mk) == (4, 7) and ks == slice(5, 16)
    # non-causal: rank 0's part of seq1 sees all of seq1
    cq, ck, mq, mk, ks = prep(cu, False, 0, 2)
    assert cq.tolist() == [0, 5, 8] and ck.tolist() == [0, 5, 12] and ks == slice(0, 12) and mk == 7
    # one rank: the plain varlen tables
    cq, ck, _, _, ks = prep([0, 5, 12, 12, 16], True, 0, 1)
    assert cq.tolist() == [0, 5, 12, 16] == ck.tolist() and ks == slice(0, 16) and cq.dtype == torch.int32
    # a sequence spanning three ranks
    cq, ck, _, _, ks = prep([0, 2, 18], True, 1, 3)
    assert cq.tolist() == [0, 6] and ck.tolist() == [0, 10] and ks == slice(2, 12)
    with pytest.raises(ValueError):
        prep([0, 5, 11], True, 0, 2)                                 # 11 tokens over 2 ranks
    with pytest.raises(ValueError):
        prep([0, 7, 5], True, 0, 1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    res = {}
    try:
        from oracle import attention_oracle as orc
        from sp_aurora_b200 import llama3_varlen as l3
        errs = {}
        T = 24 * world
        cases = [([0, 7, 7 + 16 * world, T - 3, T], 4, 2, True, 1),     # GQA, one kv head at a time
                 ([0, T], 2, 2, True, 2),                               # one sequence over all ranks
                 ([0, 5, T - 11, T], 4, 4, False, 4),                   # non-causal
                 ([0, 9, 9, T // 2, T], 4, 2, True, 2)]                 # an empty sequence, a rank boundary
        for ci, (cu, hq, hkv, causal, stride) in enumerate(cases):
            g = torch.Generator().manual_seed(100 + ci)
            D = 16
            q = torch.randn(T, hq, D, generator=g)
            k = torch.randn(T, hkv, D, generator=g)
            v = torch.randn(T, hkv, D, generator=g)
            dout = torch.randn(T, hq, D, generator=g)
            # full-stream oracle, sequence by sequence
            ro, rl = torch.zeros(T, hq, D, dtype=torch.float64), torch.zeros(hq, T, dtype=torch.float64)
            rdq, rdk, rdv = (torch.zeros(T, h, D, dtype=torch.float64) for h in (hq, hkv, hkv))
            for s0, s1 in zip(cu, cu[1:]):
                if s1 == s0:
                    continue
                sl = slice(s0, s1)
                o, l = orc.attention_ref(q[None, sl], k[None, sl], v[None, sl], None, causal)
                a, b, c = orc.attention_bwd_ref(dout[None, sl], q[None, sl], k[None, sl], v[None, sl], o, l,
                                                None, causal)
                ro[sl], rl[:, sl], rdq[sl], rdk[sl], rdv[sl] = o[0], l[0], a[0], b[0], c[0]
            per = T // world
            mine = slice(rank * per, (rank + 1) * per)
            cq, ck, _, _, ks = l3.llama3_flash_attn_prepare_cu_seqlens(cu, causal, rank, world)
            segs = l3._segments(cq, ck)
            ql, kl, vl, dl = (t[mine].contiguous() for t in (q, k, v, dout))
            out, lse = l3.llama3_forward(None, ql, kl, vl, segs, ks, stride, D ** -0.5, causal,
                                         fwd_step=orc.fwd_step_cpu)
            dq, dk, dv = l3.llama3_backward(None, dl, ql, kl, vl, out, lse, segs, ks, stride, D ** -0.5,
                                            causal, bwd_step=orc.bwd_step_cpu, delta_fn=orc.delta_cpu,
                                            cast_fn=orc.cast_cpu)
            errs[ci] = [float((out.double() - ro[mine]).abs().max()),
                        float((lse.double() - rl[:, mine]).abs().max()),
                        float((dq.double() - rdq[mine]).abs().max()),
                        float((dk.double() - rdk[mine]).abs().max()),
                        float((dv.double() - rdv[mine]).abs().max())]
        res["errs"] = errs
    except Exception:  # noqa: BLE001
        import traceback
        res["error"] = traceback.format_exc()
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_llama3_schedule_on_gloo_ranks(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        res = dict(ret[r])
        assert "error" not in res, res.get("error")
        for ci, errs in res["errs"].items():
            assert max(errs) < 2e-5, (r, ci, errs)
