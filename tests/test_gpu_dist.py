"""Multi-GPU parity tests (NCCL, one process per GPU, every visible GPU up to 8): ring,
Ulysses and hybrid attention, forward and backward, each rank compared with its slice of
the full-sequence CPU oracle (the method of the reference's
test/test_ring_attention_full_accuracy.py:108-171), plus independence of the world size,
bitwise repeatability and one BASELINE-sized case checked on row slices. Skipped when
fewer than two GPUs are visible; the schedules themselves are also covered on CPU ranks
in tests/test_host.py."""
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rand(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * std


def _errs(pairs):
    return [float((a.detach().cpu().double() - b).abs().max()) for a, b in pairs]


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from sp_aurora_b200 import high_priority_nccl_options
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            pg_options=high_priority_nccl_options())
    res = {}
    try:
        import sp_aurora_b200 as spa
        from oracle import attention_oracle as orc
        sl_of = lambda S: slice(rank * (S // world), (rank + 1) * (S // world))

        # ---- ring: fp32 anchor (B2 S1024 H32 D64 causal at W=2) and bf16 GQA kv-packed
        # causal rings run on the balanced (zigzag) schedule by default; "_contig"
        # repeats one case on the plain contiguous-shard schedule
        for tag, dtype, B, S, Hq, Hkv, D, causal, tol in (
                ("ring_fp32", torch.float32, 2, 1024, 32, 32, 64, True, 1e-4),
                ("ring_bf16_gqa", torch.bfloat16, 1, 2048, 8, 2, 128, True, 2e-2),
                ("ring_bf16_gqa_contig", torch.bfloat16, 1, 2048, 8, 2, 128, True, 2e-2),
                ("ring_bf16_noncausal", torch.bfloat16, 1, 1024, 4, 4, 128, False, 2e-2)):
            os.environ["SPA_RING_ZIGZAG"] = "0" if tag.endswith("_contig") else "1"
            q = _rand((B, S, Hq, D), 1).to(dtype)
            kv = _rand((B, S, 2, Hkv, D), 2).to(dtype)
            do = _rand((B, S, Hq, D), 3).to(dtype)
            ro, rl = orc.attention_ref(q, kv[:, :, 0], kv[:, :, 1], None, causal)
            rdq, rdk, rdv = orc.attention_bwd_ref(do, q, kv[:, :, 0], kv[:, :, 1], ro, rl, None, causal)
            sl = sl_of(S)
            ql = q[:, sl].to(dev).requires_grad_(True)
            kvl = kv[:, sl].to(dev).requires_grad_(True)
            out, lse, _ = spa.sp_aurora_kvpacked_func(ql, kvl, causal=causal, return_attn_probs=True)
            out.backward(do[:, sl].to(dev))
            spa.check_status()
            e = _errs([(out, ro[:, sl]), (ql.grad, rdq[:, sl]), (kvl.grad[:, :, 0], rdk[:, sl]),
                       (kvl.grad[:, :, 1], rdv[:, sl])])
            el = _errs([(lse, rl[:, :, sl])])[0]
            gmax = max(1.0, float(rdv.abs().max()) / 4)
            res[tag] = (max(e[:1]) <= tol and max(e[1:]) <= tol * gmax and el <= 1e-3, e, el)

        # ---- Ulysses (non-causal and causal), B=2 exercises the unpack kernels
        hw = max(4, world)             # head counts divisible by the group size
        for tag, B, S, Hq, Hkv, D, causal in (("uly_b2", 2, 1024, 2 * hw, 2 * hw, 128, False),
                                              ("uly_gqa_causal", 1, 1024, 2 * hw, hw, 128, True)):
            q = _rand((B, S, Hq, D), 4).bfloat16()
            k = _rand((B, S, Hkv, D), 5).bfloat16()
            v = _rand((B, S, Hkv, D), 6).bfloat16()
            do = _rand((B, S, Hq, D), 7).bfloat16()
            ro, rl = orc.attention_ref(q, k, v, None, causal)
            rdq, rdk, rdv = orc.attention_bwd_ref(do, q, k, v, ro, rl, None, causal)
            sl = sl_of(S)
            ql, kl, vl = (t[:, sl].to(dev).requires_grad_(True) for t in (q, k, v))
            out, lse, _ = spa.ulysses_flash_attn_func(ql, kl, vl, causal=causal, return_attn_probs=True)
            out.backward(do[:, sl].to(dev))
            spa.check_status()
            e = _errs([(out, ro[:, sl]), (ql.grad, rdq[:, sl]), (kl.grad, rdk[:, sl]), (vl.grad, rdv[:, sl])])
            el = _errs([(lse, rl[:, :, sl])])[0]
            gmax = max(1.0, float(rdv.abs().max()) / 4)
            res[tag] = (max(e[:1]) <= 2e-2 and max(e[1:]) <= 2e-2 * gmax and el <= 1e-3, e, el)

        # ---- all-to-all bit exactness on the GPU (pack kernel + NCCL + unpack kernel)
        x = (torch.arange(2 * 64 * hw * 64, dtype=torch.float32).view(2, 64, hw, 64) + 1e6 * rank).to(dev)
        ins = [(torch.arange(2 * 64 * hw * 64, dtype=torch.float32).view(2, 64, hw, 64) + 1e6 * r)
               for r in range(world)]
        y = spa.all_to_all_4D(x, 2, 1)
        z = spa.all_to_all_4D(y, 1, 2)
        want = orc.all_to_all_4d_ref(ins, 2, 1)[rank]
        res["a2a_exact"] = (bool(torch.equal(y.cpu(), want) and torch.equal(z, x)), [], 0.0)

        # ---- hybrid: Ulysses degree `world`, ring degree 1, and U=1 x R=world, qkv-packed
        for tag, U, R in (("hyb_u", world, 1), ("hyb_r", 1, world)):
            spa.destroy_seq_parallel_pg()
            spa.set_seq_parallel_pg(U, R, rank, world)
            B, S, H, D = 1, 1024, hw, 128
            qkv = _rand((B, S, 3, H, D), 8).bfloat16()
            ro, rl = orc.attention_ref(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], None, True)
            sl = sl_of(S)
            mod = spa.LongContextAttentionQKVPacked()
            out, lse, _ = mod(qkv[:, sl].to(dev), causal=True, return_attn_probs=True)
            spa.check_status()
            e = _errs([(out, ro[:, sl])])
            el = _errs([(lse, rl[:, :, sl])])[0]
            res[tag] = (e[0] <= 2e-2 and el <= 1e-3, e, el)
        # ---- hybrid module with separate q,k,v and gradients (U x R = 2 x world/2 when possible)
        U = 2 if world % 2 == 0 and world > 2 else world
        R = world // U
        spa.destroy_seq_parallel_pg()
        spa.set_seq_parallel_pg(U, R, rank, world)
        B, S, H, D = 1, 1024, 4, 128
        q, k, v, do = (_rand((B, S, H, D), 20 + i).bfloat16() for i in range(4))
        ro, rl = orc.attention_ref(q, k, v, None, True)
        rdq, rdk, rdv = orc.attention_bwd_ref(do, q, k, v, ro, rl, None, True)
        sl = sl_of(S)
        ql, kl, vl = (t[:, sl].to(dev).requires_grad_(True) for t in (q, k, v))
        mod = spa.LongContextAttention()
        out = mod(ql, kl, vl, causal=True)
        out.backward(do[:, sl].to(dev))
        spa.check_status()
        e = _errs([(out, ro[:, sl]), (ql.grad, rdq[:, sl]), (kl.grad, rdk[:, sl]), (vl.grad, rdv[:, sl])])
        gmax = max(1.0, float(rdv.abs().max()) / 4)
        res["hyb_bwd"] = (e[0] <= 2e-2 and max(e[1:]) <= 2e-2 * gmax, e, 0.0)
        spa.destroy_seq_parallel_pg()

        # ---- cfg5's split (Ulysses 4 inside, ring 2 across) when 8 GPUs are visible
        if world == 8:
            spa.set_seq_parallel_pg(4, 2, rank, world)
            B, S, H, D = 1, 8192, 16, 128
            qkv = _rand((B, S, 3, H, D), 30).bfloat16()
            ro, rl = orc.attention_ref(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], None, True,
                                       dtype=torch.float32)
            sl = sl_of(S)
            out, lse, _ = spa.LongContextAttentionQKVPacked()(qkv[:, sl].to(dev), causal=True,
                                                              return_attn_probs=True)
            spa.check_status()
            e = _errs([(out, ro[:, sl])])
            el = _errs([(lse, rl[:, :, sl])])[0]
            res["hyb_u4r2"] = (e[0] <= 2e-2 and el <= 1e-3, e, el)
            spa.destroy_seq_parallel_pg()
        else:
            res["hyb_u4r2"] = (True, ["needs 8 GPUs"], 0.0)

        # ---- independence of the world size: the ring over all ranks, rings over pairs of
        # ranks and one GPU alone give the same numbers on the same global tensors
        B, S, Hq, Hkv, D = 1, 2048, 8, 2, 128
        q = _rand((B, S, Hq, D), 41).bfloat16()
        kv = _rand((B, S, 2, Hkv, D), 42).bfloat16()
        do = _rand((B, S, Hq, D), 43).bfloat16()

        def ring_run(group, w, r):
            sl = slice(r * (S // w), (r + 1) * (S // w))
            ql = q[:, sl].to(dev).requires_grad_(True)
            kvl = kv[:, sl].to(dev).requires_grad_(True)
            out, lse, _ = spa.sp_aurora_kvpacked_func(ql, kvl, causal=True, return_attn_probs=True,
                                                      group=group, deterministic=True)
            out.backward(do[:, sl].to(dev))
            return sl, [out.detach(), lse, ql.grad, kvl.grad]

        sl_w, full = ring_run(None, world, rank)
        sl_w2, again = ring_run(None, world, rank)
        res["run_twice_bitwise"] = (all(torch.equal(a, b) for a, b in zip(full, again)), [], 0.0)
        qf, kvf = q.to(dev).requires_grad_(True), kv.to(dev).requires_grad_(True)
        o1, l1 = spa.flash_attn_forward(qf, kvf[:, :, 0], kvf[:, :, 1], None, True)
        g1 = spa.flash_attn_backward(do.to(dev), qf, kvf[:, :, 0], kvf[:, :, 1], o1, l1, None, True)
        one = [o1[:, sl_w], l1[:, :, sl_w], g1[0][:, sl_w], torch.stack((g1[1], g1[2]), dim=2)[:, sl_w]]
        diffs = [float((a.float() - b.float()).abs().max()) for a, b in zip(full, one)]
        pair_diffs = [0.0] * 4
        pairs = [dist.new_group([2 * i, 2 * i + 1]) for i in range(world // 2)]   # collective
        if world >= 4:
            sl_p, pr = ring_run(pairs[rank // 2], 2, rank % 2)
            ref2 = [o1[:, sl_p], l1[:, :, sl_p], g1[0][:, sl_p], torch.stack((g1[1], g1[2]), dim=2)[:, sl_p]]
            pair_diffs = [float((a.float() - b.float()).abs().max()) for a, b in zip(pr, ref2)]
        spa.check_status()
        gmax = max(1.0, float(g1[2].float().abs().max()) / 4)
        ok = all(d <= 2e-2 * (gmax if i >= 2 else 1.0) for i, d in enumerate(diffs) if i != 1) and \
            diffs[1] <= 1e-3 and pair_diffs[1] <= 1e-3 and \
            all(d <= 2e-2 * (gmax if i >= 2 else 1.0) for i, d in enumerate(pair_diffs) if i != 1)
        res["world_size_independence"] = (ok, diffs + pair_diffs, 0.0)

        # ---- public zigzag layout and packed variable-length sequences over the ring
        H, D = 4, 128
        lengths = [512 * world // 2, 256 * world // 2 * 2, 128 * world]      # global lengths, multiples of 2*world
        gq, gk, gv, gdo = ([_rand((1, L, H, D), 60 + 10 * t + i).bfloat16() for i, L in enumerate(lengths)]
                           for t in range(4))
        refs = []
        for i in range(len(lengths)):
            ro, rl = orc.attention_ref(gq[i], gk[i], gv[i], None, True, dtype=torch.float32)
            refs.append((ro, rl) + orc.attention_bwd_ref(gdo[i], gq[i], gk[i], gv[i], ro, rl, None, True,
                                                         dtype=torch.float32))
        worst = [0.0] * 5
        for layout in ("contiguous", "zigzag"):
            def shard(x):
                L = x.shape[1]
                if layout == "contiguous":
                    return x[0, rank * (L // world):(rank + 1) * (L // world)]
                hc = L // (2 * world)
                return torch.cat((x[0, rank * hc:(rank + 1) * hc],
                                  x[0, (2 * world - 1 - rank) * hc:(2 * world - rank) * hc]))
            ql, kl, vl, dol = (torch.cat([shard(x) for x in g]).to(dev) for g in (gq, gk, gv, gdo))
            ql, kl, vl = (t.requires_grad_(True) for t in (ql, kl, vl))
            cu = torch.tensor([0] + list(torch.tensor([L // world for L in lengths]).cumsum(0)),
                              dtype=torch.int32, device=dev)
            fn = spa.sp_aurora_varlen_func if layout == "contiguous" else spa.zigzag_sp_aurora_varlen_func
            out, lse, _ = fn(ql, kl, vl, cu, cu, max_seqlen=max(lengths) // world, causal=True,
                             return_attn_probs=True)
            out.backward(dol)
            spa.check_status()
            for i in range(len(lengths)):
                sl = slice(int(cu[i]), int(cu[i + 1]))
                want = [shard(r) if r.dim() == 4 else None for r in refs[i]]
                lse_ref = refs[i][1]
                Lg = lengths[i]
                if layout == "contiguous":
                    lw = lse_ref[0, :, rank * (Lg // world):(rank + 1) * (Lg // world)]
                else:
                    hc = Lg // (2 * world)
                    lw = torch.cat((lse_ref[0, :, rank * hc:(rank + 1) * hc],
                                    lse_ref[0, :, (2 * world - 1 - rank) * hc:(2 * world - rank) * hc]), dim=1)
                e = _errs([(out[sl], want[0]), (lse[:, sl], lw), (ql.grad[sl], want[2]), (kl.grad[sl], want[3]),
                           (vl.grad[sl], want[4])])
                worst = [max(a, b) for a, b in zip(worst, e)]
        gmax = max(1.0, max(float(r[4].abs().max()) for r in refs) / 4)
        res["varlen_and_zigzag_layout"] = (worst[0] <= 2e-2 and worst[1] <= 1e-3 and max(worst[2:]) <= 2e-2 * gmax,
                                           worst, worst[1])

        # ---- packed stream split evenly over the ranks (llama3-style: all-gather K/V, sequences
        # straddling rank boundaries), GQA, kv heads gathered two at a time, bf16, fwd + bwd
        T, hq, hkv, D = 1024 * world, 8, 4, 128
        cu = [0, 300, 300 + 640 * world, T - 200, T]
        gens = [torch.Generator().manual_seed(1200 + i) for i in range(4)]
        qg, dog = (torch.randn(T, hq, D, generator=g).bfloat16() for g in (gens[0], gens[3]))
        kg, vg = (torch.randn(T, hkv, D, generator=g).bfloat16() for g in gens[1:3])
        ro, rl = torch.zeros(T, hq, D), torch.zeros(hq, T)
        rdq, rdk, rdv = torch.zeros(T, hq, D), torch.zeros(T, hkv, D), torch.zeros(T, hkv, D)
        for s0, s1 in zip(cu, cu[1:]):
            ss = slice(s0, s1)
            o, l = orc.attention_ref(qg[None, ss], kg[None, ss], vg[None, ss], None, True, dtype=torch.float32)
            a, b_, c = orc.attention_bwd_ref(dog[None, ss], qg[None, ss], kg[None, ss], vg[None, ss], o, l,
                                             None, True, dtype=torch.float32)
            ro[ss], rl[:, ss], rdq[ss], rdk[ss], rdv[ss] = o[0], l[0], a[0], b_[0], c[0]
        mine = slice(rank * (T // world), (rank + 1) * (T // world))
        ql, kl, vl = (t[mine].to(dev).requires_grad_(True) for t in (qg, kg, vg))
        cq, ck, mq, mk, ks = spa.llama3_flash_attn_prepare_cu_seqlens(cu, True, rank, world)
        out, lse, _ = spa.llama3_flash_attn_varlen_func(ql, kl, vl, cq, ck, mq, mk, heads_k_stride=2,
                                                        local_k_slice=ks, causal=True, return_attn_probs=True)
        out.backward(dog[mine].to(dev))
        spa.check_status()
        e = _errs([(out, ro[mine]), (lse, rl[:, mine]), (ql.grad, rdq[mine]), (kl.grad, rdk[mine]),
                   (vl.grad, rdv[mine])])
        gmax = max(1.0, float(max(rdq.abs().max(), rdk.abs().max(), rdv.abs().max())) / 4)
        res["llama3_packed_stream"] = (e[0] <= 2e-2 and e[1] <= 1e-3 and max(e[2:]) <= 2e-2 * gmax, e, e[1])

        # ---- BASELINE cfg2 at its stated size: bf16 B1 S=32768 H32 D128 causal over all ranks;
        # 64-row slices of out / lse / dq per rank against the oracle, dk / dv of the last 64
        # keys on the last rank, and the two checksum identities for dk / dv of every key
        B, S, H, D = 1, 32768, 32, 128
        sl = sl_of(S)
        lo, n = sl.start, sl.stop - sl.start
        gens = [torch.Generator().manual_seed(900 + i) for i in range(3)]
        qg, kg, vg = (torch.randn(B, S, H, D, generator=g).bfloat16() for g in gens)
        dog = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(903)).bfloat16()
        ql, kl, vl = (t[:, sl].to(dev).requires_grad_(True) for t in (qg, kg, vg))
        out, lse, _ = spa.sp_aurora_func(ql, kl, vl, causal=True, return_attn_probs=True)
        out.backward(dog[:, sl].to(dev))
        spa.check_status()
        errs = [0.0] * 5
        tol_g = 2e-2
        for r0 in (n // 2, n - 64):
            g0 = lo + r0
            rows = slice(r0, r0 + 64)
            ro, rl = orc.attention_ref(qg[:, g0:g0 + 64], kg[:, :g0 + 64], vg[:, :g0 + 64], None, True,
                                       causal_off=g0, dtype=torch.float32)
            rdq, rdk, rdv = orc.attention_bwd_ref(dog[:, g0:g0 + 64], qg[:, g0:g0 + 64], kg[:, :g0 + 64],
                                                  vg[:, :g0 + 64], ro, rl, None, True, causal_off=g0,
                                                  dtype=torch.float32)
            e = _errs([(out[:, rows], ro), (lse[:, :, rows], rl), (ql.grad[:, rows], rdq)])
            errs[:3] = [max(a, b) for a, b in zip(errs[:3], e)]
            tol_g = max(tol_g, 2e-2 * float(rdq.abs().max()) / 4)
            if rank == world - 1 and r0 == n - 64:
                e = _errs([(kl.grad[:, rows], rdk[:, g0:g0 + 64]), (vl.grad[:, rows], rdv[:, g0:g0 + 64])])
                errs[3:] = e
                tol_g = max(tol_g, 2e-2 * float(rdv[:, g0:g0 + 64].abs().max()) / 4)

        def sums(a, b):
            p = a.float() * b.float()
            return torch.stack((p.sum(dtype=torch.float64), p.abs().sum(dtype=torch.float64)))
        t = torch.stack((sums(ql.grad, ql), sums(kl.grad, kl), sums(vl.grad, vl), sums(dog[:, sl].to(dev), out)))
        dist.all_reduce(t)
        t = t.cpu()
        i1 = float((t[0, 0] - t[1, 0]).abs() / torch.maximum(t[0, 1], t[1, 1]))
        i2 = float((t[2, 0] - t[3, 0]).abs() / torch.maximum(t[2, 1], t[3, 1]))
        ok = errs[0] <= 2e-2 and errs[1] <= 1e-3 and max(errs[2:]) <= tol_g and i1 <= 1e-3 and i2 <= 1e-3
        res["cfg2_full_size"] = (ok, errs + [i1, i2], errs[1])
    except Exception:  # noqa: BLE001
        res["error"] = traceback.format_exc()
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.fixture(scope="module")
def results():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 8 if n >= 8 else 4 if n >= 4 else 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    out = {r: dict(ret[r]) for r in range(world)}
    for r in out:
        assert "error" not in out[r], out[r]["error"]
    return out


@pytest.mark.parametrize("tag", ["ring_fp32", "ring_bf16_gqa", "ring_bf16_gqa_contig", "ring_bf16_noncausal", "uly_b2",
                                 "uly_gqa_causal", "a2a_exact", "hyb_u", "hyb_r", "hyb_bwd", "hyb_u4r2",
                                 "run_twice_bitwise", "world_size_independence", "varlen_and_zigzag_layout",
                                 "llama3_packed_stream", "cfg2_full_size"])
def test_multi_gpu_parity(results, tag, error_log):
    for r, res in results.items():
        ok, errs, el = res[tag]
        error_log[f"dist {tag} rank{r}"] = {"errs": errs, "lse": el}
        assert ok, f"rank {r} {tag}: errs {errs} lse {el}"


def _rope_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from sp_aurora_b200 import high_priority_nccl_options
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            pg_options=high_priority_nccl_options())
    res = {}
    try:
        import sp_aurora_b200 as spa
        from sp_aurora_b200.all_to_all import heads_all_to_all_packed
        from oracle import attention_oracle as orc
        errs = []
        for B in (1, 2):
            S, hq, hkv, D = 64 * world, 2 * world, world, 64
            gens = [torch.Generator().manual_seed(1500 + i) for i in range(3)]
            qg = torch.randn(B, S, hq, D, generator=gens[0]).bfloat16()
            kg = torch.randn(B, S, hkv, D, generator=gens[1]).bfloat16()
            vg = torch.randn(B, S, hkv, D, generator=gens[2]).bfloat16()
            cos, sin = spa.rope_tables(S, D, device=dev)
            Sl = S // world
            sl = slice(rank * Sl, (rank + 1) * Sl)
            qo, ko, vo = heads_all_to_all_packed([t[:, sl].to(dev) for t in (qg, kg, vg)], None,
                                                 rope=(cos, sin, rank * Sl, 2))
            hs = lambda h: slice(rank * (h // world), (rank + 1) * (h // world))
            rq = orc.rope_ref(qg, cos.cpu(), sin.cpu(), 1, 0)[:, :, hs(hq)]
            rk = orc.rope_ref(kg, cos.cpu(), sin.cpu(), 1, 0)[:, :, hs(hkv)]
            errs += _errs([(qo, rq), (ko, rk)])
            errs.append(0.0 if torch.equal(vo.cpu(), vg[:, :, hs(hkv)]) else 1.0)   # v: plain permutation
        res["rope_pack"] = (max(errs) <= 2e-2, errs, 0.0)
    except Exception:  # noqa: BLE001
        import traceback
        res["error"] = traceback.format_exc()
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_rope_fused_into_the_ulysses_pack():
    """q and k rotated while they are packed for the sequence -> head all-to-all (one message,
    positions offset by the rank's first token); v is the plain permutation, bit-exact."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 4 if n >= 4 else 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rope_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        res = dict(ret[r])
        assert "error" not in res, res.get("error")
        ok, errs, _ = res["rope_pack"]
        assert ok, (r, errs)


def _mpi_launch_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    for v in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR"):
        os.environ.pop(v, None)
    # what `mpiexec -n <world>` (Open MPI) gives each process on one node
    os.environ.update(OMPI_COMM_WORLD_RANK=str(rank), OMPI_COMM_WORLD_SIZE=str(world),
                      OMPI_COMM_WORLD_LOCAL_RANK=str(rank), OMPI_COMM_WORLD_LOCAL_SIZE=str(world),
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    res = {}
    try:
        import sp_aurora_b200 as spa
        info = spa.setup_mpi_distributed()
        t = torch.full((4,), float(rank + 1), device=info["device"])
        dist.all_reduce(t)
        q = torch.randn(1, 256, 2, 64, device=info["device"]).bfloat16()
        out = spa.ring_flash_attn_func(q, q, q, causal=True)            # the ring over the new group
        spa.check_status()
        res = {"info": (info["rank"], info["world_size"], info["local_rank"], info["launcher"], info["backend"],
                        str(info["device"])), "sum": float(t[0].item()), "finite": bool(torch.isfinite(out).all())}
        spa.cleanup_distributed()
    except Exception:  # noqa: BLE001
        import traceback
        res["error"] = traceback.format_exc()
    ret[rank] = res


@pytest.mark.gpu
def test_mpi_style_launch_initialises_nccl():
    """setup_mpi_distributed (sp_aurora/mpi_utils.py:293 in the reference) from an Open MPI style
    environment: NCCL group bound to the rank's device, usable by the ring."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_mpi_launch_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        res = dict(ret[r])
        assert "error" not in res, res.get("error")
        assert res["info"] == (r, 2, r, "mpiexec", "nccl", f"cuda:{r}")
        assert res["sum"] == 3.0 and res["finite"]
