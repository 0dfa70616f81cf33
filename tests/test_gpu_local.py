"""GPU parity tests of the per-device kernels against the CPU oracle.

Tolerances (max-abs), as the build's parity contract states them:
  bf16/fp16: out, dq, dk, dv <= 2e-2 ; fp32: <= 1e-4 ; lse <= 1e-3.
Everything is called through the C-ABI library (ctypes)."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}
LSE_TOL = 1e-3


@pytest.fixture(scope="module")
def spa():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import sp_aurora_b200 as m
    return m


def _rand(shape, dtype, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def _check_fwd(spa, B, Sq, Sk, Hq, Hkv, D, dtype, causal, seed=0):
    q = _rand((B, Sq, Hq, D), dtype, seed)
    k = _rand((B, Sk, Hkv, D), dtype, seed + 1)
    v = _rand((B, Sk, Hkv, D), dtype, seed + 2)
    out, lse = spa.flash_attn_forward(q.cuda(), k.cuda(), v.cuda(), None, causal)
    spa.check_status()
    ref_out, ref_lse = orc.attention_ref(q, k, v, None, causal)
    eo = (out.cpu().double() - ref_out).abs().max().item()
    el = (lse.cpu().double() - ref_lse).abs().max().item()
    assert eo <= TOL[dtype], f"out err {eo}"
    assert el <= LSE_TOL, f"lse err {el}"
    return q, k, v, out, lse, ref_out, ref_lse


def grad_tol(dtype, want):
    """Gradient bound: the stated max-abs tolerance while |gradient| <= 4. A 16-bit output
    of magnitude x carries a rounding error of up to x * 2^-9 on its own, which passes 2e-2
    at x ~ 10, so beyond 4 the bound grows in proportion (2e-2 * max|ref| / 4)."""
    return TOL[dtype] * max(1.0, want.abs().max().item() / 4)


def _check_bwd(spa, q, k, v, out, lse, ref_out, ref_lse, dtype, causal, seed=0, record=None):
    dout = _rand(tuple(q.shape), dtype, seed + 3)
    dq, dk, dv = spa.flash_attn_backward(dout.cuda(), q.cuda(), k.cuda(), v.cuda(), out, lse, None, causal)
    spa.check_status()
    rdq, rdk, rdv = orc.attention_bwd_ref(dout, q, k, v, ref_out, ref_lse, None, causal)
    for name, got, want in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        err = (got.cpu().double() - want).abs().max().item()
        if record is not None:
            record[name] = (err, want.abs().max().item())
        assert err <= grad_tol(dtype, want), f"{name} err {err} (max |ref| {want.abs().max().item()})"


# fp32 runs on the CUDA-core kernel: reference-test shapes (D 32/64/128, ragged, GQA)
FP32_CASES = [
    (1, 128, 128, 2, 2, 64, True), (1, 96, 160, 2, 2, 32, False), (2, 200, 200, 1, 1, 128, True),
    (1, 64, 64, 3, 3, 64, False), (2, 130, 77, 4, 2, 64, False), (1, 257, 257, 4, 1, 128, True),
]


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D,causal", FP32_CASES)
def test_fp32_forward_backward(spa, B, Sq, Sk, Hq, Hkv, D, causal):
    r = _check_fwd(spa, B, Sq, Sk, Hq, Hkv, D, torch.float32, causal)
    _check_bwd(spa, *r, torch.float32, causal)


# bf16 / fp16 run on the tcgen05 kernels
TC_CASES = [
    (1, 128, 128, 1, 1, 128, False), (1, 256, 256, 2, 2, 128, True), (2, 384, 384, 4, 2, 128, True),
    (1, 512, 512, 4, 1, 128, False), (1, 300, 300, 2, 2, 128, True), (1, 130, 333, 2, 1, 128, False),
    (1, 1024, 1024, 2, 2, 128, True), (1, 64, 64, 2, 2, 128, True), (2, 256, 256, 2, 2, 64, True),
    (1, 200, 200, 4, 2, 64, False),
]


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D,causal", TC_CASES)
def test_bf16_forward_backward(spa, B, Sq, Sk, Hq, Hkv, D, causal, error_log):
    r = _check_fwd(spa, B, Sq, Sk, Hq, Hkv, D, torch.bfloat16, causal)
    rec = {}
    _check_bwd(spa, *r, torch.bfloat16, causal, record=rec)
    error_log[f"bf16 B{B} Sq{Sq} Sk{Sk} Hq{Hq} Hkv{Hkv} D{D} causal{int(causal)}"] = {
        k: {"err": e, "max_ref": m, "strict_2e-2": e <= 2e-2} for k, (e, m) in rec.items()}


def test_backward_is_bitwise_reproducible(spa):
    """Every dq, dk and dv row has one owning CTA and a fixed summation order: two runs on
    the same inputs give identical bits (also with deterministic=True, which only forbids
    the split of a K/V tile's queries between CTAs in the fp32-gradient ring steps)."""
    from sp_aurora_b200 import local_attn as la
    B, S, Hq, Hkv, D = 1, 2048, 8, 2, 128
    q, k, v, do = (_rand(sh, torch.bfloat16, s).cuda() for sh, s in (
        ((B, S, Hq, D), 1), ((B, S, Hkv, D), 2), ((B, S, Hkv, D), 3), ((B, S, Hq, D), 4)))
    out, lse = spa.flash_attn_forward(q, k, v, None, True)
    out2, lse2 = spa.flash_attn_forward(q, k, v, None, True)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    a = spa.flash_attn_backward(do, q, k, v, out, lse, None, True)
    b = spa.flash_attn_backward(do, q, k, v, out, lse, None, True, deterministic=True)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    # ring-step form: fp32 dK/dV partials, non-causal, small grid (the query split would
    # apply): deterministic=True must give identical bits on two runs
    delta = la.bwd_delta(out, do)
    res = []
    for _ in range(2):
        dq_acc = torch.empty(B, S, Hq, D, device="cuda")
        dk = torch.empty(B, S, Hkv, D, device="cuda")
        dv = torch.empty_like(dk)
        la.attn_bwd_step(q, k, v, do, lse, delta, D ** -0.5, False, dq_acc, dk, dv,
                         dq_overwrite=True, deterministic=True)
        res.append((dq_acc, dk, dv))
    spa.check_status()
    for x, y in zip(*res):
        assert torch.equal(x, y)


def test_strided_lse_and_gradient_outputs(spa):
    """lse/delta with a head stride (rows of a [B,Hq,2,h] tensor) and dq/dk/dv written
    into head slices of one packed buffer give the same bits as contiguous tensors."""
    from sp_aurora_b200 import local_attn as la
    B, S, Hq, Hkv, D = 1, 512, 4, 2, 128
    q, k, v, do = (_rand(sh, torch.bfloat16, s).cuda() for sh, s in (
        ((B, S, Hq, D), 5), ((B, S, Hkv, D), 6), ((B, S, Hkv, D), 7), ((B, S, Hq, D), 8)))
    out, lse = spa.flash_attn_forward(q, k, v, None, True)
    want = spa.flash_attn_backward(do, q, k, v, out, lse, None, True)
    wide = torch.empty(B, Hq, 2, S, device="cuda")
    lse_v = wide[:, :, 1]
    out2 = torch.empty_like(out)
    la.attn_fwd_step(q, k, v, D ** -0.5, True, lse_v, out=out2)
    assert torch.equal(out2, out) and torch.equal(lse_v, lse)
    grads = torch.empty(B, S, Hq + 2 * Hkv, D, dtype=torch.bfloat16, device="cuda")
    dq, dk, dv = grads[:, :, :Hq], grads[:, :, Hq:Hq + Hkv], grads[:, :, Hq + Hkv:]
    delta = torch.empty(B, Hq, 2, S, device="cuda")
    delta[:, :, 1] = la.bwd_delta(out, do)
    la.attn_bwd_step(q, k, v, do, lse_v, delta[:, :, 1], D ** -0.5, True, None, dk, dv,
                     dq=dq, dq_overwrite=True)
    spa.check_status()
    for got, ref in zip((dq, dk, dv), want):
        assert torch.equal(got, ref)


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D,causal", TC_CASES[:4])
def test_fp16_forward_backward(spa, B, Sq, Sk, Hq, Hkv, D, causal):
    r = _check_fwd(spa, B, Sq, Sk, Hq, Hkv, D, torch.float16, causal)
    _check_bwd(spa, *r, torch.float16, causal)


def test_golden_fixtures_on_gpu(spa, golden_dir):
    """The reference's own outputs (fp32) reproduced by the CUDA path."""
    gd = np.load(os.path.join(golden_dir, "local_attention.npz"))
    for name in ("c0", "c1", "c2", "c3"):
        B, H, Sq, Sk, D, causal = [int(x) for x in gd[f"{name}_meta"]]
        q, k, v = (torch.from_numpy(gd[f"{name}_{t}"]).cuda() for t in "qkv")
        out, lse = spa.flash_attn_forward(q, k, v, D ** -0.5, bool(causal))
        assert (out.cpu() - torch.from_numpy(gd[f"{name}_out"])).abs().max() <= 1e-4
        assert (lse.cpu() - torch.from_numpy(gd[f"{name}_lse"])).abs().max() <= 1e-3
    o1, o2 = torch.from_numpy(gd["m_out1"]).cuda(), torch.from_numpy(gd["m_out2"]).cuda()
    l1, l2 = torch.from_numpy(gd["m_lse1"]).cuda(), torch.from_numpy(gd["m_lse2"]).cuda()
    out, lse = spa.update_out_and_lse(None, None, o1, l1)
    out, lse = spa.update_out_and_lse(out, lse, o2, l2)
    assert (out.cpu() - torch.from_numpy(gd["m_out"])).abs().max() <= 1e-5
    assert (lse.cpu() - torch.from_numpy(gd["m_lse"])).abs().max() <= 1e-5
    # slice_ (sp_aurora/utils.py:123-128): the second block merged into a row range only
    S = o1.shape[1]
    sl = slice(S // 4, S // 2)
    out_s, lse_s = spa.update_out_and_lse(None, None, o1, l1)
    keep_o, keep_l = out_s.clone(), lse_s.clone()
    out_s, lse_s = spa.update_out_and_lse(out_s, lse_s, o2[:, sl].contiguous(), l2[:, :, sl].contiguous(),
                                          slice_=sl)
    assert torch.equal(out_s[:, sl], out[:, sl]) and torch.equal(lse_s[:, :, sl], lse[:, :, sl])
    rest = torch.ones(S, dtype=torch.bool)
    rest[sl] = False
    assert torch.equal(out_s[:, rest], keep_o[:, rest]) and torch.equal(lse_s[:, :, rest], keep_l[:, :, rest])
    with pytest.raises(RuntimeError):
        spa.update_out_and_lse(None, None, o1, l1, slice_=sl)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_merge_equals_full_attention(spa, dtype):
    """Two key blocks through the fused merge epilogue == one call over all keys."""
    from sp_aurora_b200.local_attn import attn_fwd_step
    B, S, H, D = 1, 256, 2, 128
    q, k, v = (_rand((B, S, H, D), dtype, s).cuda() for s in (1, 2, 3))
    lse = torch.empty((B, H, S), dtype=torch.float32, device="cuda")
    acc = torch.empty((B, S, H, D), dtype=torch.float32, device="cuda")
    out = torch.empty((B, S, H, D), dtype=dtype, device="cuda")
    attn_fwd_step(q, k[:, :128], v[:, :128], D ** -0.5, False, lse, out_acc=acc)
    attn_fwd_step(q, k[:, 128:], v[:, 128:], D ** -0.5, False, lse, out=out, out_acc=acc, merge_prev=True)
    spa.check_status()
    ref_out, ref_lse = orc.attention_ref(q.cpu(), k.cpu(), v.cpu(), None, False)
    assert (out.cpu().double() - ref_out).abs().max() <= TOL[dtype]
    assert (lse.cpu().double() - ref_lse).abs().max() <= LSE_TOL


def test_causal_offset_rows_without_keys(spa):
    from sp_aurora_b200.local_attn import attn_fwd_step
    B, S, H, D = 1, 256, 1, 128
    q, k, v = (_rand((B, S, H, D), torch.bfloat16, s).cuda() for s in (4, 5, 6))
    lse = torch.empty((B, H, S), dtype=torch.float32, device="cuda")
    out = torch.empty_like(q)
    attn_fwd_step(q, k, v, D ** -0.5, True, lse, out=out, causal_off=-130)
    spa.check_status()
    ref_out, ref_lse = orc.attention_ref(q.cpu(), k.cpu(), v.cpu(), None, True, causal_off=-130)
    assert torch.isinf(lse[0, 0, :130]).all() and (out[0, :130] == 0).all()
    assert (out.cpu().double() - ref_out).abs().max() <= 2e-2
    assert (lse.cpu().double()[0, 0, 130:] - ref_lse[0, 0, 130:]).abs().max() <= LSE_TOL


def test_packed_views_equal_separate_tensors(spa):
    """kv[:, :, 0] / qkv[:, :, i] views are consumed in place (strided TMA)."""
    B, S, H, D = 1, 256, 2, 128
    qkv = _rand((B, S, 3, H, D), torch.bfloat16, 9).cuda()
    o1, l1 = spa.flash_attn_forward(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], None, True)
    o2, l2 = spa.flash_attn_forward(qkv[:, :, 0].contiguous(), qkv[:, :, 1].contiguous(),
                                    qkv[:, :, 2].contiguous(), None, True)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


def test_strided_copy_bit_exact(spa):
    from sp_aurora_b200.all_to_all import strided_copy
    x = torch.arange(2 * 6 * 4 * 3 * 64, dtype=torch.float32).view(2, 6, 4, 3, 64).to(torch.bfloat16).cuda()
    src = x.permute(2, 0, 1, 3, 4)
    dst = torch.empty(src.shape, dtype=x.dtype, device="cuda")
    strided_copy(dst, src)
    assert torch.equal(dst, src.contiguous())


def test_large_shape_against_cuda_core_kernel(spa):
    """S = 4096, GQA, causal: tensor-core kernels vs the fp32 CUDA-core kernels
    on the same bf16 data (size-independent cross-check, both on the GPU), plus a
    CPU oracle spot check on a slice of the rows."""
    B, S, Hq, Hkv, D = 1, 4096, 8, 2, 128
    dt = torch.bfloat16
    q, k, v, dout = (_rand(sh, dt, s, 1.0).cuda() for sh, s in (
        ((B, S, Hq, D), 1), ((B, S, Hkv, D), 2), ((B, S, Hkv, D), 3), ((B, S, Hq, D), 4)))
    out, lse = spa.flash_attn_forward(q, k, v, None, True)
    dq, dk, dv = spa.flash_attn_backward(dout, q, k, v, out, lse, None, True)
    spa.check_status()
    o32, l32 = spa.flash_attn_forward(q.float(), k.float(), v.float(), None, True)
    g32 = spa.flash_attn_backward(dout.float(), q.float(), k.float(), v.float(), o32, l32, None, True)
    assert (out.float() - o32).abs().max() <= 2e-2
    assert (lse - l32).abs().max() <= 1e-3
    for got, want in zip((dq, dk, dv), g32):
        assert (got.float() - want).abs().max() <= 2e-2 * max(1.0, want.abs().max().item() / 4)
    rows = slice(3000, 3128)
    ro, rl = orc.attention_ref(q[:, rows].cpu(), k.cpu(), v.cpu(), None, True, causal_off=3000)
    assert (out[:, rows].cpu().double() - ro).abs().max() <= 2e-2
    assert (lse[:, :, rows].cpu().double() - rl).abs().max() <= 1e-3


_QSPLIT_CODE = r"""
import os, sys, torch
sys.path.insert(0, %r)
import sp_aurora_b200 as spa
from sp_aurora_b200 import local_attn as la
from oracle import attention_oracle as orc
g = torch.Generator().manual_seed(11)
worst = 0.0
for (Sq, Sk, Hq, Hkv, causal, off, D) in ((1024, 1024, 4, 2, True, 0, 128), (1000, 700, 4, 1, False, 0, 128),
                                          (1024, 512, 2, 2, True, 256, 128), (2048, 2048, 2, 1, True, 0, 128),
                                          (512, 1024, 2, 2, True, 0, 128),   # last K/V tiles see no query
                                          (1024, 1024, 4, 2, True, 0, 64), (1000, 700, 2, 1, False, 0, 64)):
    q, do = (torch.randn(1, Sq, Hq, D, generator=g).bfloat16() for _ in range(2))
    k, v = (torch.randn(1, Sk, Hkv, D, generator=g).bfloat16() for _ in range(2))
    ro, rl = orc.attention_ref(q, k, v, None, causal, causal_off=off)
    rdq, rdk, rdv = orc.attention_bwd_ref(do, q, k, v, ro, rl, None, causal, causal_off=off)
    qc, kc, vc, dc = (t.cuda() for t in (q, k, v, do))
    lse = rl.float().cuda()
    delta = la.bwd_delta(ro.to(torch.bfloat16).cuda(), dc)
    for accumulate in (False, True):
        dq = torch.zeros(1, Sq, Hq, D, device="cuda")
        base = 0.5 if accumulate else float("nan")      # overwrite mode must ignore old contents
        dk = torch.full((1, Sk, Hkv, D), base, device="cuda")
        dv = torch.full((1, Sk, Hkv, D), base, device="cuda")
        la.attn_bwd_step(qc, kc, vc, dc, lse, delta, D ** -0.5, causal, dq, dk, dv,
                         dkv_accumulate=accumulate, causal_off=off)
        spa.check_status()
        add = 0.5 if accumulate else 0.0
        errs = [float((dq.cpu().double() - rdq).abs().max()),
                float((dk.cpu().double() - add - rdk).abs().max()),
                float((dv.cpu().double() - add - rdv).abs().max())]
        lim = 2e-2 * max(1.0, float(rdv.abs().max()) / 4)
        assert max(errs) <= lim, (Sq, Sk, causal, off, D, accumulate, errs)
        worst = max(worst, max(errs))
print("ok", worst)
"""


@pytest.mark.parametrize("split", ["1", "2", "8", "auto"])
def test_backward_query_split_in_subprocess(split):
    """Backward with the query tiles of a K/V tile shared by several CTAs (fp32 dK/dV
    added atomically; SPA_BWD_QSPLIT is read once per process): overwrite and
    accumulate modes, ragged and offset-causal shapes, against the CPU oracle."""
    import subprocess
    import sys
    code = _QSPLIT_CODE % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ)
    env.pop("SPA_BWD_QSPLIT", None)
    if split != "auto":
        env["SPA_BWD_QSPLIT"] = split
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr


def test_long_sequence_slices_against_oracle(spa):
    """S = 65536 causal GQA: the sizes at which both kernels switch to the
    all-tiles-of-a-head work order. Row slices of out / lse / dq and the last key
    tile of dk / dv are checked against the CPU oracle run on those rows only
    (causal_off places the slice inside the full sequence)."""
    B, S, Hq, Hkv, D = 1, 65536, 8, 2, 128
    dt = torch.bfloat16
    q, k, v, dout = (_rand(sh, dt, s, 0.5) for sh, s in (
        ((B, S, Hq, D), 11), ((B, S, Hkv, D), 12), ((B, S, Hkv, D), 13), ((B, S, Hq, D), 14)))
    qc, kc, vc, dc = (t.cuda() for t in (q, k, v, dout))
    out, lse = spa.flash_attn_forward(qc, kc, vc, None, True)
    dq, dk, dv = spa.flash_attn_backward(dc, qc, kc, vc, out, lse, None, True)
    spa.check_status()
    for r0 in (30000, S - 128):
        rows = slice(r0, r0 + 128)
        ro, rl = orc.attention_ref(q[:, rows], k, v, None, True, causal_off=r0)
        assert (out[:, rows].cpu().double() - ro).abs().max() <= 2e-2
        assert (lse[:, :, rows].cpu().double() - rl).abs().max() <= 1e-3
        rdq, rdk, rdv = orc.attention_bwd_ref(dout[:, rows], q[:, rows], k, v, ro, rl, None, True,
                                              causal_off=r0)
        lim = 2e-2 * max(1.0, float(rdv.abs().max()) / 4)
        assert (dq[:, rows].cpu().double() - rdq).abs().max() <= lim
        if r0 == S - 128:   # only these rows see the last 128 keys: their dk/dv are complete
            assert (dk[:, rows].cpu().double() - rdk[:, rows]).abs().max() <= lim
            assert (dv[:, rows].cpu().double() - rdv[:, rows]).abs().max() <= lim


def test_bounded_wait_gives_up_and_reports(spa):
    """A device-side wait on a barrier that nothing arrives at runs out of its cycle budget:
    the kernel returns normally, spa_check_status() reports SPA_ETIMEOUT with the site and
    iteration of the wait, the status word is cleared by that read, and the next attention
    call on the same context is correct."""
    import ctypes as C
    from sp_aurora_b200 import _lib
    fn = _lib.lib.spa_internal_wait_selftest
    fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_void_p]
    spa.check_status()                                   # clean before
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert fn(flag.data_ptr(), _lib.stream_ptr(flag.device)) == 0
    torch.cuda.synchronize()                             # the kernel ended by itself
    assert int(flag.item()) == 1                         # ... after its wait gave up
    with pytest.raises(_lib.SpaError, match="site 99 iteration 7"):
        spa.check_status()
    spa.check_status()                                   # the read cleared the word
    _check_fwd(spa, 1, 256, 256, 2, 2, 128, torch.bfloat16, True)


@pytest.mark.parametrize("rope_base", [None, 10000.0])
def test_attention_block_matches_a_torch_reference(spa, rope_base):
    """QKV projection -> attention -> output projection (the reference's example model shape,
    examples/example_mpi_integration.py:38-86) on one GPU, GQA, against the same block computed
    with the CPU oracle between fp32 copies of the same projections; gradients of x included.
    With rope_base, q and k are rotated between the projection and the attention."""
    torch.manual_seed(0)
    B, S, d_model, hq, hkv = 1, 384, 512, 4, 2
    D = d_model // hq
    blk = spa.SequenceParallelAttentionBlock(d_model, hq, hkv, mode="ring", device="cuda", rope_base=rope_base)
    x = (torch.randn(B, S, d_model) * 0.5).bfloat16()
    dy = (torch.randn(B, S, d_model) * 0.5).bfloat16()
    xc = x.cuda().requires_grad_(True)
    y = blk(xc, causal=True)
    y.backward(dy.cuda())
    spa.check_status()
    wq = blk.qkv_proj.weight.detach().cpu().double()
    wo = blk.out_proj.weight.detach().cpu().double()
    xr = x.double().requires_grad_(True)
    qkv = (xr @ wq.t()).view(B, S, hq + 2 * hkv, D)
    q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
    if rope_base is not None:
        cos, sin = spa.rope_tables(S, D, rope_base)
        q, k = orc.rope_ref(q, cos, sin, 1, 0), orc.rope_ref(k, cos, sin, 1, 0)
    g = hq // hkv
    qt = q.permute(0, 2, 1, 3)
    kt = k.permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vt = v.permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    sc = torch.matmul(qt, kt.transpose(-2, -1)) * D ** -0.5
    sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), diagonal=1), float("-inf"))
    o = torch.matmul(torch.softmax(sc, -1), vt).permute(0, 2, 1, 3).reshape(B, S, d_model)
    yr = o @ wo.t()
    yr.backward(dy.double())
    assert (y.detach().cpu().double() - yr.detach()).abs().max() <= 3e-2     # two bf16 GEMM roundings on top
    assert (xc.grad.cpu().double() - xr.grad).abs().max() <= 3e-2 * max(1.0, float(xr.grad.abs().max()) / 4)


@pytest.mark.parametrize("lengths", [[128, 256, 128], [100, 100, 100, 100], [512], [64, 128, 256, 512]])
def test_varlen_packed_sequences(spa, lengths):
    """Packed variable-length sequences (the shapes of the reference's
    test/flash_attention/test_intel_ring_flash_attn_varlen.py:37-77: fp16, 8 heads, D=64, causal),
    forward and backward, each sequence against the oracle; the zigzag variant on one rank is the
    same computation."""
    H, D = 8, 64
    total = sum(lengths)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    q, k, v, do = (_rand((total, H, D), torch.float16, s_) for s_ in (31, 32, 33, 34))
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out, lse, _ = spa.sp_aurora_varlen_func(qc, kc, vc, cu.cuda(), cu.cuda(), max_seqlen=max(lengths),
                                            dropout_p=0.0, causal=True, return_attn_probs=True)
    assert out.shape == (total, H, D) and lse.shape == (H, total)
    out.backward(do.cuda())
    out2 = spa.zigzag_sp_aurora_varlen_func(qc.detach(), kc.detach(), vc.detach(), cu.cuda(), cu.cuda(),
                                            max_seqlen=max(lengths), causal=True)
    spa.check_status()
    assert torch.equal(out2, out.detach())
    for i in range(len(lengths)):
        sl = slice(int(cu[i]), int(cu[i + 1]))
        ro, rl = orc.attention_ref(q[None, sl], k[None, sl], v[None, sl], None, True)
        rdq, rdk, rdv = orc.attention_bwd_ref(do[None, sl], q[None, sl], k[None, sl], v[None, sl], ro, rl,
                                              None, True)
        assert (out[sl].detach().cpu().double() - ro[0]).abs().max() <= 2e-2
        assert (lse[:, sl].cpu().double() - rl[0]).abs().max() <= 1e-3
        for got, want in ((qc.grad[sl], rdq[0]), (kc.grad[sl], rdk[0]), (vc.grad[sl], rdv[0])):
            assert (got.cpu().double() - want).abs().max() <= grad_tol(torch.float16, want)


@pytest.mark.gpu
def test_llama3_packed_stream_one_rank(spa):
    """llama3_flash_attn_varlen_func on one rank (the all-gather is the identity): GQA, kv heads
    two at a time, bf16, sequences of ragged lengths, forward and backward vs the oracle; strided
    out / lse / dq views and fp32 dK/dV buffers are what the multi-rank path uses too."""
    lengths = [300, 1, 515, 0, 208]
    H, Hkv, D = 8, 4, 128
    T = sum(lengths)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    q, do = (_rand((T, H, D), torch.bfloat16, s_) for s_ in (41, 44))
    k, v = (_rand((T, Hkv, D), torch.bfloat16, s_) for s_ in (42, 43))
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    cq, ck, mq, mk, ks = spa.llama3_flash_attn_prepare_cu_seqlens(cu, True, 0, 1)
    assert ks == slice(0, T) and mq == 515
    out, lse, _ = spa.llama3_flash_attn_varlen_func(qc, kc, vc, cq, ck, mq, mk, heads_k_stride=2,
                                                    local_k_slice=ks, causal=True, return_attn_probs=True)
    out.backward(do.cuda())
    spa.check_status()
    assert out.shape == (T, H, D) and lse.shape == (H, T)
    for a, b in zip(cu, cu[1:]):
        if a == b:
            continue
        sl = slice(a, b)
        ro, rl = orc.attention_ref(q[None, sl], k[None, sl], v[None, sl], None, True)
        rdq, rdk, rdv = orc.attention_bwd_ref(do[None, sl], q[None, sl], k[None, sl], v[None, sl], ro, rl,
                                              None, True)
        assert (out[sl].detach().cpu().double() - ro[0]).abs().max() <= 2e-2
        assert (lse[:, sl].cpu().double() - rl[0]).abs().max() <= 1e-3
        for got, want in ((qc.grad[sl], rdq[0]), (kc.grad[sl], rdk[0]), (vc.grad[sl], rdv[0])):
            assert (got.cpu().double() - want).abs().max() <= grad_tol(torch.bfloat16, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rope_copy_matches_the_formula(spa, dtype):
    """spa_rope_rows: rotated copy into a strided destination (the head slice of a packed
    message), a position offset, the inverse rotation, and the autograd form."""
    B, S, H, D, off = 2, 96, 4, 128, 37
    cos, sin = spa.rope_tables(off + S, D, device="cuda")
    x = _rand((B, S, H, D), dtype, 51)
    ref = orc.rope_ref(x, cos.cpu(), sin.cpu(), 1, off)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    # into head slice [2, 6) of a wider buffer, sequence-major like the all-to-all message
    wide = torch.zeros(B, S, 10, D, dtype=dtype, device="cuda")
    spa.rope_copy(wide[:, :, 2:6], x.cuda(), cos, sin, 1, off)
    assert (wide[:, :, 2:6].cpu().double() - ref).abs().max() <= tol
    assert wide[:, :, :2].abs().max() == 0 and wide[:, :, 6:].abs().max() == 0
    # permuted source view: positions along dim 2 of a [H, B, S, D] view
    y = torch.empty(H, B, S, D, dtype=dtype, device="cuda")
    spa.rope_copy(y, x.cuda().permute(2, 0, 1, 3), cos, sin, 2, off)
    assert (y.permute(1, 2, 0, 3).cpu().double() - ref).abs().max() <= tol
    # the inverse rotation undoes it (up to the rounding of the intermediate)
    back = spa.rope_copy(torch.empty_like(y), y, cos, sin, 2, off, inverse=True)
    assert (back.permute(1, 2, 0, 3).cpu().double() - x.double()).abs().max() <= 2 * tol
    # autograd: gradient = inverse rotation of the incoming gradient
    xg = x.cuda().requires_grad_(True)
    g = _rand((B, S, H, D), dtype, 52)
    spa.apply_rope(xg, cos, sin, pos_offset=off).backward(g.cuda())
    want = orc.rope_ref(g, cos.cpu(), sin.cpu(), 1, off, inverse=True)
    assert (xg.grad.cpu().double() - want).abs().max() <= tol
    with pytest.raises(spa.SpaError):            # positions beyond the tables are refused
        spa.rope_copy(torch.empty_like(y), y, cos, sin, 2, off + 1)
