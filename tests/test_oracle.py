"""Pin the CPU oracle to outputs of the reference's own code (tests/golden/*.npz,
made by tests/golden/make_golden.py from the unmodified reference functions)."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc


@pytest.fixture(scope="module")
def local_npz(golden_dir):
    return np.load(os.path.join(golden_dir, "local_attention.npz"))


@pytest.fixture(scope="module")
def dist_npz(golden_dir):
    return np.load(os.path.join(golden_dir, "distributed.npz"))


@pytest.mark.parametrize("name", ["c0", "c1", "c2", "c3"])
def test_local_forward_matches_reference(local_npz, name):
    B, H, Sq, Sk, D, causal = [int(x) for x in local_npz[f"{name}_meta"]]
    q, k, v = (torch.from_numpy(local_npz[f"{name}_{t}"]) for t in "qkv")
    out, lse = orc.attention_ref(q, k, v, D ** -0.5, bool(causal))
    ref_out = torch.from_numpy(local_npz[f"{name}_out"]).double()
    ref_lse = torch.from_numpy(local_npz[f"{name}_lse"]).double()
    # the reference computes in fp32: its own error bounds the difference
    assert (out - ref_out).abs().max() < 5e-6
    assert (lse - ref_lse).abs().max() < 5e-6


def test_merge_matches_reference(local_npz):
    o1, o2 = torch.from_numpy(local_npz["m_out1"]), torch.from_numpy(local_npz["m_out2"])
    l1, l2 = torch.from_numpy(local_npz["m_lse1"]), torch.from_numpy(local_npz["m_lse2"])
    out, lse = orc.merge_ref(o1, l1, o2, l2)
    assert (out - torch.from_numpy(local_npz["m_out"]).double()).abs().max() < 5e-6
    assert (lse - torch.from_numpy(local_npz["m_lse"]).double()).abs().max() < 5e-6


def test_merge_step_function_equals_reference_formula(local_npz):
    """fwd_step_cpu's logaddexp form == the reference's sigmoid form."""
    o1, o2 = torch.from_numpy(local_npz["m_out1"]), torch.from_numpy(local_npz["m_out2"])
    l1, l2 = torch.from_numpy(local_npz["m_lse1"]), torch.from_numpy(local_npz["m_lse2"])
    want_out, want_lse = orc.merge_ref(o1, l1, o2, l2)
    mx = torch.maximum(l1, l2).double()
    s = torch.exp(l1.double() - mx) + torch.exp(l2.double() - mx)
    got_lse = mx + torch.log(s)
    w1 = (torch.exp(l1.double() - mx) / s).permute(0, 2, 1).unsqueeze(-1)
    got_out = w1 * o1.double() + (1 - w1) * o2.double()
    assert (got_lse - want_lse).abs().max() < 1e-12
    assert (got_out - want_out).abs().max() < 1e-12


def test_all_to_all_matches_reference(dist_npz):
    for tag, ref_fn, idx in (("a4", orc.all_to_all_4d_ref, (2, 1)), ("a5", orc.all_to_all_5d_ref, (3, 1))):
        ins = [torch.from_numpy(dist_npz[f"{tag}_in_rank{r}"]) for r in range(2)]
        fwd = ref_fn(ins, *idx)
        for r in range(2):
            assert torch.equal(fwd[r], torch.from_numpy(dist_npz[f"{tag}_fwd_rank{r}"]))
        back = ref_fn(fwd, idx[1], idx[0])
        for r in range(2):
            assert torch.equal(back[r], torch.from_numpy(dist_npz[f"{tag}_back_rank{r}"]))
            assert torch.equal(back[r], ins[r])


@pytest.mark.parametrize("name", ["r0", "r1"])
def test_ring_forward_matches_reference(dist_npz, name):
    """Per-rank slices of the full-sequence oracle == the reference's ring forward
    (run over gloo ranks in its own [B,H,S,D] layout)."""
    B, H, S, D, causal, W = [int(x) for x in dist_npz[f"{name}_meta"]]
    q, k, v = (torch.from_numpy(dist_npz[f"{name}_{t}"]) for t in "qkv")
    out, lse = orc.attention_ref(q, k, v, D ** -0.5, bool(causal))
    sl = S // W
    for r in range(W):
        ref_out = torch.from_numpy(dist_npz[f"{name}_out_rank{r}"]).double()
        ref_lse = torch.from_numpy(dist_npz[f"{name}_lse_rank{r}"]).double()
        assert (out[:, r * sl:(r + 1) * sl] - ref_out).abs().max() < 5e-6
        assert (lse[:, :, r * sl:(r + 1) * sl] - ref_lse).abs().max() < 5e-6


@pytest.mark.parametrize("causal,hq,hkv", [(True, 4, 4), (False, 4, 2), (True, 6, 2)])
def test_backward_oracle_matches_autograd(causal, hq, hkv):
    """No reference output exists for backward/GQA: check the closed-form
    gradients against autograd through the forward oracle."""
    g = torch.Generator().manual_seed(5)
    B, Sq, Sk, D = 2, 48, 48, 16
    q = torch.randn(B, Sq, hq, D, generator=g, dtype=torch.float64, requires_grad=True)
    k = torch.randn(B, Sk, hkv, D, generator=g, dtype=torch.float64, requires_grad=True)
    v = torch.randn(B, Sk, hkv, D, generator=g, dtype=torch.float64, requires_grad=True)
    dout = torch.randn(B, Sq, hq, D, generator=g, dtype=torch.float64)
    rep = hq // hkv
    scores = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(rep, 2)) * D ** -0.5
    if causal:
        scores = scores.masked_fill(torch.triu(torch.ones(Sq, Sk, dtype=torch.bool), 1), float("-inf"))
    out = torch.einsum("bhqk,bkhd->bqhd", scores.softmax(-1), v.repeat_interleave(rep, 2))
    out.backward(dout)
    o2, lse = orc.attention_ref(q.detach(), k.detach(), v.detach(), None, causal)
    assert (o2 - out.detach()).abs().max() < 1e-12
    dq, dk, dv = orc.attention_bwd_ref(dout, q.detach(), k.detach(), v.detach(), o2, lse, None, causal)
    assert (dq - q.grad).abs().max() < 1e-11
    assert (dk - k.grad).abs().max() < 1e-11
    assert (dv - v.grad).abs().max() < 1e-11


def test_causal_offset_and_empty_rows():
    """Rows with no visible key: out = 0, lse = -inf (negative causal offset)."""
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 8, 1, 16, generator=g)
    k = torch.randn(1, 8, 1, 16, generator=g)
    v = torch.randn(1, 8, 1, 16, generator=g)
    out, lse = orc.attention_ref(q, k, v, None, True, causal_off=-3)
    assert torch.isinf(lse[0, 0, :3]).all() and (out[0, :3] == 0).all()
    assert torch.isfinite(lse[0, 0, 3:]).all()
