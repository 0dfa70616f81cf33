"""The allocation-free backward entry point (spa_attn_bwd_noalloc), for callers
that cannot allocate device memory: its results must equal the regular
backward entry point's and the CPU oracle's, on two calls in a row (the shared
built-in scratch is reused), and the calls must not change the amount of free
device memory. Collected last so that a failure here cannot hide another test."""
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _rand(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_backward_matches_regular_entry_point_twice(dtype):
    import sp_aurora_b200 as spa
    from sp_aurora_b200 import no_alloc
    B, Sq, Sk, Hq, Hkv, D = 2, 320, 320, 4, 2, 128
    dq = torch.empty((B, Sq, Hq, D), dtype=dtype, device="cuda")
    dk = torch.empty((B, Sk, Hkv, D), dtype=dtype, device="cuda")
    dv = torch.empty_like(dk)
    for call in range(2):                      # two calls in a row, different data
        hq = _rand((B, Sq, Hq, D), dtype, 10 + call)
        hk = _rand((B, Sk, Hkv, D), dtype, 20 + call)
        hv = _rand((B, Sk, Hkv, D), dtype, 30 + call)
        hdo = _rand((B, Sq, Hq, D), dtype, 40 + call)
        q, k, v, dout = hq.cuda(), hk.cuda(), hv.cuda(), hdo.cuda()
        out, lse = spa.flash_attn_forward(q, k, v, None, True)
        want = spa.flash_attn_backward(dout, q, k, v, out, lse, None, True)
        ro, rl = orc.attention_ref(hq, hk, hv, None, True)
        oracle = orc.attention_bwd_ref(hdo, hq, hk, hv, ro, rl, None, True)
        torch.cuda.synchronize()
        if call == 1:
            free_before = torch.cuda.mem_get_info()[0]
            torch_before = torch.cuda.memory_allocated()
        no_alloc.flash_attn_backward_noalloc(dout, q, k, v, out, lse, dq, dk, dv, None, True)
        torch.cuda.synchronize()
        if call == 1:                          # the first call did the one-time set-up
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.cuda.memory_allocated() == torch_before
        spa.check_status()
        for name, got, ref, ora in zip(("dq", "dk", "dv"), (dq, dk, dv), want, oracle):
            # same kernels, same fixed summation order: the two entry points agree bit for bit
            assert torch.equal(got, ref), f"call {call} {name}: differs from spa_attn_bwd"
            err = (got.cpu().double() - ora).abs().max().item()
            lim = TOL[dtype] * max(1.0, ora.abs().max().item() / 4)
            assert err <= lim, f"call {call} {name}: {err} > {lim} against the oracle"


def test_noalloc_rejects_problems_beyond_the_scratch():
    from sp_aurora_b200 import _lib, no_alloc
    assert no_alloc.scratch_bytes() == 16 << 20
    B, S, H, D = 1, 70000, 64, 32              # needs 70000*64*4 B = 17.9 MB > 16 MiB
    q = torch.empty((B, S, H, D), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty((B, H, S), dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.SpaError, match="scratch"):
        no_alloc.flash_attn_backward_noalloc(q, q, q, q, q, lse, torch.empty_like(q),
                                             torch.empty_like(q), torch.empty_like(q))
