"""Generate tests/golden/*.npz by running the UNMODIFIED reference functions.

Run in the build container only (needs the reference tree; pass its path):

    python tests/golden/make_golden.py /path/to/sp-aurora

The reference imports intel_extension_for_pytorch and raises without an XPU, so
it is loaded with an empty stub for that module and with the package object
pointed at the source directory (its __init__.py is never executed); the ring
forward additionally gets `device='xpu'` literals redirected to CPU. The
reference is fed its own `[B, H, S, D]` layout, fp32, with causal S <= 512 per
call -- the envelope in which its local attention is correct. Fixtures store
tensors in THIS package's layout ([B, S, H, D]; lse [B, H, S]).
"""
import importlib.machinery as machinery
import os
import sys
import types

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_root):
    stub = types.ModuleType("intel_extension_for_pytorch")
    stub.__spec__ = machinery.ModuleSpec("intel_extension_for_pytorch", None)
    sys.modules["intel_extension_for_pytorch"] = stub
    pkg = types.ModuleType("sp_aurora")
    pkg.__path__ = [os.path.join(ref_root, "sp_aurora")]
    pkg.__spec__ = machinery.ModuleSpec("sp_aurora", None, is_package=True)
    pkg.__spec__.submodule_search_locations = pkg.__path__
    sys.modules["sp_aurora"] = pkg


class _TorchProxy:
    """Module proxy: torch.tensor(..., device='xpu') -> CPU; everything else passes."""

    def __init__(self, real):
        self._real = real

    def __getattr__(self, name):
        return getattr(self._real, name)

    def tensor(self, *a, **kw):
        if kw.get("device") == "xpu":
            kw["device"] = "cpu"
        return self._real.tensor(*a, **kw)


def bshd(x):  # reference [B,H,S,D] -> package [B,S,H,D]
    return x.transpose(1, 2).contiguous()


def gen_local(ref_root):
    load_reference(ref_root)
    from sp_aurora.intel_flash_attn import intel_flash_attn_forward
    from sp_aurora.utils import update_out_and_lse
    out = {}
    cases = [("c0", 1, 2, 128, 128, 64, True), ("c1", 1, 2, 96, 160, 32, False),
             ("c2", 2, 1, 200, 200, 128, True), ("c3", 1, 3, 64, 64, 64, False)]
    for name, B, H, Sq, Sk, D, causal in cases:
        g = torch.Generator().manual_seed(sum(map(ord, name)) + 7)
        q = torch.randn(B, H, Sq, D, generator=g)
        k = torch.randn(B, H, Sk, D, generator=g)
        v = torch.randn(B, H, Sk, D, generator=g)
        scale = D ** -0.5
        o, lse = intel_flash_attn_forward(q, k, v, dropout_p=0.0, softmax_scale=scale, causal=causal)
        out.update({f"{name}_q": bshd(q).numpy(), f"{name}_k": bshd(k).numpy(),
                    f"{name}_v": bshd(v).numpy(), f"{name}_out": bshd(o).numpy(),
                    f"{name}_lse": lse.numpy(),
                    f"{name}_meta": np.array([B, H, Sq, Sk, D, int(causal)])})
    # merge of two partial results (reference layouts: out [B,H,S,D] fp32, lse [B,H,S,1])
    g = torch.Generator().manual_seed(99)
    B, H, S, D = 2, 3, 40, 32
    o1 = torch.randn(B, H, S, D, generator=g)
    o2 = torch.randn(B, H, S, D, generator=g)
    l1 = torch.randn(B, H, S, generator=g) * 3
    l2 = torch.randn(B, H, S, generator=g) * 3
    mo, ml = update_out_and_lse(o1.clone(), l1.clone().unsqueeze(-1), o2, l2.unsqueeze(-1))
    out.update({"m_out1": bshd(o1).numpy(), "m_out2": bshd(o2).numpy(), "m_lse1": l1.numpy(),
                "m_lse2": l2.numpy(), "m_out": bshd(mo).numpy(), "m_lse": ml.squeeze(-1).numpy()})
    np.savez(os.path.join(HERE, "local_attention.npz"), **out)
    print("local_attention.npz", len(out))


def _dist_worker(rank, world, ref_root, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    load_reference(ref_root)
    import sp_aurora.intel_ring_flash_attn as ring_mod
    from sp_aurora.comm.all_to_all import all_to_all_5D
    from sp_aurora.intel_ulysses_attn import intel_all_to_all_4d
    ring_mod.torch = _TorchProxy(torch)
    res = {}
    # --- all-to-all permutations (integers: exact) ---
    B, Sl, H, D = 2, 4, 4, 8
    x = (torch.arange(B * Sl * H * D, dtype=torch.float32).view(B, Sl, H, D) + 10000 * rank)
    y = intel_all_to_all_4d(x, 2, 1, group=None)
    z = intel_all_to_all_4d(y, 1, 2, group=None)
    res.update(a4_in=x.numpy(), a4_fwd=y.numpy(), a4_back=z.numpy())
    x5 = (torch.arange(B * Sl * 3 * H * D, dtype=torch.float32).view(B, Sl, 3, H, D) + 100000 * rank)
    y5 = all_to_all_5D(x5, 3, 1, group=None)
    z5 = all_to_all_5D(y5, 1, 3, group=None)
    res.update(a5_in=x5.numpy(), a5_fwd=y5.numpy(), a5_back=z5.numpy())
    # --- ring forward, reference layout [B,H,S_loc,D], contiguous shards ---
    for name, B, H, S, D, causal in [("r0", 1, 2, 128, 64, True), ("r1", 2, 2, 64, 32, False)]:
        g = torch.Generator().manual_seed(1234 + len(name) + S)
        q = torch.randn(B, H, S, D, generator=g)
        k = torch.randn(B, H, S, D, generator=g)
        v = torch.randn(B, H, S, D, generator=g)
        sl = S // world
        qs, ks, vs = (t[:, :, rank * sl:(rank + 1) * sl].contiguous() for t in (q, k, v))
        o, lse = ring_mod.intel_ring_flash_attn_forward(None, qs, ks, vs, D ** -0.5, 0.0, causal)
        if lse.dim() == 4:
            lse = lse.squeeze(-1)
        res.update({f"{name}_q": bshd(q).numpy(), f"{name}_k": bshd(k).numpy(),
                    f"{name}_v": bshd(v).numpy(), f"{name}_out": bshd(o.float()).numpy(),
                    f"{name}_lse": lse.float().numpy(),
                    f"{name}_meta": np.array([B, H, S, D, int(causal), world])})
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


def gen_dist(ref_root, world=2):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_dist_worker, args=(world, ref_root, 29611, ret), nprocs=world, join=True)
    out = {}
    for r in range(world):
        for key, val in ret[r].items():
            if key.endswith(("_q", "_k", "_v", "_meta")):
                out[key] = val          # identical on every rank
            else:
                out[f"{key}_rank{r}"] = val
    np.savez(os.path.join(HERE, "distributed.npz"), **out)
    print("distributed.npz", len(out))


if __name__ == "__main__":
    root = sys.argv[1]
    gen_local(root)
    gen_dist(root)
