"""transformers hook (sp_aurora/adapters/hf_adapter.py:34-61,285-385 in the reference): plumbing
only, on CPU, with a torch stand-in for the varlen kernel call."""
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

transformers = pytest.importorskip("transformers")


def _fake_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q=None, max_seqlen_k=None,
                 heads_k_stride=None, local_k_slice=None, softmax_scale=None, causal=False,
                 deterministic=False, group=None, **kw):
    from oracle import attention_oracle as orc
    assert causal and local_k_slice == slice(0, q.shape[0]) and heads_k_stride == 2
    out = torch.empty_like(q)
    cu = cu_seqlens_q.tolist()
    for a, b in zip(cu, cu[1:]):
        o, _ = orc.attention_ref(q[None, a:b], k[None, a:b], v[None, a:b], softmax_scale, True)
        out[a:b] = o[0].to(q.dtype)
    return out


@pytest.fixture
def hooked(monkeypatch):
    import transformers.modeling_flash_attention_utils as fa_utils
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    from sp_aurora_b200.adapters import hf_adapter as hf
    calls = []

    def original(query_states, key_states, value_states, attention_mask, query_length, is_causal,
                 dropout=0.0, position_ids=None, softmax_scale=None, **kwargs):
        calls.append("original")
        return query_states

    saved_fn = fa_utils._flash_attention_forward
    saved_entry = ALL_ATTENTION_FUNCTIONS["flash_attention_2"]
    fa_utils._flash_attention_forward = original
    monkeypatch.setattr(hf, "llama3_flash_attn_varlen_func", _fake_varlen)
    hf.DATA_PARAMS.clear()
    hf.use_ring_attn(True)
    yield hf, fa_utils, ALL_ATTENTION_FUNCTIONS, calls
    fa_utils._flash_attention_forward = saved_fn
    ALL_ATTENTION_FUNCTIONS["flash_attention_2"] = saved_entry
    hf.DATA_PARAMS.clear()
    hf.use_ring_attn(True)


def _reference(q, k, v, cu, scale):
    from oracle import attention_oracle as orc
    out = torch.empty_like(q)
    for a, b in zip(cu, cu[1:]):
        o, _ = orc.attention_ref(q[:, a:b], k[:, a:b], v[:, a:b], scale, True)
        out[:, a:b] = o.to(q.dtype)
    return out


def test_substituted_hooks_route_through_the_varlen_path(hooked):
    hf, fa_utils, table, calls = hooked
    g = torch.Generator().manual_seed(3)
    S, H, Hkv, D = 12, 4, 2, 8
    q = torch.randn(1, S, H, D, generator=g)
    k = torch.randn(1, S, Hkv, D, generator=g)
    v = torch.randn(1, S, Hkv, D, generator=g)
    cu = [0, 5, 12]
    with pytest.raises(RuntimeError, match="update_ring_flash_attn_params"):
        hf._ring_attention(q, k, v, process_group=None, heads_k_stride=2)
    hf.update_ring_flash_attn_params(torch.tensor(cu, dtype=torch.int32), None)
    assert hf.DATA_PARAMS["cu_seqlens_q"].tolist() == cu and hf.DATA_PARAMS["local_k_slice"] == slice(0, S)
    hf.substitute_hf_flash_attn(None, heads_k_stride=2)
    ref = _reference(q, k, v, cu, D ** -0.5)

    # the legacy hook, called the way transformers' integration calls it
    out = fa_utils._flash_attention_forward(q, k, v, None, query_length=S, is_causal=True, dropout=0.0,
                                            softmax_scale=D ** -0.5, sliding_window=None, softcap=None,
                                            use_top_left_mask=False, target_dtype=None)
    assert out.shape == (1, S, H, D) and torch.allclose(out, ref, atol=1e-5)
    # the attention-function table: [B, H, S, D] in, ([B, S, H, D], None) out
    module = types.SimpleNamespace(is_causal=True)
    for name in ("flash_attention_2", "sp_aurora"):
        o2, w = table[name](module, q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None,
                            dropout=0.0, scaling=D ** -0.5, sliding_window=4096)
        assert w is None and o2.shape == (1, S, H, D) and torch.allclose(o2, ref, atol=1e-5)
    assert calls == []

    hf.use_ring_attn(False)
    back = fa_utils._flash_attention_forward(q, k, v, None, query_length=S, is_causal=True)
    assert back is q and calls == ["original"]
    hf.use_ring_attn(True)
    # substituting twice does not stack wrappers
    wrapped = fa_utils._flash_attention_forward
    hf.substitute_hf_flash_attn(None, heads_k_stride=2)
    assert fa_utils._flash_attention_forward is wrapped


def test_unsupported_arguments_raise(hooked):
    hf, fa_utils, table, _ = hooked
    q = torch.randn(1, 8, 2, 8)
    hf.update_ring_flash_attn_params([0, 8], None)
    kw = dict(process_group=None, heads_k_stride=2)
    with pytest.raises(NotImplementedError):
        hf._ring_attention(q, q, q, dropout=0.1, **kw)
    with pytest.raises(NotImplementedError):
        hf._ring_attention(q, q, q, softcap=30.0, **kw)
    with pytest.raises(NotImplementedError):
        hf._ring_attention(q, q, q, sliding_window=4, **kw)
    with pytest.raises(NotImplementedError):
        hf._ring_attention(q, q, q, is_causal=False, **kw)
    with pytest.raises(ValueError):
        hf._ring_attention(torch.randn(2, 8, 2, 8), q, q, **kw)


def test_tiny_llama_runs_through_the_hook(hooked, monkeypatch):
    """A two-layer Llama (GQA) from transformers with `_attn_implementation="sp_aurora"`: one
    sequence against the eager model, and two sequences packed into one stream (position ids
    restarting) against the eager model run on each sequence alone. Checks the layout, scaling
    and GQA plumbing of the table entry with a torch stand-in for the kernel call."""
    from transformers import LlamaConfig, LlamaModel
    hf, fa_utils, table, _ = hooked

    def stand_in(q, k, v, cu_seqlens_q, cu_seqlens_k, **kw):
        kw.update(heads_k_stride=2, local_k_slice=slice(0, q.shape[0]))
        return _fake_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, **kw)
    monkeypatch.setattr(hf, "llama3_flash_attn_varlen_func", stand_in)
    cfg = LlamaConfig(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    model = LlamaModel(cfg).eval()
    ids = torch.randint(0, 100, (1, 20))
    with torch.no_grad():
        ref_one = model(input_ids=ids).last_hidden_state
        ref_a = model(input_ids=ids[:, :7]).last_hidden_state
        ref_b = model(input_ids=ids[:, 7:]).last_hidden_state
    hf.substitute_hf_flash_attn(None, heads_k_stride=1)
    model.config._attn_implementation = "sp_aurora"
    with torch.no_grad():
        hf.update_ring_flash_attn_params([0, 20], None)
        out_one = model(input_ids=ids).last_hidden_state
        hf.update_ring_flash_attn_params([0, 7, 20], None)
        pos = torch.cat((torch.arange(7), torch.arange(13)))[None]
        out_packed = model(input_ids=ids, position_ids=pos).last_hidden_state
    assert (out_one - ref_one).abs().max() <= 1e-5
    assert (out_packed[:, :7] - ref_a).abs().max() <= 1e-5
    assert (out_packed[:, 7:] - ref_b).abs().max() <= 1e-5
