"""CPU semantics: two-stream KSA == the reference's interleaved dense-mask formulation; tiny model trains."""
import math

import pytest
import torch

from ksa_b200.config import get_preset, load_config, parse_layer_pattern, Qwen3SummaryAttentionConfig
from ksa_b200.models import Qwen3SummaryModel, get_model_class
from ksa_b200.ops import reference as ref
from ksa_b200.ops.layout import (SummaryLayout, count_attended_pairs, dense_interleaved_mask, get_layout,
                                 two_stream_masks)


def test_pattern_parser():
    assert parse_layer_pattern("([1]*3+[0]*1)*2") == [1, 1, 1, 0, 1, 1, 1, 0]
    assert len(parse_layer_pattern("([128]*3+[1024]*1)*6")) == 24
    with pytest.raises(ValueError):
        parse_layer_pattern("__import__('os')")


def test_config_roundtrip(tmp_path):
    cfg = get_preset("qwen3-1.9b-ksa")
    assert sum(cfg.get_layer_is_summary()) == 21 and cfg.num_layers == 28
    p = tmp_path / "m.json"
    cfg.save(str(p))
    again = load_config(str(p))
    assert isinstance(again, Qwen3SummaryAttentionConfig) and again.to_dict() == cfg.to_dict()
    assert abs(cfg.num_parameters() - 2.21e9) < 0.05e9


def test_shipped_reference_json_loads():
    """A model JSON in the reference's own format (pattern strings, ``__class__`` dispatch) loads unchanged; with
    ``KSA_REFERENCE_DIR`` set, the file that the reference ships is loaded too."""
    import os
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    paths = [os.path.join(here, "examples", "pretrain", "model_config", "model_config_1b9_shipped_shape.json")]
    ref_dir = os.environ.get("KSA_REFERENCE_DIR")
    if ref_dir:
        paths.append(os.path.join(ref_dir, "examples", "pretrain", "model_config", "model_config_1b9_hybrid.json"))
    for path in paths:
        cfg = load_config(path)
        assert cfg.summary_chunk_size == 8 and cfg.get_layer_sliding_chunk_num(3) == 1024


@pytest.mark.parametrize("L,C,S,W", [(256, 32, 1, 2), (192, 16, 2, 1), (128, 8, 1, 4), (100, 32, 1, 1)])
def test_two_stream_masks_equal_interleaved(L, C, S, W):
    lay = SummaryLayout(L, C, S)
    tt, ts, st, ss = two_stream_masks(L, C, S, W)
    if L % C == 0:
        dense = dense_interleaved_mask(lay.expanded_len, C, S, W)
        ti, si = lay.text_rows_in_expanded(), lay.summary_rows_in_expanded()
        assert torch.equal(dense[ti][:, ti], tt) and torch.equal(dense[ti][:, si], ts)
        assert torch.equal(dense[si][:, ti], st) and torch.equal(dense[si][:, si], ss)
    n = int(tt.sum() + ts.sum() + st.sum() + ss.sum())
    assert n == count_attended_pairs(L, C, S, W)


def test_two_stream_attention_equals_interleaved():
    torch.manual_seed(0)
    B, L, Hq, Hkv, D, C, S, W = 2, 256, 4, 2, 16, 32, 2, 2
    lay = SummaryLayout(L, C, S)
    T = lay.expanded_len
    q, k, v = torch.randn(B, T, Hq, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)
    o = ref.interleaved_ksa_attention(q, k, v, C, S, W)
    (qt, qs), (kt, ks), (vt, vs) = lay.split(q), lay.split(k), lay.split(v)
    ot, os_ = ref.ksa_attention(qt, kt, vt, qs, ks, vs, C, S, W)
    o_t_ref, o_s_ref = lay.split(o)
    assert torch.allclose(ot, o_t_ref, atol=1e-4) and torch.allclose(os_, o_s_ref, atol=1e-4)


def test_position_ids_match_reference_rule():
    lay = SummaryLayout(64, 16, 2, "origin", "last_chunk_slice_right")
    assert lay.summary_position_ids().tolist() == [7, 15, 23, 31, 39, 47, 55, 63]
    lay1 = SummaryLayout(64, 16, 1, "origin", "last_chunk_slice_right")
    assert lay1.summary_position_ids().tolist() == [15, 31, 47, 63]
    assert SummaryLayout(64, 16, 1, "inner_chunk", "zeros").text_position_ids()[17] == 1
    cu = torch.tensor([0, 20, 64])
    assert lay1.remap_cu_seqlens(cu).tolist() == [0, 21, 68]


def _interleaved_model_forward(model, tokens):
    """The reference formulation: one interleaved sequence, dense mask, summary rows overwritten per layer."""
    cfg = model.config
    B, L = tokens.shape
    C, S = cfg.summary_chunk_size, cfg.summary_token_num
    lay = get_layout(L, C, S, cfg.summary_chunk_position_ids_type, cfg.summary_token_position_ids_type)
    Hq, Hkv, Dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    x_t = torch.nn.functional.embedding(tokens, model.tok_embeddings.weight)
    x_s = model.summary_embedding.weight.repeat(B, lay.n_chunks, 1)
    x = lay.interleave(x_t, x_s)
    pos = lay.expanded_position_ids()
    smask = lay.summary_mask_expanded()
    for i, layer in enumerate(model.layers):
        a = layer.attn
        if layer.is_summary_layer:
            h = ref.rms_norm(x, layer.sa_norm.scale)
            qkv = h @ a.wqkv.weight.t()
            qkv[:, smask] = h[:, smask] @ a.wqkv_summary.weight.t()
            q, k, v = qkv.split([Hq * Dh, Hkv * Dh, Hkv * Dh], -1)
            q, k = q.reshape(B, -1, Hq, Dh), k.reshape(B, -1, Hkv, Dh)
            q, k = ref.qk_norm_rope(q, k, a.q_norm.scale, a.k_norm.scale, pos, cfg.rope_base)
            o = ref.interleaved_ksa_attention(q, k, v.reshape(B, -1, Hkv, Dh), C, S, layer.window_chunks)
            x = x + o.reshape(B, -1, Hq * Dh) @ a.output_proj.weight.t()
            h2 = ref.rms_norm(x, layer.mlp_norm.scale)
            x = x + ref.swiglu(h2 @ layer.mlp.w13.weight.t()) @ layer.mlp.w2.weight.t()
        else:
            xt = x[:, ~smask]
            h = ref.rms_norm(xt, layer.sa_norm.scale)
            qkv = h @ a.wqkv.weight.t()
            q, k, v = qkv.split([Hq * Dh, Hkv * Dh, Hkv * Dh], -1)
            q, k = q.reshape(B, -1, Hq, Dh), k.reshape(B, -1, Hkv, Dh)
            q, k = ref.qk_norm_rope(q, k, a.q_norm.scale, a.k_norm.scale, pos[~smask], cfg.rope_base)
            o = ref.causal_attention(q, k, v.reshape(B, -1, Hkv, Dh))
            xt = xt + o.reshape(B, -1, Hq * Dh) @ a.output_proj.weight.t()
            h2 = ref.rms_norm(xt, layer.mlp_norm.scale)
            xt = xt + ref.swiglu(h2 @ layer.mlp.w13.weight.t()) @ layer.mlp.w2.weight.t()
            x = x.clone()
            x[:, ~smask] = xt
    h = ref.rms_norm(x[:, ~smask], model.norm.scale)
    return h @ model.output.weight.t()


def test_tiny_model_matches_interleaved_reference_and_trains():
    torch.manual_seed(0)
    cfg = get_preset("qwen3-ksa-tiny")
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    tokens = torch.randint(0, cfg.vocab_size, (2, 512))
    logits = model(tokens)
    with torch.no_grad():
        expect = _interleaved_model_forward(model, tokens)
    assert torch.allclose(logits, expect, atol=1e-4), (logits - expect).abs().max()
    labels = torch.roll(tokens, -1, 1)
    labels[:, -1] = -100
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    losses = []
    for _ in range(3):
        loss = model(tokens, labels=labels)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert abs(losses[0] - math.log(cfg.vocab_size)) < 0.5 and losses[-1] < losses[0]


def test_summary_mix_qkv_blends_after_the_qk_norm_with_each_side_norm():
    """``summary_mix_qkv``: mix = 1 is the model without the anneal; mix = 0 treats the summary rows with the base
    projections AND the base QK norms; in between the rotated rows are the linear blend of the two ends."""
    base_cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 1], "embed_dim": 64,
                                                    "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16,
                                                    "summary_independent_qk_norm": True})
    cfg = base_cfg.merge({"summary_mix_qkv": True, "summary_mix_start_iter": 0, "summary_mix_end_iter": 10})
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    with torch.no_grad():   # make the two norms differ
        for layer in model.layers:
            layer.attn.q_norm_summary.scale.mul_(1.5)
            layer.attn.k_norm.scale.mul_(0.7)
    tokens = torch.randint(0, cfg.vocab_size, (1, 256))

    def first_layer_rows(m, it):
        m.set_mix_coeff(it)
        got = {}
        m(tokens, kv_sink=lambda i, qkv, is_sum: got.setdefault(i, qkv.detach().clone()))
        return got[0]

    with torch.no_grad():
        q1, qh, q0 = first_layer_rows(model, 0), first_layer_rows(model, 5), first_layer_rows(model, 10)
        assert model.layers[0].attn.mix_coeff == 0.0
        plain = get_model_class(base_cfg.model_class)(base_cfg)
        plain.load_state_dict(model.state_dict())
        assert torch.allclose(first_layer_rows(plain, 0), q1, atol=1e-6)
        assert torch.allclose(qh, 0.5 * (q0 + q1), atol=1e-5)
        shared = get_model_class(base_cfg.model_class)(base_cfg)
        sd = model.state_dict()
        for i in range(2):
            sd[f"layers.{i}.attn.wqkv_summary.weight"] = sd[f"layers.{i}.attn.wqkv.weight"]
            sd[f"layers.{i}.attn.q_norm_summary.scale"] = sd[f"layers.{i}.attn.q_norm.scale"]
            sd[f"layers.{i}.attn.k_norm_summary.scale"] = sd[f"layers.{i}.attn.k_norm.scale"]
        shared.load_state_dict(sd)
        assert torch.allclose(first_layer_rows(shared, 0), q0, atol=1e-5)


def test_packed_documents_do_not_see_each_other_in_full_attention_layers():
    """``cu_seqlens``: with every layer a full-attention layer the logits of a document do not depend on the tokens of
    the documents packed in front of it; without it they do."""
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "use_summary_attention": False, "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16})
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    a = torch.randint(0, 256, (1, 96))
    b = a.clone()
    b[:, :40] = torch.randint(0, 256, (1, 40))           # another first document
    cu = torch.tensor([0, 40, 96], dtype=torch.int32)
    with torch.no_grad():
        la, lb = model(a, cu_seqlens=cu), model(b, cu_seqlens=cu)
        assert torch.allclose(la[:, 40:], lb[:, 40:], atol=1e-6)
        assert not torch.allclose(model(a)[:, 40:], model(b)[:, 40:], atol=1e-4)


def test_muse_and_hf_key_roundtrip():
    cfg = get_preset("qwen3-ksa-tiny")
    model = Qwen3SummaryModel(cfg)
    model.init_weights(seed=1)
    muse = model.muse_state_dict()
    assert "model.layers.0.attn.q_proj_summary.weight" in muse and "model.layers.3.attn.q_proj_summary.weight" not in muse
    assert "model.layers.0.mlp.w1.weight" in muse and "summary_embedding.weight" in muse
    hf = model.revert_hf_state_dict(model.state_dict())
    assert hf["model.embed_tokens.weight"].shape[0] == cfg.vocab_size + cfg.summary_token_num
    assert hf["lm_head.weight"].shape[0] == cfg.vocab_size + cfg.summary_token_num
    assert "model.layers.0.self_attn.q_proj_summary.weight" in hf and "model.layers.1.mlp.gate_proj.weight" in hf
    assert "model.layers.2.input_layernorm.weight" in hf and "model.layers.2.self_attn.q_norm.weight" in hf
    other = Qwen3SummaryModel(cfg)
    other.load_state_dict(other.convert_hf_state_dict(hf))
    for (k, a), (_, b) in zip(model.state_dict().items(), other.state_dict().items()):
        assert torch.equal(a, b), k


def test_summary_attention_modes_agree():
    """``summary_attention_mode`` "mask" (dense mask) and "block" (query blocks with gathered keys) give the same model
    output and gradients as the default; the block form alone is also checked against the dense oracle on ragged
    shapes."""
    import torch
    from ksa_b200.config import get_preset
    from ksa_b200.models import get_model_class
    from ksa_b200.ops import reference as ref
    torch.manual_seed(0)
    for (L, C, S, W, qb) in [(256, 32, 1, 2, 64), (192, 16, 2, 1, 48), (100, 32, 1, 1, 32), (257, 16, 2, 3, 64)]:
        B, Hq, Hkv, D = 2, 4, 2, 16
        Ns = ((L + C - 1) // C) * S
        q, k, v = torch.randn(B, L, Hq, D), torch.randn(B, L, Hkv, D), torch.randn(B, L, Hkv, D)
        qs, ks, vs = torch.randn(B, Ns, Hq, D), torch.randn(B, Ns, Hkv, D), torch.randn(B, Ns, Hkv, D)
        a = ref.ksa_attention(q, k, v, qs, ks, vs, C, S, W)
        b = ref.ksa_attention_blockwise(q, k, v, qs, ks, vs, C, S, W, q_block=qb)
        assert torch.allclose(a[0], b[0], atol=2e-6) and torch.allclose(a[1], b[1], atol=2e-6)
    base = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "head_dim": 16,
                                               "summary_chunk_size": 16, "summary_sliding_chunk_num": 2})
    tokens = torch.randint(0, 200, (2, 80))
    outs = {}
    for mode in ("kernel", "mask", "block"):
        cfg = base.merge({"summary_attention_mode": mode})
        model = get_model_class(cfg.model_class)(cfg)
        model.init_weights(seed=0)
        loss = model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        outs[mode] = (float(loss.detach()), model.layers[0].attn.wqkv.weight.grad.clone())
    for mode in ("mask", "block"):
        assert abs(outs[mode][0] - outs["kernel"][0]) < 1e-5
        assert torch.allclose(outs[mode][1], outs["kernel"][1], atol=1e-5)


@pytest.mark.parametrize("safetensors,shard", [(True, "5GB"), (True, "1MB"), (False, "5GB"), (False, "1MB")])
def test_save_pretrained_and_from_pretrained_roundtrip(tmp_path, safetensors, shard):
    """HF-layout directories in both weight formats, one file or sharded with an index, load back bit for bit."""
    import json
    import os
    cfg = get_preset("qwen3-ksa-tiny")
    model = Qwen3SummaryModel(cfg)
    model.init_weights(seed=2)
    model.save_pretrained(str(tmp_path), max_shard_size=shard, save_safetensors=safetensors)
    files = sorted(os.listdir(tmp_path))
    ext = ".safetensors" if safetensors else ".bin"
    weights = [f for f in files if f.endswith(ext)]
    if shard == "5GB":
        assert weights == ["model.safetensors" if safetensors else "pytorch_model.bin"]
    else:
        index_name = "model.safetensors.index.json" if safetensors else "pytorch_model.bin.index.json"
        assert len(weights) > 1 and index_name in files
        index = json.load(open(tmp_path / index_name))
        assert set(index["weight_map"].values()) == set(weights)
    back = Qwen3SummaryModel.from_pretrained(str(tmp_path))
    for (k, a), (_, b) in zip(model.state_dict().items(), back.state_dict().items()):
        assert torch.equal(a, b), k


def test_optimizer_groups_and_hf_state_dict_helpers():
    """One parameter group with weight decay on everything (the reference's choice), usable by torch.optim.AdamW."""
    cfg = get_preset("qwen3-ksa-tiny")
    model = Qwen3SummaryModel(cfg)
    model.init_weights(seed=0)
    groups = model.get_optimizer_grouped_parameters(0.1, learning_rate=3e-4)
    assert len(groups) == 1 and groups[0]["weight_decay"] == 0.1 and groups[0]["lr"] == 3e-4
    assert len(groups[0]["params"]) == len(list(model.parameters()))
    assert "lr" not in model.get_optimizer_grouped_parameters(0.1)[0]
    torch.optim.AdamW(groups)
    assert set(model.get_hf_state_dict()) == set(model.revert_hf_state_dict(dict(model.state_dict())))


def test_load_full_state_dict_allow_and_skip_rules():
    """Missing or reshaped parameters keep their initialisation only when named; skipped ones are never loaded;
    anything else is an error (the reference's ``load_from_full_model_state_dict`` rules)."""
    from ksa_b200.models.base import load_full_state_dict
    cfg = get_preset("qwen3-ksa-tiny")
    src = Qwen3SummaryModel(cfg)
    src.init_weights(seed=1)
    state = {k: v.clone() for k, v in src.state_dict().items()}

    def fresh():
        m = Qwen3SummaryModel(cfg)
        m.init_weights(seed=2)
        return m
    # complete state dict: everything is taken
    m = fresh()
    kept = load_full_state_dict(m, state)
    assert kept == {"skipped": [], "missing": [], "shape": []}
    assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), src.state_dict().values()))
    # a missing parameter and a reshaped one
    partial = dict(state)
    del partial["summary_embedding.weight"]
    partial["tok_embeddings.weight"] = state["tok_embeddings.weight"][:-8]
    with pytest.raises(RuntimeError, match="allow_random_init_params"):
        load_full_state_dict(fresh(), partial)
    m, init = fresh(), fresh()
    kept = load_full_state_dict(m, partial, allow_random_init_params="summary_embedding.weight,tok_embeddings.weight")
    assert kept["missing"] == ["summary_embedding.weight"] and kept["shape"] == ["tok_embeddings.weight"]
    assert torch.equal(m.tok_embeddings.weight, init.tok_embeddings.weight)          # kept its own initialisation
    assert torch.equal(m.layers[0].attn.wqkv.weight, src.layers[0].attn.wqkv.weight)  # the rest was loaded
    # skipped by substring, although present
    m, init = fresh(), fresh()
    kept = load_full_state_dict(m, state, skip_load_params=["_summary", "norm.scale"])
    assert kept["skipped"] and all("_summary" in k or "norm.scale" in k for k in kept["skipped"])
    assert torch.equal(m.layers[0].attn.wqkv_summary.weight, init.layers[0].attn.wqkv_summary.weight)
    assert torch.equal(m.layers[0].mlp.w2.weight, src.layers[0].mlp.w2.weight)
    # a key the model does not know
    with pytest.raises(RuntimeError, match="does not have"):
        load_full_state_dict(fresh(), dict(state, extra=torch.zeros(1)))
