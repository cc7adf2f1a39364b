"""train -> DCP save -> convert -> HF ``trust_remote_code`` load -> logits / generation match the framework model."""
import os

import pytest
import torch

from ksa_b200.config import get_preset
from ksa_b200.inference import KsaInferenceEngine
from ksa_b200.models import get_model_class
from ksa_b200.tools.convert import (convert_dcp_to_hf, hf_config_from_model_config, load_hf_checkpoint,
                                    model_config_from_hf_config)
from ksa_b200.training.checkpoint import AppState, DistributedCheckpointer, save_checkpoint
from ksa_b200.training.engine import TrainEngine

TEMPLATE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ksa_b200", "hf")


def _export(tmp_path):
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 4, "embed_dim": 64, "intermediate_dim": 128,
                                               "vocab_size": 256, "summary_token_begin": 256, "head_dim": 16, "summary_chunk_size": 8,
                                               "summary_sliding_chunk_num": 2})
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.mul_(3.0)
    eng = TrainEngine(model, lr=1e-3)
    save_checkpoint(AppState(eng), DistributedCheckpointer(), str(tmp_path), 1)
    out = convert_dcp_to_hf(str(tmp_path), "global_step1", TEMPLATE, dtype="fp32", remap="muse2hf",
                            config_overrides=hf_config_from_model_config(cfg))
    return cfg, model, out


def test_hf_roundtrip_logits_and_generation(tmp_path):
    from transformers import AutoModelForCausalLM
    cfg, model, out = _export(tmp_path)
    hf = AutoModelForCausalLM.from_pretrained(out, trust_remote_code=True, torch_dtype=torch.float32)
    hf.eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 37))
    model.drop_partial_summary = True
    with torch.no_grad():
        expect = model(tokens)
        got = hf(tokens).logits
        pure = hf.lm_head(hf.model(tokens).last_hidden_state)[..., :cfg.vocab_size]   # dependency-free path
    assert got.shape[-1] == hf.config.vocab_size and bool(torch.isinf(got[..., cfg.vocab_size:]).all())
    got = got[..., :cfg.vocab_size]
    assert torch.allclose(got, expect, atol=1e-4), (got - expect).abs().max()
    assert torch.allclose(pure, expect, atol=2e-4), (pure - expect).abs().max()
    gen = hf.generate(tokens, max_new_tokens=12, eos_token_id=-1)
    ref = KsaInferenceEngine(model, max_len=64, batch=2).generate(tokens, 12)
    assert torch.equal(gen, ref)


def test_converted_directory_loads_into_the_engine(tmp_path):
    """The converted directory is enough to rebuild this package's model: config.json maps back to the model config
    and the engine generates the same tokens as the model that was exported."""
    import json
    cfg, model, out = _export(tmp_path)
    back = model_config_from_hf_config(json.load(open(os.path.join(out, "config.json"))))
    for f in ("vocab_size", "embed_dim", "intermediate_dim", "num_layers", "num_heads", "num_kv_heads", "head_dim",
              "summary_chunk_size", "summary_token_num", "summary_token_begin", "summary_sliding_chunk_num",
              "summary_independent_parameters", "rope_base", "tie_word_embeddings"):
        assert getattr(back, f) == getattr(cfg, f), f
    assert list(back.get_layer_is_summary()) == list(cfg.get_layer_is_summary())
    loaded = load_hf_checkpoint(out, dtype=torch.float32)
    tokens = torch.randint(0, cfg.vocab_size, (2, 37))
    want = KsaInferenceEngine(model, max_len=64, batch=2).generate(tokens, 12)
    got = KsaInferenceEngine(loaded, max_len=64, batch=2).generate(tokens, 12)
    assert torch.equal(got, want)


def test_truncate_predict_nums_limits_logits_and_generated_tokens(tmp_path):
    from transformers import AutoModelForCausalLM
    cfg, model, out = _export(tmp_path)
    hf = AutoModelForCausalLM.from_pretrained(out, trust_remote_code=True, torch_dtype=torch.float32).eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 21))
    full = hf(tokens).logits
    assert full.shape[-1] == hf.config.vocab_size == cfg.vocab_size + cfg.summary_token_num
    hf.config.truncate_predict_nums = 100
    cut = hf(tokens).logits
    assert cut.shape[-1] == 100 and torch.equal(cut, full[..., :100])
    gen = hf.generate(tokens, max_new_tokens=8, eos_token_id=-1)
    assert int(gen[:, 21:].max()) < 100


def test_hf_generate_sampling_options(tmp_path):
    """top_k = 1 is greedy whatever the temperature; sampling with a seed is reproducible."""
    from transformers import AutoModelForCausalLM
    cfg, model, out = _export(tmp_path)
    hf = AutoModelForCausalLM.from_pretrained(out, trust_remote_code=True, torch_dtype=torch.float32).eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 19))
    greedy = hf.generate(tokens, max_new_tokens=6, eos_token_id=-1)
    assert torch.equal(hf.generate(tokens, max_new_tokens=6, eos_token_id=-1, do_sample=True, temperature=1.3, top_k=1), greedy)
    torch.manual_seed(4)
    a = hf.generate(tokens, max_new_tokens=6, eos_token_id=-1, do_sample=True, temperature=0.9, top_p=0.8, top_k=20)
    torch.manual_seed(4)
    b = hf.generate(tokens, max_new_tokens=6, eos_token_id=-1, do_sample=True, temperature=0.9, top_p=0.8, top_k=20)
    assert torch.equal(a, b) and a.shape == (2, 25)
