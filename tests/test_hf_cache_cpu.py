"""The HF model's ring-buffer KV cache: stock ``generate`` against recomputing the whole sequence every step, and the
cache state machine against a naive decoder that re-evaluates the full two-stream masks."""
import importlib.util
import os
import sys

import pytest
import torch
from hypothesis import given, settings, strategies as st

HF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ksa_b200", "hf")


def _load_module():
    """The template as a stand-alone module (the way ``trust_remote_code`` loads it from a checkpoint directory)."""
    sys.path.insert(0, HF_DIR)
    try:
        spec = importlib.util.spec_from_file_location("modeling_qwen3sa_standalone", os.path.join(HF_DIR, "modeling_qwen3sa.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod        # transformers looks the defining module up by name
        spec.loader.exec_module(mod)
    finally:
        sys.path.remove(HF_DIR)
    return mod


MOD = _load_module()


def _model(S=1, C=8, W=2, layers=4, freq="([1]*3+[0]*1)*1", seed=0, **kw):
    cfg = MOD.Qwen3SAConfig(vocab_size=128 + S, hidden_size=32, intermediate_size=64, num_hidden_layers=layers,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=8, summary_token_begin=128,
                            summary_chunk_size=C, summary_token_num=S, summary_sliding_chunk_num=W,
                            summary_layer_freq=freq, max_position_embeddings=4096, **kw)
    torch.manual_seed(seed)
    m = MOD.Qwen3ForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.mul_(4.0)          # spread the logits so that greedy choices are not ties
    return m


@pytest.mark.parametrize("S", [1, 2])
@pytest.mark.parametrize("framework", [True, False])
def test_stock_generate_equals_recomputing_every_step(S, framework, monkeypatch):
    """3:1 hybrid stack, batch 2, prompt ending inside a chunk, 3 chunks of new tokens through ``GenerationMixin``'s own
    loop: cached decoding and ``use_cache=False`` (whole sequence re-run each step) give the same tokens, with the
    ``ksa_b200`` package importable and without it."""
    if not framework:
        monkeypatch.setattr(MOD, "_framework", lambda: None)
    m = _model(S=S)
    C = m.config.summary_chunk_size
    prompt = torch.randint(0, 128, (2, 2 * C + 3))
    with torch.no_grad():
        cached = m.generate(prompt, max_new_tokens=3 * C, do_sample=False, use_cache=True, eos_token_id=-1)
        plain = m.generate(prompt, max_new_tokens=3 * C, do_sample=False, use_cache=False, eos_token_id=-1)
    assert cached.shape == (2, prompt.shape[1] + 3 * C)
    assert torch.equal(cached, plain)
    assert int(cached.max()) < 128                      # no summary id ever leaves the model


def test_generate_features_of_the_library_work_on_the_ring_cache():
    """Stopping criteria, a streamer, sampling processors and beam search come from ``GenerationMixin``."""
    from transformers import StoppingCriteria, StoppingCriteriaList
    from transformers.generation.streamers import BaseStreamer

    class StopAt(StoppingCriteria):
        def __call__(self, input_ids, scores, **kw):
            return torch.full((input_ids.shape[0],), input_ids.shape[1] >= 30, dtype=torch.bool)

    class Collect(BaseStreamer):
        def __init__(self):
            self.chunks = []

        def put(self, value):
            self.chunks.append(value.clone())

        def end(self):
            pass

    m = _model()
    prompt = torch.randint(0, 128, (1, 19))
    streamer = Collect()
    out = m.generate(prompt, max_new_tokens=40, do_sample=False, eos_token_id=-1, streamer=streamer,
                     stopping_criteria=StoppingCriteriaList([StopAt()]))
    assert out.shape[1] == 30 and len(streamer.chunks) == 1 + 11
    torch.manual_seed(3)
    a = m.generate(prompt, max_new_tokens=12, do_sample=True, top_k=5, temperature=0.7, eos_token_id=-1)
    torch.manual_seed(3)
    b = m.generate(prompt, max_new_tokens=12, do_sample=True, top_k=5, temperature=0.7, eos_token_id=-1)
    assert torch.equal(a, b)
    beams = m.generate(prompt, max_new_tokens=10, num_beams=3, do_sample=False, eos_token_id=-1)
    assert beams.shape == (1, 29)
    with pytest.raises(NotImplementedError, match="padded"):
        mask = torch.ones(2, 19, dtype=torch.long)
        mask[0, :3] = 0
        m.generate(prompt.repeat(2, 1), attention_mask=mask, max_new_tokens=2, eos_token_id=-1)


def test_prepare_inputs_appends_summary_tokens_at_chunk_boundaries():
    m = _model(S=2)
    cfg = m.config
    C, S = cfg.summary_chunk_size, cfg.summary_token_num
    prompt = torch.randint(0, 128, (1, C - 1))
    with torch.no_grad():
        out = m(prompt, use_cache=True)
    cache = out.past_key_values
    assert isinstance(cache, MOD.KsaRingBufferCache) and cache.get_seq_length() == C - 1 and cache.boundary_due()
    seq = torch.cat([prompt, torch.tensor([[5]])], 1)
    inputs = m.prepare_inputs_for_generation(seq, past_key_values=cache, next_sequence_length=1, use_cache=True)
    assert inputs["input_ids"].tolist() == [[5, 128, 129]]
    assert inputs["position_ids"].tolist() == [[C - 1, C // 2 - 1, C - 1]]
    with torch.no_grad():
        m(**inputs)
    assert cache.n_chunks == 1 and cache.cur_len == 0 and cache.get_seq_length() == C
    seq = torch.cat([seq, torch.tensor([[6]])], 1)
    inputs = m.prepare_inputs_for_generation(seq, past_key_values=cache, next_sequence_length=1, use_cache=True)
    assert inputs["input_ids"].tolist() == [[6]] and "position_ids" not in inputs


@settings(max_examples=12, deadline=None)
@given(S=st.integers(1, 2), C=st.sampled_from([2, 4, 8]), W=st.integers(1, 3), prompt_len=st.integers(1, 40),
       new=st.integers(1, 40), hybrid=st.booleans(), seed=st.integers(0, 3))
def test_cache_state_machine_against_a_naive_full_mask_decoder(S, C, W, prompt_len, new, hybrid, seed):
    """Any prompt length and any number of decoded tokens (ring wrap-around, regrowth of the summary region, chunk
    boundaries): the logits of cached decoding equal those of running the whole sequence through the dense masks."""
    m = _model(S=S, C=C, W=W, layers=2, freq=[1, 0] if hybrid else [1, 1], seed=seed)
    torch.manual_seed(seed)
    seq = torch.randint(0, 128, (1, prompt_len + new))
    with torch.no_grad():
        out = m.model(seq[:, :prompt_len], use_cache=True)
        cache = out.past_key_values
        for t in range(prompt_len, prompt_len + new):
            h = m.model(seq[:, t:t + 1], past_key_values=cache, use_cache=True).last_hidden_state[:, -1]
            full = m.model(seq[:, :t + 1]).last_hidden_state[:, -1]
            assert torch.allclose(h, full, atol=2e-4), (t, (h - full).abs().max())
    assert cache.get_seq_length() == prompt_len + new
    assert cache.n_chunks == (prompt_len + new) // C and cache.cur_len == (prompt_len + new) % C
