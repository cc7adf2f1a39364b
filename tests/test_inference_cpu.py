"""Ring-buffer decoding equals recomputing the whole sequence with the training graph (CPU, fp32)."""
import pytest
import torch

from ksa_b200.config import get_preset
from ksa_b200.inference import KsaInferenceEngine
from ksa_b200.models import get_model_class


def _model(chunk=8, n_sum=1, window=2, layers=4, freq=None):
    cfg = get_preset("qwen3-ksa-tiny").merge({
        "num_layers": layers, "summary_layer_freq": freq or [1, 1, 0, 1][:layers], "embed_dim": 64,
        "intermediate_dim": 128, "vocab_size": 128, "head_dim": 16, "num_heads": 4, "num_kv_heads": 2,
        "summary_chunk_size": chunk, "summary_token_num": n_sum, "summary_sliding_chunk_num": window})
    torch.manual_seed(0)
    m = get_model_class(cfg.model_class)(cfg)
    m.init_weights(seed=0)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.mul_(3.0)   # make attention patterns non-trivial
    return m.eval()


@pytest.mark.parametrize("chunk,n_sum,window,prompt_len", [(8, 1, 2, 21), (8, 2, 1, 16), (4, 1, 3, 5), (8, 1, 0, 19)])
def test_decode_matches_full_recompute(chunk, n_sum, window, prompt_len):
    model = _model(chunk, n_sum, window)
    B, new = 2, 3 * chunk + 2
    torch.manual_seed(1)
    prompt = torch.randint(0, model.config.vocab_size, (B, prompt_len))
    eng = KsaInferenceEngine(model, max_len=prompt_len + new + 4, batch=B)
    seq = prompt
    logits = eng.prefill(prompt)
    model.drop_partial_summary = True
    for step in range(new):
        with torch.no_grad():
            full = model(seq)[:, -1].float()
        assert torch.allclose(logits, full, atol=2e-4, rtol=1e-3), (step, (logits - full).abs().max())
        nxt = full.argmax(-1)
        seq = torch.cat([seq, nxt[:, None]], dim=1)
        logits = eng.decode_step(nxt)


def test_generate_runs_and_cache_is_smaller_than_full_attention():
    model = _model(8, 1, 2)
    eng = KsaInferenceEngine(model, max_len=256, batch=1)
    out = eng.generate(torch.randint(0, 128, (1, 30)), max_new_tokens=20)
    assert out.shape == (1, 50)
    full = 2 * 256 * model.config.num_kv_heads * model.config.head_dim * 4 * model.config.num_layers
    assert eng.cache_bytes() < full


def test_cache_state_machine_against_recompute_on_random_schedules():
    """Random chunk sizes, windows, summary counts, prompt lengths and step counts (hypothesis): after every step the
    cached decode equals a full recompute, across chunk boundaries, ring wrap-around and a second prefill that reuses
    the engine."""
    from hypothesis import given, settings, strategies as st

    models = {}

    @settings(max_examples=12, deadline=None)
    @given(chunk=st.sampled_from([4, 8]), n_sum=st.sampled_from([1, 2]), window=st.integers(0, 3),
           prompt_len=st.integers(1, 30), steps=st.integers(1, 20), second=st.integers(1, 12))
    def run(chunk, n_sum, window, prompt_len, steps, second):
        key = (chunk, n_sum, window)
        if key not in models:
            models[key] = _model(chunk, n_sum, window, layers=2, freq=[1, 0])
        model = models[key]
        eng = KsaInferenceEngine(model, max_len=64, batch=1)
        model.drop_partial_summary = True
        g = torch.Generator().manual_seed(prompt_len * 31 + steps)
        for plen, n in ((prompt_len, steps), (second, 3)):       # the second round checks that prefill resets the state
            seq = torch.randint(0, model.config.vocab_size, (1, plen), generator=g)
            logits = eng.prefill(seq)
            for _ in range(n):
                with torch.no_grad():
                    full = model(seq)[:, -1].float()
                assert torch.allclose(logits, full, atol=3e-4, rtol=1e-3)
                nxt = full.argmax(-1)
                seq = torch.cat([seq, nxt[:, None]], dim=1)
                logits = eng.decode_step(nxt)

    run()


def test_sampling_restricts_to_top_k_and_top_p_and_stops_at_eos():
    from ksa_b200.inference.engine import sample_next
    logits = torch.tensor([[4.0, 3.0, 2.0, 1.0, 0.0, -1.0]]).repeat(64, 1)
    g = torch.Generator().manual_seed(0)
    assert sample_next(logits).tolist() == [0] * 64                                   # greedy
    assert set(sample_next(logits, 1.0, top_k=2, generator=g).tolist()) <= {0, 1}
    # softmax mass: 0.64, 0.24, 0.09, ...: top_p = 0.7 keeps tokens 0 and 1
    assert set(sample_next(logits, 1.0, top_p=0.7, generator=g).tolist()) <= {0, 1}
    assert set(sample_next(logits, 1.0, top_p=0.5, generator=g).tolist()) == {0}
    assert len(set(sample_next(logits, 5.0, generator=g).tolist())) > 2               # a hot distribution spreads
    model = _model(8, 1, 2, layers=2, freq=[1, 0])
    eng = KsaInferenceEngine(model, max_len=64, batch=2)
    prompt = torch.randint(0, 128, (2, 9))
    first = eng.generate(prompt, 3)[:, 9]
    out = eng.generate(prompt, 12, eos_id=int(first[0]))
    assert out.shape[1] <= 21 and (out[0, 9:] == int(first[0])).all()                   # a finished row keeps emitting eos
    s1 = eng.generate(prompt, 6, temperature=0.8, top_k=20, generator=torch.Generator().manual_seed(5))
    s2 = eng.generate(prompt, 6, temperature=0.8, top_k=20, generator=torch.Generator().manual_seed(5))
    assert torch.equal(s1, s2)


@pytest.mark.parametrize("lengths", [(21, 13), (16, 16), (5, 30)])
def test_unequal_prompt_lengths_decode_like_each_sequence_alone(lengths):
    """A batch whose prompts differ in length (right-padded) is prefilled group by group and then decoded together,
    every sequence at its own chunk phase; every step equals the whole-sequence recompute of that sequence."""
    model = _model(8, 1, 2)
    B, new = len(lengths), 20
    torch.manual_seed(3)
    Lmax = max(lengths)
    prompt = torch.randint(0, model.config.vocab_size, (B, Lmax))
    eng = KsaInferenceEngine(model, max_len=Lmax + new + 4, batch=B)
    seqs = [prompt[i, :l] for i, l in enumerate(lengths)]
    logits = eng.prefill(prompt, lengths=list(lengths), batch_chunk=1)
    model.drop_partial_summary = True
    for step in range(new):
        with torch.no_grad():
            full = torch.stack([model(s[None])[0, -1].float() for s in seqs])
        assert torch.allclose(logits, full, atol=2e-4, rtol=1e-3), (step, (logits - full).abs().max())
        nxt = full.argmax(-1)
        seqs = [torch.cat([s, n[None]]) for s, n in zip(seqs, nxt)]
        logits = eng.decode_step(nxt)


def test_cache_grows_when_a_sequence_outlives_its_capacity():
    """``max_len`` is only the initial capacity: a prompt longer than it, and decoding past it, re-allocate the caches
    (text of full layers, summary region of summary layers) and keep their contents."""
    model = _model(4, 1, 2)
    torch.manual_seed(4)
    prompt = torch.randint(0, model.config.vocab_size, (2, 10))
    small = KsaInferenceEngine(model, max_len=8, batch=2)        # smaller than the prompt
    big = KsaInferenceEngine(model, max_len=128, batch=2)
    a, b = small.prefill(prompt), big.prefill(prompt)
    assert small.max_len >= 10
    for step in range(40):                                       # crosses the grown capacity more than once
        assert torch.allclose(a, b, atol=1e-5), step
        nxt = b.argmax(-1)
        a, b = small.decode_step(nxt), big.decode_step(nxt)
    assert small.max_len >= 50 and small.max_len < 128


def test_decode_ops_fall_back_to_their_unfused_forms_on_cpu():
    """The two fused decode operators (projection + SwiGLU, QK-norm + RoPE + cache append) have plain PyTorch
    fall-backs that the CPU engine runs: they must equal the separate operators."""
    from ksa_b200 import ops
    torch.manual_seed(7)
    x, w13 = torch.randn(3, 32), torch.randn(2 * 24, 32) * 0.2
    assert torch.allclose(ops.linear_swiglu(x, w13), ops.swiglu(ops.linear(x, w13)), atol=1e-6)
    Hq, Hkv, D, cap = 4, 2, 16, 9
    qkv = torch.randn(5, (Hq + 2 * Hkv) * D)
    qw, kw = 1 + 0.1 * torch.randn(D), 1 + 0.1 * torch.randn(D)
    pos = torch.tensor([3, 11, 0, 7, 5], dtype=torch.int32)
    slots = torch.tensor([4, -1, 8], dtype=torch.int32)          # three sequences; the second is not cached
    kc, vc = torch.zeros(3, Hkv, cap, D), torch.zeros(3, Hkv, cap, D)
    out = ops.qk_norm_rope_decode(qkv, qw, kw, pos, Hq, Hkv, D, 1e4, 1e-6, False, kc, vc, slots)
    expect = ops.qk_norm_rope_packed(qkv, qw, kw, pos, Hq, Hkv, D, 1e4, 1e-6, False)
    assert torch.equal(out, expect)
    assert torch.equal(kc[0, :, 4], expect[0, Hq * D:(Hq + Hkv) * D].view(Hkv, D))
    assert torch.equal(vc[2, :, 8], expect[2, (Hq + Hkv) * D:].view(Hkv, D))
    assert kc[1].abs().sum() == 0 and vc[1].abs().sum() == 0
