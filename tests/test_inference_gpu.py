"""Decode attention / cache kernels and the inference engine on the GPU against the CPU formulas."""
import copy

import pytest
import torch

from ksa_b200 import ops
from ksa_b200.config import get_preset
from ksa_b200.inference import KsaInferenceEngine
from ksa_b200.inference.engine import _cache_append, _cache_move, _decode_attention
from ksa_b200.models import get_model_class
from ksa_b200.ops import _lib, reference as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,Tq,Hq,Hkv,D,cap", [(2, 1, 8, 2, 128, 1500), (1, 2, 4, 2, 64, 300), (3, 1, 16, 8, 128, 9000),
                                               (2, 2, 8, 2, 128, 777), (2, 3, 8, 2, 128, 2200), (1, 2, 32, 4, 128, 640),
                                               (4, 1, 32, 8, 128, 131)])
def test_decode_attention_kernel(B, Tq, Hq, Hkv, D, cap):
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, Tq, Hq, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, Hkv, cap, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, Hkv, cap, D, device="cuda", generator=g).to(torch.bfloat16)
    start = torch.randint(0, cap // 4, (B, Tq), device="cuda", dtype=torch.int32)
    length = torch.randint(1, cap // 2, (B, Tq), device="cuda", dtype=torch.int32)
    out = _decode_attention(q, k, v, start, length, D ** -0.5)
    _lib.check_status()
    for t in range(Tq):
        expect = ref.decode_attention(q[:, t:t + 1].float(), k.float(), v.float(), length[:, t].long(), start[:, t].long(), D ** -0.5)
        err = (out[:, t:t + 1].float() - expect).norm() / expect.norm()
        assert err < 1.5e-2, (t, err)


def test_cache_append_and_move():
    B, T, H, D, cap = 2, 3, 2, 128, 64
    k_new = torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16)
    v_new = torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16)
    kc = torch.zeros(B, H, cap, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.tensor([[5, -1, 7], [0, 63, 2]], device="cuda", dtype=torch.int32)
    _cache_append(k_new, v_new, kc, vc, slots)
    assert torch.equal(kc[0, :, 5], k_new[0, 0]) and torch.equal(vc[1, :, 63], v_new[1, 1])
    assert kc[0, :, 6].abs().sum() == 0
    src = torch.tensor([5, 0], device="cuda", dtype=torch.int32)
    dst = torch.tensor([20, 30], device="cuda", dtype=torch.int32)
    en = torch.tensor([1, 0], device="cuda", dtype=torch.int32)
    _cache_move(kc, vc, src, dst, en, 3)
    assert torch.equal(kc[0, :, 20:23], kc[0, :, 5:8]) and kc[1, :, 30:33].abs().sum() == 0
    _lib.check_status()


@pytest.mark.parametrize("rows,cached,interleaved", [(1, 1, False), (4, 4, False), (6, 4, True), (18, 16, False)])
def test_decode_norm_rope_with_cache_append(rows, cached, interleaved):
    """The decode form of QK-norm + RoPE (one warp per row and head, K / V of the first ``cached`` rows written into
    the cache) against the training form followed by a separate append."""
    Hq, Hkv, D, cap = 8, 2, 128, 40
    g = torch.Generator(device="cuda").manual_seed(rows)
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * D, device="cuda", generator=g).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    pos = torch.randint(0, 5000, (rows,), device="cuda", generator=g).int()
    slots = torch.randint(0, cap, (cached,), device="cuda", generator=g).int()
    slots[-1] = -1                                                       # this sequence's row is not cached
    kc = torch.zeros(cached, Hkv, cap, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    with torch.no_grad():
        expect = ops.qk_norm_rope_packed(qkv, qw, kw, pos, Hq, Hkv, D, 1e6, 1e-6, interleaved)
        out = ops.qk_norm_rope_decode(qkv, qw, kw, pos, Hq, Hkv, D, 1e6, 1e-6, interleaved, kc, vc, slots)
    assert torch.equal(out, expect)
    ke, ve = torch.zeros_like(kc), torch.zeros_like(vc)
    for i, s_ in enumerate(slots.tolist()):
        if s_ >= 0:
            ke[i, :, s_] = expect[i, Hq * D:(Hq + Hkv) * D].view(Hkv, D)
            ve[i, :, s_] = expect[i, (Hq + Hkv) * D:].view(Hkv, D)
    assert torch.equal(kc, ke) and torch.equal(vc, ve)
    _lib.check_status()


def test_engine_matches_cpu_engine():
    cfg = get_preset("qwen3-ksa-tiny").merge({"head_dim": 128, "num_heads": 4, "num_kv_heads": 2, "embed_dim": 256,
                                               "summary_chunk_size": 128, "summary_sliding_chunk_num": 2})
    torch.manual_seed(0)
    cpu_model = get_model_class(cfg.model_class)(cfg)
    cpu_model.init_weights(seed=0)
    with torch.no_grad():
        for p in cpu_model.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    gpu_model = copy.deepcopy(cpu_model).cuda().to(torch.bfloat16)
    # Prompts of 300 and 250 tokens: sequence 1 closes chunks at steps 6 and 134, sequence 0 at step 84, so the
    # boundary form of the step runs eagerly once, is captured, and is replayed; the GPU engine starts with room for
    # 400 tokens and has to grow its caches (and capture its graphs again) on the way.
    B, lengths, new = 2, [300, 250], 140
    prompt = torch.randint(0, cfg.vocab_size, (B, max(lengths)))
    e_cpu = KsaInferenceEngine(cpu_model, max_len=512, batch=B)
    e_gpu = KsaInferenceEngine(gpu_model, max_len=400, batch=B)
    lc, lg = e_cpu.prefill(prompt, lengths=lengths), e_gpu.prefill(prompt.cuda(), lengths=lengths)
    for step in range(new):
        err = (lg.cpu() - lc).norm() / lc.norm()
        assert err < 5e-2, (step, err)
        nxt = lc.argmax(-1)
        lc, lg = e_cpu.decode_step(nxt), e_gpu.decode_step(nxt.cuda())
    assert e_gpu.max_len > 400 and set(e_gpu._graphs) == {False, True}
    _lib.check_status()


def test_hf_generate_on_gpu_runs_on_the_engine_behind_past_key_values():
    """The HF model on a GPU with this package importable: stock ``generate`` prefills and decodes through
    ``KsaInferenceEngine`` (the cache object carries it) and returns the engine's own greedy tokens."""
    from ksa_b200.hf.modeling_qwen3sa import KsaRingBufferCache, Qwen3ForCausalLM, Qwen3SAConfig
    cfg = Qwen3SAConfig(vocab_size=513, hidden_size=256, intermediate_size=512, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=128, summary_token_begin=512,
                        summary_chunk_size=128, summary_token_num=1, summary_sliding_chunk_num=2,
                        summary_layer_freq="([1]*3+[0]*1)*1", max_position_embeddings=4096)
    torch.manual_seed(0)
    hf = Qwen3ForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() >= 2:
                p.mul_(3.0)
    hf = hf.cuda().to(torch.bfloat16)
    prompt = torch.randint(0, 512, (2, 200), device="cuda")
    before = _lib.launch_count()
    out = hf.generate(prompt, max_new_tokens=80, do_sample=False, eos_token_id=-1)      # crosses the boundary at 256
    assert _lib.launch_count() > before, "the sm_100a kernels did not run"
    want = KsaInferenceEngine(hf.framework_model(), max_len=512, batch=2).generate(prompt, 80)
    assert torch.equal(out, want)
    step = hf(prompt, use_cache=True)
    assert isinstance(step.past_key_values, KsaRingBufferCache) and step.past_key_values.engine is not None
    assert step.logits.shape == (2, 1, 513)
    _lib.check_status()
