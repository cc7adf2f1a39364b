"""Generic layer modules on CPU against direct PyTorch statements of the same math."""
import math

import torch

from ksa_b200 import layers as L


def test_rms_norm_and_fp32_layer_norm():
    x = torch.randn(3, 5, 16)
    n = L.RMSNorm(16, eps=1e-5)
    with torch.no_grad():
        n.scale.copy_(torch.rand(16) + 0.5)
    ref = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * n.scale
    torch.testing.assert_close(n(x), ref)
    ln = L.Fp32LayerNorm(16)
    xb = x.bfloat16()
    assert ln(xb).dtype == torch.bfloat16
    torch.testing.assert_close(ln(xb).float(), torch.nn.functional.layer_norm(xb.float(), (16,)), atol=1e-2, rtol=1e-2)


def test_rope_variants_rotate_pairs_and_follow_input_pos():
    x = torch.randn(2, 6, 3, 8)
    half, inter = L.RotaryPositionalEmbeddings(8, 32, 100.0), L.LlamaRotaryPositionalEmbeddings(8, 32, 100.0)
    pos = torch.tensor([[3, 4, 5, 6, 7, 8], [0, 1, 2, 3, 4, 5]])
    y = half(x, input_pos=pos)
    theta = 1.0 / (100.0 ** (torch.arange(0, 8, 2).float() / 8))
    ang = pos[..., None].float() * theta
    x1, x2 = x[..., :4], x[..., 4:]
    ref = torch.cat([x1 * ang.cos()[:, :, None] - x2 * ang.sin()[:, :, None],
                     x2 * ang.cos()[:, :, None] + x1 * ang.sin()[:, :, None]], -1)
    torch.testing.assert_close(y, ref)
    torch.testing.assert_close(half(x)[1], y[1])                  # default positions are 0..s-1
    # the interleaved variant is the half-split one under a permutation of the feature axis
    perm = torch.cat([torch.arange(0, 8, 2), torch.arange(1, 8, 2)])
    torch.testing.assert_close(inter(x, input_pos=pos)[..., perm], half(x[..., perm], input_pos=pos))
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1))   # rotations keep norms


def test_feed_forward_tied_linear_kv_cache():
    ff = L.FeedForward(8, 16)
    x = torch.randn(2, 3, 8)
    ref = ff.w2(torch.nn.functional.silu(ff.w1(x)) * ff.w3(x))
    torch.testing.assert_close(ff(x), ref, atol=1e-5, rtol=1e-5)
    emb = torch.nn.Embedding(11, 8)
    tied = L.TiedLinear(emb)
    assert len(list(tied.parameters())) == 0
    torch.testing.assert_close(tied(x), x @ emb.weight.t(), atol=1e-5, rtol=1e-5)
    cache = L.KVCache(2, 8, 2, 4, dtype=torch.float32)
    k, v = torch.randn(2, 3, 2, 4), torch.randn(2, 3, 2, 4)
    cache.update(k, v)
    k2, v2 = cache.update(k[:, :1], v[:, :1])
    assert k2.shape == (2, 4, 2, 4) and torch.equal(k2[:, :3], k) and torch.equal(v2[:, 3:], v[:, :1])
    cache.reset()
    assert cache.size == 0


def _decoder(dim=16, heads=4, kv=2, hd=4, layers=2, vocab=50):
    def block():
        attn = L.MultiHeadAttention(dim, heads, kv, hd, pos_embeddings=L.RotaryPositionalEmbeddings(hd, 64),
                                    q_norm=L.RMSNorm(hd), k_norm=L.RMSNorm(hd), max_seq_len=64)
        return L.TransformerSelfAttentionLayer(attn, L.FeedForward(dim, 32), L.RMSNorm(dim), L.RMSNorm(dim))
    emb = torch.nn.Embedding(vocab, dim)
    return L.TransformerDecoder(emb, [block() for _ in range(layers)], 64, heads, hd, L.RMSNorm(dim), L.TiedLinear(emb))


def test_decoder_incremental_decoding_matches_full_forward():
    torch.manual_seed(0)
    dec = _decoder().eval()
    toks = torch.randint(0, 50, (2, 9))
    with torch.no_grad():
        full = dec(toks)
        dec.setup_caches(2, torch.float32)
        outs = [dec(toks[:, :5], input_pos=torch.arange(5)[None].expand(2, -1))]
        for t in range(5, 9):
            outs.append(dec(toks[:, t:t + 1], input_pos=torch.full((2, 1), t)))
    torch.testing.assert_close(torch.cat(outs, dim=1), full, atol=1e-4, rtol=1e-4)
    dec.reset_caches()
    dec.skip_output_layer = True
    for l in dec.layers:
        l.attn.cache_enabled = False
    assert dec(toks).shape == (2, 9, 16)


def test_cross_attention_layer_and_backends():
    torch.manual_seed(0)
    attn = L.MultiHeadAttention(16, 4, 4, 4, is_causal=False, attention_backend="eager")
    layer = L.TransformerCrossAttentionLayer(attn, L.FeedForward(16, 32), L.RMSNorm(16), L.RMSNorm(16))
    x, enc = torch.randn(2, 5, 16), torch.randn(2, 7, 16)
    assert torch.equal(layer(x), x)
    assert layer(x, encoder_input=enc).shape == x.shape
    q, k, v = torch.randn(1, 6, 4, 8), torch.randn(1, 6, 2, 8), torch.randn(1, 6, 2, 8)
    o = L.get_attention_backend("flash_attention_2")(q, k, v, window=3)
    kk, vv = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) / math.sqrt(8)
    i = torch.arange(6)
    m = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < 3)
    p = s.masked_fill(~m, float("-inf")).softmax(-1)
    torch.testing.assert_close(o, torch.einsum("bhqk,bkhd->bqhd", p, vv), atol=1e-5, rtol=1e-5)


def test_summary_batch_builder_matches_python_loop():
    ids = torch.arange(1, 23)[None].repeat(2, 1)
    sb = L.build_summary_batch(ids, chunk=8, n_sum=2, summary_token_begin=100, cu_seqlens=torch.tensor([0, 22]))
    expect = []
    for c in range(0, 22, 8):
        expect += list(range(c + 1, min(c + 8, 22) + 1)) + [100, 101]
    assert sb.input_ids[0].tolist() == expect
    assert sb.summary_mask.tolist() == [t >= 100 for t in expect]
    assert sb.position_ids.shape == sb.input_ids.shape
    assert sb.cu_seqlens.tolist() == [0, len(expect)]
