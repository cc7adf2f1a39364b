"""HuggingFace ``trust_remote_code`` model: Qwen3 + Kwai Summary Attention, with its ring-buffer KV cache.

Counterpart of ``examples/pretrain/hf_template/modeling_qwen3sa.py`` of the reference.  The module tree carries the
parameters under the HF names written by the converter (``model.layers.{i}.self_attn.q_proj_summary.weight`` ...; the
summary embedding rows are the tail of ``embed_tokens``).

Generation runs through the stock ``GenerationMixin.generate`` (stopping criteria, streamers, logits processors,
sampling and beam search are the library's): ``forward`` takes ``past_key_values`` / ``use_cache``, the first call
prefills the prompt and builds a :class:`KsaRingBufferCache`, later calls decode one token against it, and
``prepare_inputs_for_generation`` appends the ``S`` summary tokens (and their position ids) to the step whose text
token completes a chunk (``modeling_qwen3sa.py:1430-1560`` of the reference template).  The cache holds, per
summary-attention layer, one contiguous K and one V buffer laid out as

    [ scratch (S) | current chunk (C, filled right -> left) | sliding-chunk ring (W*C) | summaries (append) ]

(``modeling_qwen3sa.py:85-505`` of the reference template) and, per full-attention layer, an append-only text
buffer.  Everything in this file is plain PyTorch and needs no other package.  Where the ``ksa_b200`` package is
importable and the model sits on a GPU, the same ``forward`` hands prefill and decode to its ``KsaInferenceEngine``
(sm_100a kernels, the same cache layout with device-resident counters) behind the same ``past_key_values`` contract.

Unlike the reference template, a true summary / full-attention hybrid (``summary_layer_freq``), batch sizes above
one (equal prompt lengths, no padding) and ``S > 1`` with causal summary tokens are supported, and full-attention
layers behave identically in prefill and decode.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from transformers import PretrainedConfig, PreTrainedModel
from transformers.cache_utils import Cache, CacheLayerMixin
from transformers.generation import GenerationMixin
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast

try:  # stand-alone checkpoint directory: the helper sits next to this file
    from .summary_context import SummaryContext, parse_pattern
except ImportError:  # pragma: no cover
    from summary_context import SummaryContext, parse_pattern


class Qwen3SAConfig(PretrainedConfig):
    model_type = "qwen3sa"

    def __init__(self, vocab_size=151937, hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
                 num_attention_heads=16, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
                 max_position_embeddings=131072, tie_word_embeddings=False, use_summary_attention=True,
                 summary_token_begin=151936, summary_chunk_size=128, summary_token_num=1, summary_sliding_chunk_num=8,
                 summary_layer_freq=0, summary_chunk_position_ids_type="origin",
                 summary_token_position_ids_type="last_chunk_slice_right", summary_independent_parameters=True,
                 summary_independent_attention_layernorm=False, summary_independent_qk_norm=False,
                 truncate_predict_nums=0, **kwargs):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_hidden_layers = num_hidden_layers
        self.num_attention_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads
        self.head_dim = head_dim
        self.rms_norm_eps = rms_norm_eps
        self.rope_theta = rope_theta
        self.max_position_embeddings = max_position_embeddings
        self.use_summary_attention = use_summary_attention
        self.summary_token_begin = summary_token_begin
        self.summary_chunk_size = summary_chunk_size
        self.summary_token_num = summary_token_num
        self.summary_sliding_chunk_num = summary_sliding_chunk_num
        self.summary_layer_freq = summary_layer_freq
        self.summary_chunk_position_ids_type = summary_chunk_position_ids_type
        self.summary_token_position_ids_type = summary_token_position_ids_type
        self.summary_independent_parameters = summary_independent_parameters
        self.summary_independent_attention_layernorm = summary_independent_attention_layernorm
        self.summary_independent_qk_norm = summary_independent_qk_norm
        # logits (and sampled tokens) are restricted to the first N vocabulary entries; 0 keeps the text vocabulary
        # (the reference's template reads the same attribute, examples/pretrain/hf_template/modeling_qwen3sa.py:1402)
        self.truncate_predict_nums = truncate_predict_nums
        super().__init__(tie_word_embeddings=tie_word_embeddings, **kwargs)

    # ---- per-layer views -------------------------------------------------------------------------
    def layer_is_summary(self) -> List[bool]:
        n = self.num_hidden_layers
        if not self.use_summary_attention:
            return [False] * n
        f = self.summary_layer_freq
        if isinstance(f, int):
            return [True] * n if f == 0 else [(i % f == 0) for i in range(n)]
        return [bool(v) for v in parse_pattern(f, n)]

    def layer_window(self) -> List[int]:
        return parse_pattern(self.summary_sliding_chunk_num, self.num_hidden_layers)

    @property
    def text_vocab_size(self) -> int:
        """Rows of ``embed_tokens`` that are ordinary tokens (the summary embedding rows follow them)."""
        if self.use_summary_attention and self.summary_independent_parameters:
            return int(self.summary_token_begin)
        return int(self.vocab_size)


class _Norm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


class _Attention(nn.Module):
    def __init__(self, cfg: Qwen3SAConfig, is_summary: bool):
        super().__init__()
        D, Hq, Hkv, Dh = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.q_proj = nn.Linear(D, Hq * Dh, bias=False)
        self.k_proj = nn.Linear(D, Hkv * Dh, bias=False)
        self.v_proj = nn.Linear(D, Hkv * Dh, bias=False)
        self.o_proj = nn.Linear(Hq * Dh, D, bias=False)
        self.q_norm = _Norm(Dh, cfg.rms_norm_eps)
        self.k_norm = _Norm(Dh, cfg.rms_norm_eps)
        if is_summary and cfg.summary_independent_parameters:
            self.q_proj_summary = nn.Linear(D, Hq * Dh, bias=False)
            self.k_proj_summary = nn.Linear(D, Hkv * Dh, bias=False)
            self.v_proj_summary = nn.Linear(D, Hkv * Dh, bias=False)
            if cfg.summary_independent_qk_norm:
                self.q_norm_summary = _Norm(Dh, cfg.rms_norm_eps)
                self.k_norm_summary = _Norm(Dh, cfg.rms_norm_eps)


class _Mlp(nn.Module):
    def __init__(self, cfg: Qwen3SAConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class _Layer(nn.Module):
    def __init__(self, cfg: Qwen3SAConfig, is_summary: bool, window: int):
        super().__init__()
        self.is_summary, self.window = is_summary, window
        self.input_layernorm = _Norm(cfg.hidden_size, cfg.rms_norm_eps)
        if is_summary and cfg.summary_independent_parameters and cfg.summary_independent_attention_layernorm:
            self.input_layernorm_summary = _Norm(cfg.hidden_size, cfg.rms_norm_eps)
        self.self_attn = _Attention(cfg, is_summary)
        self.post_attention_layernorm = _Norm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mlp = _Mlp(cfg)


def _rope(x, pos, theta):
    """Half-split rotary on ``x`` ``[B, T, H, D]`` with positions ``pos`` ``[T]``."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D // 2, device=x.device, dtype=torch.float32) * 2.0 / D))
    ang = pos.float()[:, None] * inv
    c, s = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    xf = x.float()
    x1, x2 = xf[..., :D // 2], xf[..., D // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


def _attend(q, k, v, mask):
    """``q`` ``[B,Tq,H,D]``, ``k``/``v`` ``[B,Tk,Hkv,D]``, ``mask`` ``[Tq,Tk]``; fp32 softmax."""
    rep = q.shape[2] // k.shape[2]
    k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(q.shape[-1])
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    return torch.einsum("bhqk,bkhd->bqhd", p, v.float()).to(q.dtype)


def _attend_slice(q, k, v):
    """One query token per sequence over a cache slice, no mask: ``q`` ``[B, Hq, D]``, ``k``/``v`` ``[B, Hkv, n, D]``."""
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    qg = q.view(B, Hkv, Hq // Hkv, D).float()
    s = torch.einsum("bhgd,bhnd->bhgn", qg, k.float()) / math.sqrt(D)
    o = torch.einsum("bhgn,bhnd->bhgd", torch.softmax(s, -1), v.float())
    return o.reshape(B, Hq * D).to(q.dtype)


# =================================================================================================== KV cache
class KsaCacheLayer(CacheLayerMixin):
    """KV buffers of one layer: ``keys`` / ``values`` ``[B, Hkv, capacity, D]``, K stored after RoPE.

    ``kind == "summary"``: ``[scratch S | current chunk C | ring W*C | summaries ...]``; ``kind == "full"``: text rows
    appended left to right.  The counters (text length, fill of the current chunk, finished chunks) live in the
    owning :class:`KsaRingBufferCache`; all layers advance in lock step."""

    is_compileable = False
    is_sliding = False

    def __init__(self, kind: str, chunk: int, n_sum: int, window: int, owner: "KsaRingBufferCache"):
        super().__init__()
        self.kind, self.C, self.S, self.W = kind, chunk, n_sum, window
        self.owner = owner

    # ---- layout -------------------------------------------------------------------------------------
    @property
    def text0(self) -> int:       # first slot after the current-chunk region = first ring slot
        return self.S + self.C

    @property
    def sum0(self) -> int:        # first slot of the summary region
        return self.S + self.C + self.W * self.C

    def _ensure(self, like: torch.Tensor, need: int) -> None:
        """Allocate on first use and grow by doubling (``like``: a ``[B, Hkv, *, D]`` tensor for shape and dtype)."""
        if not self.is_initialized:
            B, H, _, D = like.shape
            cap = max(need, (self.sum0 + 64 * max(self.S, 1)) if self.kind == "summary" else 256)
            self.keys = like.new_zeros(B, H, cap, D)
            self.values = like.new_zeros(B, H, cap, D)
            self.dtype, self.device = like.dtype, like.device
            self.is_initialized = True
        elif self.keys.shape[2] < need:
            cap = max(need, 2 * self.keys.shape[2])
            pad = cap - self.keys.shape[2]
            self.keys = torch.cat([self.keys, self.keys.new_zeros(*self.keys.shape[:2], pad, self.keys.shape[3])], 2)
            self.values = torch.cat([self.values, self.values.new_zeros(*self.values.shape[:2], pad, self.values.shape[3])], 2)

    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        self._ensure(key_states, 0)

    # ---- prefill ------------------------------------------------------------------------------------
    def fill(self, k_t, v_t, k_s, v_s) -> None:
        """Build the decode-time layout from the rotated keys / values of a prompt: ``k_t``/``v_t`` ``[B, L, Hkv, D]``,
        ``k_s``/``v_s`` ``[B, n_chunks*S, Hkv, D]`` (None for a full-attention layer)."""
        L = k_t.shape[1]
        kt, vt = k_t.transpose(1, 2), v_t.transpose(1, 2)            # [B, Hkv, L, D]
        if self.kind == "full":
            self._ensure(kt, L + 64)
            self.keys[:, :, :L], self.values[:, :, :L] = kt, vt
            return
        C, S, W = self.C, self.S, self.W
        n_full, rem = L // C, L % C
        self._ensure(kt, self.sum0 + (n_full + 64) * S)
        if rem:                                                      # current chunk, newest token leftmost
            self.keys[:, :, self.text0 - rem:self.text0] = kt[:, :, n_full * C:].flip(2)
            self.values[:, :, self.text0 - rem:self.text0] = vt[:, :, n_full * C:].flip(2)
        for c in range(max(0, n_full - W), n_full):                  # the last W finished chunks, one ring slot each
            dst = self.text0 + (c % W) * C
            self.keys[:, :, dst:dst + C] = kt[:, :, c * C:(c + 1) * C].flip(2)
            self.values[:, :, dst:dst + C] = vt[:, :, c * C:(c + 1) * C].flip(2)
        if n_full and S:
            self.keys[:, :, self.sum0:self.sum0 + n_full * S] = k_s.transpose(1, 2)
            self.values[:, :, self.sum0:self.sum0 + n_full * S] = v_s.transpose(1, 2)

    # ---- decode -------------------------------------------------------------------------------------
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
        """Store the K / V of ONE new text token (``[B, Hkv, 1, D]``) and return the slice it attends (no mask)."""
        o = self.owner
        if self.kind == "full":
            self._ensure(key_states, o.text_len + 1)
            self.keys[:, :, o.text_len] = key_states[:, :, 0]
            self.values[:, :, o.text_len] = value_states[:, :, 0]
            return self.keys[:, :, :o.text_len + 1], self.values[:, :, :o.text_len + 1]
        self._ensure(key_states, self.sum0 + (o.n_chunks + 2) * self.S)
        slot = self.text0 - 1 - o.cur_len
        self.keys[:, :, slot] = key_states[:, :, 0]
        self.values[:, :, slot] = value_states[:, :, 0]
        if o.n_chunks < self.W:      # ring not full yet: its valid part is contiguous, no summary is visible
            end = self.text0 + o.n_chunks * self.C
        else:                        # whole ring + the summaries of the chunks older than the window
            end = self.sum0 + (o.n_chunks - self.W) * self.S
        return self.keys[:, :, slot:end], self.values[:, :, slot:end]

    def update_summary(self, k_s: torch.Tensor, v_s: torch.Tensor):
        """Chunk boundary: store the ``S`` summary tokens' K / V (``[B, Hkv, S, D]``) in the scratch region, summary
        ``j`` at slot ``S-1-j``, and return per summary token the slice it attends: itself, the summaries before it and
        the chunk's text (the current-chunk region is full at this point)."""
        S = self.S
        self.keys[:, :, :S] = k_s.flip(2)
        self.values[:, :, :S] = v_s.flip(2)
        return [(self.keys[:, :, S - 1 - j:self.text0], self.values[:, :, S - 1 - j:self.text0]) for j in range(S)]

    def flush_chunk(self) -> None:
        """Chunk boundary, after attention: the finished chunk goes to its ring slot, its summaries to the summary region."""
        o = self.owner
        dst = self.text0 + (o.n_chunks % self.W) * self.C
        self.keys[:, :, dst:dst + self.C] = self.keys[:, :, self.S:self.text0]
        self.values[:, :, dst:dst + self.C] = self.values[:, :, self.S:self.text0]
        at = self.sum0 + o.n_chunks * self.S
        self.keys[:, :, at:at + self.S] = self.keys[:, :, :self.S].flip(2)
        self.values[:, :, at:at + self.S] = self.values[:, :, :self.S].flip(2)

    # ---- container protocol -------------------------------------------------------------------------
    def get_seq_length(self) -> int:
        return self.owner.text_len

    def get_mask_sizes(self, query_length: int) -> Tuple[int, int]:
        return self.owner.text_len + query_length, 0

    def get_max_cache_shape(self) -> int:
        return -1

    def crop(self, max_length: int) -> None:
        raise NotImplementedError("the ring-buffer cache cannot be rolled back (assisted / contrastive decoding)")

    def batch_repeat_interleave(self, repeats: int) -> None:
        if self.is_initialized:
            self.keys = self.keys.repeat_interleave(repeats, dim=0)
            self.values = self.values.repeat_interleave(repeats, dim=0)

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        if self.is_initialized:
            self.keys, self.values = self.keys[indices, ...], self.values[indices, ...]


class KsaRingBufferCache(Cache):
    """``past_key_values`` of the Qwen3-KSA model: one :class:`KsaCacheLayer` per decoder layer plus the counters that
    all layers share.  Sequences of a batch advance together (equal prompt lengths, no padding)."""

    def __init__(self, config: "Qwen3SAConfig"):
        use_sum = config.use_summary_attention and config.summary_token_num > 0
        is_sum, win = config.layer_is_summary(), config.layer_window()
        C = config.summary_chunk_size if use_sum else 1
        S = config.summary_token_num if use_sum else 0
        layers = [KsaCacheLayer("summary" if (use_sum and is_sum[i]) else "full", C, S, win[i], self)
                  for i in range(config.num_hidden_layers)]
        super().__init__(layers=layers)
        self.chunk, self.n_sum, self.use_summary = C, S, use_sum
        self.text_len = 0     # text tokens stored
        self.cur_len = 0      # text tokens in the unfinished chunk
        self.n_chunks = 0     # finished chunks (each has its S summaries stored)
        self.engine = None    # set when a ksa_b200 inference engine serves this cache instead of the layers above

    def boundary_due(self) -> bool:
        """True when the NEXT text token completes a chunk, i.e. its step also carries the S summary tokens."""
        return self.use_summary and self.cur_len == self.chunk - 1

    def advance(self) -> None:
        self.text_len += 1
        self.cur_len += 1
        if self.use_summary and self.cur_len == self.chunk:
            self.cur_len, self.n_chunks = 0, self.n_chunks + 1

    def set_prompt(self, length: int) -> None:
        self.text_len = length
        if self.use_summary:
            self.n_chunks, self.cur_len = length // self.chunk, length % self.chunk

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.text_len

    def reorder_cache(self, beam_idx: torch.LongTensor) -> None:
        if self.engine is not None:
            raise NotImplementedError("beam search is not available on the engine-backed cache")
        super().reorder_cache(beam_idx)


class Qwen3PreTrainedModel(PreTrainedModel):
    config_class = Qwen3SAConfig
    base_model_prefix = "model"
    _no_split_modules = ["_Layer"]
    supports_gradient_checkpointing = False

    def _init_weights(self, module):
        if isinstance(module, (nn.Linear, nn.Embedding)):
            module.weight.data.normal_(0.0, 0.02)


class Qwen3Model(Qwen3PreTrainedModel):
    """Decoder stack in plain PyTorch: two-stream prefill over a whole sequence, one-token decode on the ring buffer."""

    def __init__(self, config: Qwen3SAConfig):
        super().__init__(config)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        is_sum, win = config.layer_is_summary(), config.layer_window()
        self.layers = nn.ModuleList([_Layer(config, is_sum[i], win[i]) for i in range(config.num_hidden_layers)])
        self.norm = _Norm(config.hidden_size, config.rms_norm_eps)
        self.post_init()

    def get_input_embeddings(self):
        return self.embed_tokens

    # ---- helpers ------------------------------------------------------------------------------------
    def _use_summary(self) -> bool:
        return bool(self.config.use_summary_attention and self.config.summary_token_num > 0)

    def _summary_embeddings(self, B: int, device) -> torch.Tensor:
        cfg = self.config
        ids = torch.arange(cfg.summary_token_begin, cfg.summary_token_begin + cfg.summary_token_num, device=device)
        return self.embed_tokens(ids).unsqueeze(0).expand(B, -1, -1)

    def _summary_positions(self, chunk_idx: int, device) -> torch.Tensor:
        """Position ids of the S summary tokens of chunk ``chunk_idx`` (same rule as SummaryContext)."""
        cfg = self.config
        C, S = cfg.summary_chunk_size, cfg.summary_token_num
        j = torch.arange(S, device=device)
        if cfg.summary_token_position_ids_type == "zeros":
            return torch.zeros_like(j)
        start = chunk_idx * C
        if cfg.summary_token_position_ids_type == "last_chunk_slice_right":
            pos = start + ((j + 1) * C) // S - 1
        else:
            pos = start + (j * C) // S - 1
        return torch.clamp(pos, min=start)

    def _qkv(self, layer: "_Layer", h: torch.Tensor, pos: torch.Tensor, summary_rows: bool):
        """Projections, QK norm and RoPE of normalised rows ``h`` ``[B, T, D]`` -> q ``[B,T,Hq,Dh]``, k, v ``[B,T,Hkv,Dh]``."""
        cfg, a = self.config, layer.self_attn
        B, T, _ = h.shape
        Hq, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        own = summary_rows and hasattr(a, "q_proj_summary")
        q = (a.q_proj_summary if own else a.q_proj)(h).view(B, T, Hq, Dh)
        k = (a.k_proj_summary if own else a.k_proj)(h).view(B, T, Hkv, Dh)
        v = (a.v_proj_summary if own else a.v_proj)(h).view(B, T, Hkv, Dh)
        qn = getattr(a, "q_norm_summary", a.q_norm) if summary_rows else a.q_norm
        kn = getattr(a, "k_norm_summary", a.k_norm) if summary_rows else a.k_norm
        return _rope(qn(q), pos, cfg.rope_theta), _rope(kn(k), pos, cfg.rope_theta), v

    # ---- prefill: the whole sequence, dense two-stream masks ---------------------------------------------
    def _prefill(self, input_ids: torch.Tensor, cache: Optional[KsaRingBufferCache]) -> torch.Tensor:
        cfg = self.config
        B, L = input_ids.shape
        Hq, Dh = cfg.num_attention_heads, cfg.head_dim
        use_sum = self._use_summary()
        ctx = SummaryContext(L, cfg.summary_chunk_size if use_sum else max(L, 1), cfg.summary_token_num if use_sum else 0,
                             cfg.summary_chunk_position_ids_type, cfg.summary_token_position_ids_type)
        Ns = ctx.n_summary_rows if use_sum else 0
        dev = input_ids.device
        x_t = self.embed_tokens(input_ids)
        pos_t = ctx.text_position_ids(dev) if use_sum else torch.arange(L, device=dev)
        x_s = pos_s = None
        if Ns > 0:
            x_s = self._summary_embeddings(B, dev).repeat(1, ctx.n_chunks, 1)
            pos_s = ctx.summary_position_ids(dev)
        causal = torch.tril(torch.ones(L, L, dtype=torch.bool, device=dev))
        for li, layer in enumerate(self.layers):
            a = layer.self_attn
            if layer.is_summary and use_sum:
                q_t, k_t, v_t = self._qkv(layer, layer.input_layernorm(x_t), pos_t, False)
                k_s = v_s = None
                if Ns > 0:
                    n_s = getattr(layer, "input_layernorm_summary", layer.input_layernorm)
                    q_s, k_s, v_s = self._qkv(layer, n_s(x_s), pos_s, True)
                    tt, ts, st, ss = ctx.masks(layer.window, dev)
                    k_all, v_all = torch.cat([k_t, k_s], 1), torch.cat([v_t, v_s], 1)
                    o_t = _attend(q_t, k_all, v_all, torch.cat([tt, ts], 1))
                    o_s = _attend(q_s, k_all, v_all, torch.cat([st, ss], 1))
                    x_s = x_s + a.o_proj(o_s.reshape(B, Ns, Hq * Dh))
                    x_s = x_s + layer.mlp(layer.post_attention_layernorm(x_s))
                else:       # no finished chunk yet: causal attention inside the window
                    tt = ctx.masks(layer.window, dev)[0]
                    o_t = _attend(q_t, k_t, v_t, tt)
                x_t = x_t + a.o_proj(o_t.reshape(B, L, Hq * Dh))
                x_t = x_t + layer.mlp(layer.post_attention_layernorm(x_t))
                if cache is not None:
                    cache.layers[li].fill(k_t, v_t, k_s, v_s)
            else:  # full attention on the text rows; summary rows bypass the layer
                q, k, v = self._qkv(layer, layer.input_layernorm(x_t), pos_t, False)
                o = _attend(q, k, v, causal)
                x_t = x_t + a.o_proj(o.reshape(B, L, Hq * Dh))
                x_t = x_t + layer.mlp(layer.post_attention_layernorm(x_t))
                if cache is not None:
                    cache.layers[li].fill(k, v, None, None)
        if cache is not None:
            cache.set_prompt(L)
        return self.norm(x_t)

    # ---- decode: one text token (plus the S summary tokens when it completes a chunk) ---------------------
    def _decode_token(self, token: torch.Tensor, cache: KsaRingBufferCache) -> torch.Tensor:
        """``token`` ``[B]`` -> final hidden state of the text token ``[B, D]``; advances the cache by one position."""
        cfg = self.config
        B = token.shape[0]
        dev = token.device
        Hq, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        boundary = cache.boundary_due()
        t = cache.text_len
        pos_t = torch.tensor([t if cfg.summary_chunk_position_ids_type == "origin" or not cache.use_summary
                              else t % cache.chunk], device=dev)
        x_t = self.embed_tokens(token)[:, None, :]                       # [B, 1, D]
        x_s = pos_s = None
        if boundary:
            x_s = self._summary_embeddings(B, dev)                       # [B, S, D]
            pos_s = self._summary_positions(cache.n_chunks, dev)
        for li, layer in enumerate(self.layers):
            a, lc = layer.self_attn, cache.layers[li]
            q, k, v = self._qkv(layer, layer.input_layernorm(x_t), pos_t, False)
            k_att, v_att = cache.update(k.transpose(1, 2), v.transpose(1, 2), li)
            o_t = _attend_slice(q[:, 0], k_att, v_att)
            x_t = x_t + a.o_proj(o_t)[:, None, :]
            x_t = x_t + layer.mlp(layer.post_attention_layernorm(x_t))
            if boundary and lc.kind == "summary":
                n_s = getattr(layer, "input_layernorm_summary", layer.input_layernorm)
                q_s, k_s, v_s = self._qkv(layer, n_s(x_s), pos_s, True)
                slices = lc.update_summary(k_s.transpose(1, 2), v_s.transpose(1, 2))
                o_s = torch.stack([_attend_slice(q_s[:, j], *slices[j]) for j in range(len(slices))], 1)
                x_s = x_s + a.o_proj(o_s)
                x_s = x_s + layer.mlp(layer.post_attention_layernorm(x_s))
                lc.flush_chunk()
        cache.advance()
        return self.norm(x_t[:, 0])

    def forward(self, input_ids: torch.Tensor, past_key_values: Optional[KsaRingBufferCache] = None,
                use_cache: bool = False, attention_mask: Optional[torch.Tensor] = None, **_unused) -> BaseModelOutputWithPast:
        """Hidden states of the text tokens of ``input_ids``.  Without a (non-empty) cache the whole sequence is processed
        at once; with one, the tokens are decoded one after another against it.  Summary token ids that
        ``prepare_inputs_for_generation`` appended to a chunk-completing step are recognised and dropped: the model
        runs the summary tokens of a finished chunk itself."""
        if attention_mask is not None and attention_mask.ndim == 2 and not bool(attention_mask.bool().all()):
            raise NotImplementedError("padded batches are not supported: pass prompts of equal length without padding")
        cfg = self.config
        if past_key_values is not None and not isinstance(past_key_values, KsaRingBufferCache):
            if past_key_values.get_seq_length() != 0:
                raise TypeError("past_key_values must be a KsaRingBufferCache (or None / an empty cache on the first call)")
            past_key_values = None
        if past_key_values is None or past_key_values.get_seq_length() == 0:
            cache = (past_key_values or KsaRingBufferCache(cfg)) if use_cache else None
            return BaseModelOutputWithPast(last_hidden_state=self._prefill(input_ids, cache), past_key_values=cache)
        cache = past_key_values
        if self._use_summary():   # injected summary ids carry no information of their own
            input_ids = input_ids[:, : input_ids.shape[1] - int((input_ids[0] >= cfg.summary_token_begin).sum())]
        hs = [self._decode_token(input_ids[:, i], cache) for i in range(input_ids.shape[1])]
        return BaseModelOutputWithPast(last_hidden_state=torch.stack(hs, 1), past_key_values=cache)


def _framework():
    """The ``ksa_b200`` package if it can be imported, else None (pure PyTorch path)."""
    try:
        import ksa_b200  # noqa: F401
        from ksa_b200.config.model_config import Qwen3SummaryAttentionConfig
        from ksa_b200.inference import KsaInferenceEngine
        from ksa_b200.models import Qwen3SummaryModel
        return Qwen3SummaryAttentionConfig, Qwen3SummaryModel, KsaInferenceEngine
    except Exception:  # noqa: BLE001
        return None


class Qwen3ForCausalLM(Qwen3PreTrainedModel, GenerationMixin):
    _tied_weights_keys = ["lm_head.weight"]

    def __init__(self, config: Qwen3SAConfig):
        super().__init__(config)
        self.model = Qwen3Model(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self._fw_model = None
        self.post_init()

    def get_output_embeddings(self):
        return self.lm_head

    def get_input_embeddings(self):
        return self.model.embed_tokens

    @classmethod
    def _supports_default_dynamic_cache(cls) -> bool:
        """``generate`` must not build a ``DynamicCache``: the first forward call creates the ring-buffer cache."""
        return False

    # ---- bridge to the framework model ---------------------------------------------------------
    def framework_config(self):
        fw = _framework()
        if fw is None:
            return None
        c = self.config
        return fw[0](
            vocab_size=c.text_vocab_size, embed_dim=c.hidden_size, num_layers=c.num_hidden_layers,
            num_heads=c.num_attention_heads, num_kv_heads=c.num_key_value_heads, head_dim=c.head_dim,
            intermediate_dim=c.intermediate_size, max_seq_len=c.max_position_embeddings, rope_base=c.rope_theta,
            norm_eps=c.rms_norm_eps, tie_word_embeddings=False, rope_impl="hf",
            use_summary_attention=c.use_summary_attention, summary_chunk_size=c.summary_chunk_size,
            summary_token_num=c.summary_token_num, summary_token_begin=c.summary_token_begin,
            summary_sliding_chunk_num=c.layer_window(), summary_layer_freq=[int(b) for b in c.layer_is_summary()],
            summary_chunk_position_ids_type=c.summary_chunk_position_ids_type,
            summary_token_position_ids_type=c.summary_token_position_ids_type,
            summary_independent_parameters=c.summary_independent_parameters,
            summary_independent_attention_layernorm=c.summary_independent_attention_layernorm,
            summary_independent_qk_norm=c.summary_independent_qk_norm)

    def framework_model(self):
        """The weights of this module loaded into a ``ksa_b200`` model (built once, then cached)."""
        if self._fw_model is not None:
            return self._fw_model
        fw = _framework()
        if fw is None:
            return None
        cfg = self.framework_config()
        p = next(self.parameters())
        with torch.device("meta"):
            m = fw[1](cfg)
        m = m.to_empty(device=p.device).to(p.dtype)
        hf_state = {k: v for k, v in self.state_dict().items()}
        if not cfg.summary_independent_parameters:
            cfg_vocab = cfg.vocab_size
            hf_state["model.embed_tokens.weight"] = hf_state["model.embed_tokens.weight"][:cfg_vocab]
        m.load_state_dict(m.convert_hf_state_dict(hf_state), strict=True)
        m.drop_partial_summary = True
        self._fw_model = m.eval()
        return self._fw_model

    def _truncate(self, logits: torch.Tensor) -> torch.Tensor:
        """``truncate_predict_nums`` > 0 keeps the first N vocabulary entries.  Otherwise the logits get one column per
        row of ``embed_tokens`` (``config.vocab_size``, what the generation utilities expect), the columns of the
        summary token ids at -inf: a summary token is never predicted, sampled or scored."""
        n = int(getattr(self.config, "truncate_predict_nums", 0) or 0)
        if 0 < n < logits.shape[-1]:
            return logits[..., :n]
        pad = self.config.vocab_size - logits.shape[-1]
        return F.pad(logits, (0, pad), value=float("-inf")) if pad > 0 else logits

    def _engine_backed(self, input_ids: torch.Tensor) -> bool:
        """Prefill and decode go to the ``ksa_b200`` inference engine when the package is there and the model is on a GPU."""
        return input_ids.is_cuda and _framework() is not None

    # ---- generation plumbing ----------------------------------------------------------------------
    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None,
                                      next_sequence_length=None, **kwargs):
        """One new token per step once the cache holds the prompt.  The step whose text token completes a chunk also
        carries the ``S`` summary tokens: their ids (``summary_token_begin + j``) are appended to ``input_ids`` and
        their position ids to ``position_ids``, as the reference template does
        (``modeling_qwen3sa.py:1473-1538``)."""
        cfg = self.config
        cache = past_key_values if isinstance(past_key_values, KsaRingBufferCache) else None
        filled = cache is not None and cache.get_seq_length() > 0
        if filled:
            n_new = next_sequence_length if next_sequence_length is not None else input_ids.shape[1] - cache.get_seq_length()
            ids = input_ids[:, -max(int(n_new), 1):].clone(memory_format=torch.contiguous_format)
        else:
            ids = input_ids.clone(memory_format=torch.contiguous_format)
        position_ids = None
        if filled and cache.engine is None and ids.shape[1] == 1 and cache.boundary_due():
            B, dev = ids.shape[0], ids.device
            extra = torch.arange(cfg.summary_token_begin, cfg.summary_token_begin + cfg.summary_token_num, device=dev)
            ids = torch.cat([ids, extra[None, :].expand(B, -1)], 1)
            t = cache.text_len
            pos_t = t if cfg.summary_chunk_position_ids_type == "origin" else t % cache.chunk
            position_ids = torch.cat([torch.tensor([pos_t], device=dev), self.model._summary_positions(cache.n_chunks, dev)])
            position_ids = position_ids[None, :].expand(B, -1)
        out = {"input_ids": ids, "past_key_values": past_key_values, "attention_mask": attention_mask,
               "use_cache": kwargs.get("use_cache", True)}
        if position_ids is not None:
            out["position_ids"] = position_ids
        if "logits_to_keep" in kwargs:
            out["logits_to_keep"] = kwargs["logits_to_keep"]
        return out

    # ---- forward ------------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor = None, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, past_key_values: Optional[Cache] = None,
                labels: Optional[torch.Tensor] = None, use_cache: Optional[bool] = None, logits_to_keep: int = 0,
                **kwargs) -> CausalLMOutputWithPast:
        """Logits of the text tokens of ``input_ids`` (``logits_to_keep`` > 0: of the last ones only); with ``labels``
        also the shifted LM loss.  ``use_cache`` / ``past_key_values`` select prefill + cached decoding as described at
        the top of this file.  ``position_ids`` is accepted for API compatibility: positions follow from the layout."""
        use_cache = bool(use_cache) if use_cache is not None else False
        cached_call = isinstance(past_key_values, KsaRingBufferCache) and past_key_values.get_seq_length() > 0
        if attention_mask is not None and attention_mask.ndim == 2 and not bool(attention_mask.bool().all()):
            raise NotImplementedError("padded batches are not supported: pass prompts of equal length without padding")
        if (use_cache or cached_call) and self._engine_backed(input_ids):
            return self._forward_engine(input_ids, past_key_values, kwargs.get("max_cache_len"))
        fm = self.framework_model() if not (use_cache or cached_call) else None
        if fm is not None:      # scoring a whole sequence: the package's model (kernels on a GPU)
            with torch.set_grad_enabled(torch.is_grad_enabled() and not input_ids.is_cuda):
                logits = fm(input_ids)
            cache = None
        else:
            out = self.model(input_ids, past_key_values=past_key_values, use_cache=use_cache)
            h, cache = out.last_hidden_state, out.past_key_values
            if logits_to_keep and labels is None:
                h = h[:, -logits_to_keep:]
            logits = self.lm_head(h)[..., :self.config.text_vocab_size]
        logits = self._truncate(logits)
        loss = None
        if labels is not None:
            loss = F.cross_entropy(logits[:, :-1].float().reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1),
                                   ignore_index=-100)
        if logits_to_keep and logits.shape[1] > logits_to_keep:
            logits = logits[:, -logits_to_keep:]
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=cache)

    def _forward_engine(self, input_ids, past_key_values, max_cache_len) -> CausalLMOutputWithPast:
        """GPU + ``ksa_b200``: the cache object carries a ``KsaInferenceEngine`` (its own ring buffer with device-side
        counters, sm_100a kernels); the engine runs the summary tokens of a finished chunk itself."""
        cfg = self.config
        cache = past_key_values if isinstance(past_key_values, KsaRingBufferCache) else None
        if cache is None or cache.get_seq_length() == 0:
            B, L = input_ids.shape
            cache = KsaRingBufferCache(cfg)
            limit = int(max_cache_len or getattr(self.generation_config, "max_length", 0) or 0)
            limit = max(limit, L + int(getattr(self.generation_config, "max_new_tokens", 0) or 0), L + 1024) + 1
            cache.engine = _framework()[2](self.framework_model(), max_len=limit, batch=B)
            logits = cache.engine.prefill(input_ids)
            cache.set_prompt(L)
        else:
            ids = input_ids[:, : input_ids.shape[1] - int((input_ids[0] >= cfg.summary_token_begin).sum())] \
                if cache.use_summary else input_ids
            for i in range(ids.shape[1]):
                logits = cache.engine.decode_step(ids[:, i])
                cache.advance()
        return CausalLMOutputWithPast(logits=self._truncate(logits)[:, None, :], past_key_values=cache)


__all__ = ["Qwen3SAConfig", "Qwen3Model", "Qwen3ForCausalLM", "KsaRingBufferCache", "KsaCacheLayer"]
