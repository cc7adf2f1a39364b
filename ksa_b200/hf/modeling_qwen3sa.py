"""HuggingFace ``trust_remote_code`` model: Qwen3 + Kwai Summary Attention.

Counterpart of ``examples/pretrain/hf_template/modeling_qwen3sa.py`` of the reference.  The module tree carries the
parameters under the HF names written by the converter (``model.layers.{i}.self_attn.q_proj_summary.weight`` ...; the
summary embedding rows are the tail of ``embed_tokens``).  Computation:

* when the ``ksa_b200`` package is importable, the weights are handed (fused, zero-copy where possible) to its
  ``Qwen3SummaryModel`` and ``KsaInferenceEngine``: sm_100a kernels and the ring-buffer KV cache on a GPU, the
  package's PyTorch formulas on CPU;
* otherwise ``forward`` uses the plain PyTorch path in this file (dense two-stream masks), enough for scoring and
  short generations without any extra dependency.

Unlike the reference template, a true summary / full-attention hybrid (``summary_layer_freq``) and batch sizes above
one are supported, and full-attention layers behave identically in prefill and decode.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from transformers import PretrainedConfig, PreTrainedModel
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


class Qwen3PreTrainedModel(PreTrainedModel):
    config_class = Qwen3SAConfig
    base_model_prefix = "model"
    _no_split_modules = ["_Layer"]
    supports_gradient_checkpointing = False

    def _init_weights(self, module):
        if isinstance(module, (nn.Linear, nn.Embedding)):
            module.weight.data.normal_(0.0, 0.02)


class Qwen3Model(Qwen3PreTrainedModel):
    """Decoder stack; plain PyTorch two-stream forward over a whole sequence (no cache)."""

    def __init__(self, config: Qwen3SAConfig):
        super().__init__(config)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        is_sum, win = config.layer_is_summary(), config.layer_window()
        self.layers = nn.ModuleList([_Layer(config, is_sum[i], win[i]) for i in range(config.num_hidden_layers)])
        self.norm = _Norm(config.hidden_size, config.rms_norm_eps)
        self.post_init()

    def get_input_embeddings(self):
        return self.embed_tokens

    def forward(self, input_ids: torch.Tensor, **_unused) -> BaseModelOutputWithPast:
        cfg = self.config
        B, L = input_ids.shape
        Hq, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        use_sum = cfg.use_summary_attention and cfg.summary_token_num > 0
        ctx = SummaryContext(L, cfg.summary_chunk_size if use_sum else max(L, 1), cfg.summary_token_num if use_sum else 0,
                             cfg.summary_chunk_position_ids_type, cfg.summary_token_position_ids_type)
        Ns = ctx.n_summary_rows if use_sum else 0
        dev = input_ids.device
        x_t = self.embed_tokens(input_ids)
        pos_t = ctx.text_position_ids(dev) if use_sum else torch.arange(L, device=dev)
        x_s = None
        if Ns > 0:
            ids = torch.arange(cfg.summary_token_begin, cfg.summary_token_begin + cfg.summary_token_num, device=dev)
            x_s = self.embed_tokens(ids).repeat(ctx.n_chunks, 1).unsqueeze(0).expand(B, -1, -1)
            pos_s = ctx.summary_position_ids(dev)
        causal = torch.tril(torch.ones(L, L, dtype=torch.bool, device=dev))
        for layer in self.layers:
            a = layer.self_attn
            if layer.is_summary and Ns > 0:
                h_t = layer.input_layernorm(x_t)
                n_s = getattr(layer, "input_layernorm_summary", layer.input_layernorm)
                h_s = n_s(x_s)
                has = hasattr(a, "q_proj_summary")
                q_t, k_t, v_t = a.q_proj(h_t), a.k_proj(h_t), a.v_proj(h_t)
                q_s = (a.q_proj_summary if has else a.q_proj)(h_s)
                k_s = (a.k_proj_summary if has else a.k_proj)(h_s)
                v_s = (a.v_proj_summary if has else a.v_proj)(h_s)
                qn_s, kn_s = getattr(a, "q_norm_summary", a.q_norm), getattr(a, "k_norm_summary", a.k_norm)
                q_t = _rope(a.q_norm(q_t.view(B, L, Hq, Dh)), pos_t, cfg.rope_theta)
                k_t = _rope(a.k_norm(k_t.view(B, L, Hkv, Dh)), pos_t, cfg.rope_theta)
                q_s = _rope(qn_s(q_s.reshape(B, Ns, Hq, Dh)), pos_s, cfg.rope_theta)
                k_s = _rope(kn_s(k_s.reshape(B, Ns, Hkv, Dh)), pos_s, cfg.rope_theta)
                v_t, v_s = v_t.view(B, L, Hkv, Dh), v_s.reshape(B, Ns, Hkv, Dh)
                tt, ts, st, ss = ctx.masks(layer.window, dev)
                k_all, v_all = torch.cat([k_t, k_s], 1), torch.cat([v_t, v_s], 1)
                o_t = _attend(q_t, k_all, v_all, torch.cat([tt, ts], 1))
                o_s = _attend(q_s, k_all, v_all, torch.cat([st, ss], 1))
                x_t = x_t + a.o_proj(o_t.reshape(B, L, Hq * Dh))
                x_s = x_s + a.o_proj(o_s.reshape(B, Ns, Hq * Dh))
                x_t = x_t + layer.mlp(layer.post_attention_layernorm(x_t))
                x_s = x_s + layer.mlp(layer.post_attention_layernorm(x_s))
            else:  # full attention on the text rows; summary rows bypass the layer
                h = layer.input_layernorm(x_t)
                q = _rope(a.q_norm(a.q_proj(h).view(B, L, Hq, Dh)), pos_t, cfg.rope_theta)
                k = _rope(a.k_norm(a.k_proj(h).view(B, L, Hkv, Dh)), pos_t, cfg.rope_theta)
                o = _attend(q, k, a.v_proj(h).view(B, L, Hkv, Dh), causal)
                x_t = x_t + a.o_proj(o.reshape(B, L, Hq * Dh))
                x_t = x_t + layer.mlp(layer.post_attention_layernorm(x_t))
        return BaseModelOutputWithPast(last_hidden_state=self.norm(x_t))


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
        self._engine = None
        self.post_init()

    def get_output_embeddings(self):
        return self.lm_head

    def get_input_embeddings(self):
        return self.model.embed_tokens

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
        n = int(getattr(self.config, "truncate_predict_nums", 0) or 0)
        return logits[..., :n] if 0 < n < logits.shape[-1] else logits

    # ---- scoring ----------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None, logits_to_keep: int = 0,
                **kwargs) -> CausalLMOutputWithPast:
        """Logits for a whole sequence (no cache); with ``labels`` also the shifted LM loss."""
        fm = self.framework_model()
        if fm is not None:
            with torch.set_grad_enabled(torch.is_grad_enabled() and not input_ids.is_cuda):
                logits = fm(input_ids)
        else:
            h = self.model(input_ids).last_hidden_state
            logits = self.lm_head(h)[..., :self.config.text_vocab_size]
        logits = self._truncate(logits)
        loss = None
        if labels is not None:
            loss = F.cross_entropy(logits[:, :-1].float().reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1),
                                   ignore_index=-100)
        if logits_to_keep:
            logits = logits[:, -logits_to_keep:]
        return CausalLMOutputWithPast(loss=loss, logits=logits)

    # ---- generation -------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor = None, max_new_tokens: int = 32, do_sample: bool = False,
                 temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0, eos_token_id=None, attention_mask=None,
                 **kwargs):
        """Greedy / top-k / nucleus decoding on the ring-buffer KV cache (batch >= 1, equal prompt lengths)."""
        if input_ids is None:
            input_ids = kwargs.pop("inputs")
        fm = self.framework_model()
        eos = eos_token_id if eos_token_id is not None else self.generation_config.eos_token_id
        eos = set(eos) if isinstance(eos, (list, tuple)) else ({eos} if eos is not None else set())
        B, L = input_ids.shape

        def pick(logits):
            logits = self._truncate(logits)
            if not do_sample or temperature <= 0:
                return logits.argmax(-1)
            logits = logits.float() / temperature
            if top_k and 0 < top_k < logits.shape[-1]:
                kth = logits.topk(top_k, dim=-1).values[..., -1:]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            probs = torch.softmax(logits, -1)
            sp, si = probs.sort(-1, descending=True)
            keep = (sp.cumsum(-1) - sp) < top_p
            sp = sp * keep
            return si.gather(-1, torch.multinomial(sp / sp.sum(-1, keepdim=True), 1)).squeeze(-1)

        out = [input_ids]
        done = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
        if fm is not None:
            fw = _framework()
            engine = fw[2](fm, max_len=L + max_new_tokens + 1, batch=B)
            logits = engine.prefill(input_ids)
            step = engine.decode_step
        else:
            seq = input_ids
            logits = self.forward(seq).logits[:, -1]

            def step(tok):
                nonlocal seq
                seq = torch.cat([seq, tok[:, None]], 1)
                return self.forward(seq).logits[:, -1]
        for i in range(max_new_tokens):
            nxt = pick(logits)
            out.append(nxt[:, None])
            if eos:
                done |= torch.isin(nxt, torch.tensor(sorted(eos), device=nxt.device))
                if bool(done.all()):
                    break
            if i + 1 < max_new_tokens:
                logits = step(nxt)
        return torch.cat(out, dim=1)


__all__ = ["Qwen3SAConfig", "Qwen3Model", "Qwen3ForCausalLM"]
