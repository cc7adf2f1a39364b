"""Qwen3 and Qwen3 + Kwai Summary Attention (KSA) in the two-stream layout.

The reference interleaves summary tokens into the text sequence and scatters /
gathers summary rows with boolean masks in every layer
(``muse/models/qwen3_sa/modeling.py:58-399``, ``muse/models/qwen3_sa/_layers.py:30-237``).
Here the hidden state is one row-major buffer ``[B*L + B*Ns, D]`` whose first
``B*L`` rows are the text tokens of all sequences and whose last ``B*Ns`` rows are
the summary tokens (``Ns = ceil(L/C) * S``):

* weights shared by text and summary rows (o_proj, MLP, norms) run once on the
  whole buffer; independent summary projections run on the summary row range
  (``ops.dual_linear``); nothing is ever masked, scattered or concatenated;
* summary-attention layers call ``ops.attention_packed`` (block structure in
  closed form); full-attention layers of a hybrid stack touch the text rows only
  and the summary rows bypass them unchanged
  (``FullAttentionLayerWithSummaryBypass``, ``muse/models/qwen3_sa/modeling.py:126-168``);
* each sub-layer returns its output un-added; the residual add is fused into the
  next RMSNorm (``ops.add_rms_norm``);
* the loss head is a fused, token-chunked linear + cross-entropy, so the
  ``[tokens, vocab]`` logits never exist at once (the reference needs a separate
  chunked-loss computer for that, ``muse/losses/chunked_distill_loss_computer.py:46-214``).

Projection weights are stored fused (``wqkv`` = q|k|v rows, ``w13`` = gate|up
rows); ``muse_state_dict`` / ``load_muse_state_dict`` translate to and from the
reference's parameter names, which the checkpoint and HF converters use.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..config.model_config import Qwen3Config, Qwen3SummaryAttentionConfig
from ..ops.layout import SummaryLayout, get_layout
from .base import Model, register_model


class RMSNormParam(nn.Module):
    """Holder of an RMSNorm scale (named ``scale`` like ``muse/layers/rms_norm.py:64``)."""

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.scale = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return ops.rms_norm(x, self.scale, self.eps)


class FusedLinear(nn.Module):
    """Bias-free linear layer whose weight may hold several projections stacked along the output dim."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features))

    def forward(self, x):
        return ops.linear(x, self.weight)


class KsaAttention(nn.Module):
    def __init__(self, cfg: Qwen3Config, layer_idx: int, is_summary_layer: bool):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.is_summary_layer = is_summary_layer
        D, Hq, Hkv, Dh = cfg.embed_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        self.wqkv = FusedLinear(D, (Hq + 2 * Hkv) * Dh)
        self.output_proj = FusedLinear(Hq * Dh, D)
        self.q_norm = RMSNormParam(Dh, cfg.norm_eps) if cfg.q_norm else None
        self.k_norm = RMSNormParam(Dh, cfg.norm_eps) if cfg.k_norm else None
        self.wqkv_summary = None
        self.q_norm_summary = self.k_norm_summary = None
        if is_summary_layer and getattr(cfg, "use_independent_qkv", False):
            self.wqkv_summary = FusedLinear(D, (Hq + 2 * Hkv) * Dh)
            if cfg.summary_independent_qk_norm and cfg.q_norm:
                self.q_norm_summary = RMSNormParam(Dh, cfg.norm_eps)
                self.k_norm_summary = RMSNormParam(Dh, cfg.norm_eps)
        # summary_mix_qkv anneal: the host value (for logging) and, once the trainer has set it, a device scalar
        # that every layer shares, so that a step replayed from a CUDA graph reads the current value
        self.mix_coeff = 1.0
        self.mix_coeff_dev: Optional[torch.Tensor] = None

    def _norm_w(self, m):
        return None if m is None else m.scale


def _row_linear(tp, x: torch.Tensor, weight: torch.Tensor, residual_rows: Optional[int] = None) -> torch.Tensor:
    """Row-parallel projection: with a tensor-parallel group the result is this rank's partial sum.
    ``residual_rows``: rows of the residual stream that the ``_add_norm`` consuming the result gets (lets the group
    scatter the rows to their owners from the GEMM; the result may then only be handed to that ``_add_norm``)."""
    return ops.linear(x, weight) if tp is None else tp.row_parallel_linear(x, weight, residual_rows)


def _add_norm(tp, x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
              defer: bool = False):
    """Residual add + RMSNorm; with a tensor-parallel group ``delta`` is a partial sum that is all-reduced in the
    same kernel.  ``defer``: the normalised rows go to ``_col_linear`` next and the residual rows are not read before
    the next ``_add_norm`` / ``_row_linear`` (the group may then overlap its gathers with that projection)."""
    if tp is None or delta is None:
        return ops.add_rms_norm(x, delta, weight, eps)
    return tp.add_rms_norm(x, delta, weight, eps, defer_gather=defer)


def _col_linear(tp, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Column-parallel projection (no communication of its own; may carry a deferred gather of ``x``)."""
    return ops.linear(x, weight) if tp is None else tp.col_parallel_linear(x, weight)


class SwiGluMlp(nn.Module):
    """``w2(silu(w1 x) * w3 x)`` with w1|w3 fused into ``w13`` (``muse/layers/feed_forward.py:44-83``)."""

    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.w13 = FusedLinear(dim, 2 * hidden)
        self.w2 = FusedLinear(hidden, dim)

    def forward_after_norm(self, x, delta, norm_scale, eps):
        """``res = x + delta``; the block on ``rms_norm(res)``.  Returns ``(res, block output)``.  For the few rows of a
        decode step the residual add, the norm, the gate/up projection and SwiGLU are one launch."""
        res, h = ops.norm_linear(x, delta, norm_scale, eps, self.w13.weight, glu=True)
        return res, ops.linear(h, self.w2.weight)

    def forward(self, x, tp=None, residual_rows: Optional[int] = None):
        if x.dim() == 2 and x.shape[0] <= 16 and (tp is None or getattr(tp, "_pending", None) is None):
            h = ops.linear_swiglu(x, self.w13.weight)       # decode: projection and activation in one kernel
        else:
            h = ops.swiglu(_col_linear(tp, x, self.w13.weight))
        return _row_linear(tp, h, self.w2.weight, residual_rows)


class KsaDecoderLayer(nn.Module):
    """One decoder layer; ``is_summary_layer`` selects summary attention or full attention + summary bypass."""

    def __init__(self, cfg: Qwen3Config, layer_idx: int, is_summary_layer: bool, window_chunks: int,
                 tok_window: int):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.is_summary_layer = is_summary_layer
        self.window_chunks = window_chunks
        self.tok_window = tok_window
        self.sa_norm = RMSNormParam(cfg.embed_dim, cfg.norm_eps)
        self.sa_norm_summary = None
        if (is_summary_layer and getattr(cfg, "summary_independent_parameters", False)
                and getattr(cfg, "summary_independent_attention_layernorm", False)):
            self.sa_norm_summary = RMSNormParam(cfg.embed_dim, cfg.norm_eps)
        self.attn = KsaAttention(cfg, layer_idx, is_summary_layer)
        self.mlp_norm = RMSNormParam(cfg.embed_dim, cfg.norm_eps)
        self.mlp = SwiGluMlp(cfg.embed_dim, cfg.intermediate_dim)
        # selective recomputation: drop the gate/up projection and the SwiGLU output (3 x intermediate_dim of the
        # roughly 5 x embed_dim + 3 x intermediate_dim values a layer keeps per token) and recompute them in the
        # backward pass; attention, its projections and the norms are kept (training/activations.py, mode "mlp")
        self.recompute_mlp = False

    def _mlp(self, h: torch.Tensor, tp, rows: Optional[int]) -> torch.Tensor:
        if self.recompute_mlp and tp is None and torch.is_grad_enabled() and h.requires_grad:
            from torch.utils.checkpoint import checkpoint
            return checkpoint(self.mlp, h, None, None, use_reentrant=False)
        return self.mlp(h, tp, rows)

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], meta: "BatchMeta",
                collect: Optional[list] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``x`` ``[R, D]`` (residual stream), ``delta``: pending sub-layer output for the first rows of ``x``.

        Returns the new residual stream and the MLP output that the next norm will add.
        """
        cfg, a = self.cfg, self.attn
        Hq, Hkv, Dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        n_text = meta.B * meta.L
        tp = meta.tp
        summary_path = self.is_summary_layer and meta.Ns > 0
        # rows of the residual stream, for row-parallel outputs that go straight into the next _add_norm; the last
        # layer's MLP output is sliced by the caller first, and collected attention outputs are read as they are
        rows_attn = x.shape[0] if collect is None else None
        rows_mlp = x.shape[0] if self.layer_idx != cfg.num_layers - 1 else None
        # the normalised rows go straight into the column-parallel projection unless the summary rows have a norm of
        # their own
        plain = not summary_path or self.sa_norm_summary is None
        x, h = _add_norm(tp, x, delta, self.sa_norm.scale, cfg.norm_eps, defer=plain)
        if summary_path:
            if self.sa_norm_summary is not None:
                h = torch.cat([h[:n_text], ops.rms_norm(x[n_text:], self.sa_norm_summary.scale, cfg.norm_eps)])
            if a.wqkv_summary is not None:
                if tp is not None and tp.fused_gather and not torch.is_grad_enabled():
                    # text rows: projection that carries the gather of h; summary rows: their own weights, afterwards
                    qkv = torch.empty((h.shape[0], a.wqkv.weight.shape[0]), dtype=h.dtype, device=h.device)
                    tp.col_parallel_linear(h[:n_text], a.wqkv.weight, out=qkv[:n_text])
                    ops.gemm(h[n_text:], a.wqkv_summary.weight, out=qkv[n_text:])
                else:
                    qkv = ops.dual_linear(h, a.wqkv.weight, a.wqkv_summary.weight, n_text)
            else:
                qkv = _col_linear(tp, h, a.wqkv.weight)
            if a.wqkv_summary is not None and getattr(cfg, "summary_mix_qkv", False):
                # Anneal of the summary rows from their own projections towards the base ones, blended AFTER the QK
                # norm, each side with its own norm weights (muse/models/qwen3_sa/_layers.py:153-171).  RoPE is
                # linear, so blending the rotated rows equals rotating the blend.
                nq, nk = a._norm_w(a.q_norm), a._norm_w(a.k_norm)
                sq = a.q_norm_summary.scale if a.q_norm_summary is not None else nq
                sk = a.k_norm_summary.scale if a.k_norm_summary is not None else nk
                rot = lambda rows, wq, wk, pos: ops.qk_norm_rope_packed(  # noqa: E731
                    rows.contiguous(), wq, wk, pos, Hq, Hkv, Dh, cfg.rope_base, cfg.norm_eps, meta.rope_interleaved)
                own = rot(qkv[n_text:], sq, sk, meta.pos[n_text:])
                base = rot(ops.linear(h[n_text:], a.wqkv.weight), nq, nk, meta.pos[n_text:])
                mix = a.mix_coeff_dev if a.mix_coeff_dev is not None else a.mix_coeff
                mixed = torch.lerp(base.float(), own.float(), mix.to(base.device) if torch.is_tensor(mix) else mix)
                qkv = torch.cat([rot(qkv[:n_text], nq, nk, meta.pos[:n_text]), mixed.to(qkv.dtype)])
            elif a.q_norm_summary is not None:
                qkv = torch.cat([
                    ops.qk_norm_rope_packed(qkv[:n_text].contiguous(), a._norm_w(a.q_norm), a._norm_w(a.k_norm),
                                            meta.pos[:n_text], Hq, Hkv, Dh, cfg.rope_base, cfg.norm_eps,
                                            meta.rope_interleaved),
                    ops.qk_norm_rope_packed(qkv[n_text:].contiguous(), a.q_norm_summary.scale,
                                            a.k_norm_summary.scale, meta.pos[n_text:], Hq, Hkv, Dh, cfg.rope_base,
                                            cfg.norm_eps, meta.rope_interleaved)])
            else:
                qkv = ops.qk_norm_rope_packed(qkv, a._norm_w(a.q_norm), a._norm_w(a.k_norm), meta.pos, Hq, Hkv, Dh,
                                              cfg.rope_base, cfg.norm_eps, meta.rope_interleaved)
            if meta.kv_sink is not None:
                meta.kv_sink(self.layer_idx, qkv, True)
            if meta.cp is not None:
                from ..parallel.cp import cp_attention_packed
                att = cp_attention_packed(qkv, meta.cp, Hq, Hkv, Dh, self.window_chunks, True)
            else:
                att = ops.attention_packed(qkv, meta.B, meta.L, meta.Ns, Hq, Hkv, Dh, meta.chunk, meta.n_sum,
                                           self.window_chunks, mode=getattr(cfg, "summary_attention_mode", "kernel"))
            attn_out = _row_linear(tp, att, a.output_proj.weight, rows_attn)
            if collect is not None:
                collect.append(attn_out[:n_text])
            x, h2 = _add_norm(tp, x, attn_out, self.mlp_norm.scale, cfg.norm_eps, defer=True)
            return x, self._mlp(h2, tp, rows_mlp)
        # full causal attention on the text rows; summary rows (if any) pass through unchanged
        qkv = _col_linear(tp, h[:n_text], a.wqkv.weight)
        qkv = ops.qk_norm_rope_packed(qkv, a._norm_w(a.q_norm), a._norm_w(a.k_norm), meta.pos[:n_text], Hq, Hkv, Dh,
                                      cfg.rope_base, cfg.norm_eps, meta.rope_interleaved)
        if meta.kv_sink is not None:
            # a summary layer lands here when the prompt has no complete chunk yet: its cache keeps its own layout
            meta.kv_sink(self.layer_idx, qkv, self.is_summary_layer)
        if meta.cp is not None:
            from ..parallel.cp import cp_attention_packed
            att = cp_attention_packed(qkv, meta.cp, Hq, Hkv, Dh, None, False, self.tok_window)
        else:
            att = ops.attention_packed(qkv, meta.B, meta.L, 0, Hq, Hkv, Dh, tok_window=self.tok_window,
                                       cu_seqlens=getattr(meta, "cu_seqlens", None))
        attn_out = _row_linear(tp, att, a.output_proj.weight, rows_attn)
        if collect is not None:
            collect.append(attn_out)
        x, h2 = _add_norm(tp, x, attn_out, self.mlp_norm.scale, cfg.norm_eps, defer=True)
        return x, self._mlp(h2[:n_text], tp, rows_mlp)


class BatchMeta:
    """Per-shape constants of a batch: sizes and the per-row position ids (text rows, then summary rows)."""

    def __init__(self, B: int, L: int, layout: Optional[SummaryLayout], device, rope_interleaved: bool,
                 position_ids: Optional[torch.Tensor] = None, cp=None):
        self.B, self.L = B, L
        self.rope_interleaved = rope_interleaved
        self.cp = cp          # context-parallel group state: this rank holds one contiguous shard of the sequence
        self.tp = None        # tensor-parallel group state (inference): row-parallel outputs are partial sums
        self.kv_sink = None   # optional callable(layer_idx, qkv_rot, is_summary_layer): prefill fills KV caches with it
        self.cu_seqlens = None  # packed-document offsets for the full-attention layers
        if cp is not None:
            # ``layout`` describes the whole sequence; keep this shard's rows of its position ids
            r, Ll = cp.rank, cp.shape.local_len
            self.L = Ll
            text = layout.text_position_ids(device) if layout is not None else torch.arange(cp.shape.seq_len, device=device)
            parts = [text[r * Ll:(r + 1) * Ll].repeat(B)]
            if layout is not None:
                self.chunk, self.n_sum = layout.chunk, layout.n_sum
                self.Ns = cp.shape.local_sum
                parts.append(layout.summary_position_ids(device)[r * self.Ns:(r + 1) * self.Ns].repeat(B))
            else:
                self.Ns, self.chunk, self.n_sum = 0, 128, 1
            self.pos = torch.cat(parts).to(torch.int32)
            return
        if layout is not None:
            self.Ns, self.chunk, self.n_sum = layout.n_summary_rows, layout.chunk, layout.n_sum
            pos_t = layout.text_position_ids(device) if position_ids is None else None
            pos_s = layout.summary_position_ids(device)
        else:
            self.Ns, self.chunk, self.n_sum = 0, 128, 1
            pos_t = torch.arange(L, device=device) if position_ids is None else None
            pos_s = None
        if position_ids is not None:
            text = position_ids.reshape(B * L).to(device)
        else:
            text = pos_t.repeat(B)
        parts = [text]
        if pos_s is not None and self.Ns > 0:
            parts.append(pos_s.repeat(B))
        self.pos = torch.cat(parts).to(torch.int32)


@register_model("Qwen3Model")
class Qwen3Model(Model):
    """Dense Qwen3 decoder (``muse/models/qwen3/modeling.py:59-117``): the KSA stack with no summary rows."""

    config_class = Qwen3Config

    def __init__(self, config: Qwen3Config):
        super().__init__(config)
        cfg = config
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.embed_dim)
        is_sum = self._layer_is_summary()
        self.layers = nn.ModuleList([
            KsaDecoderLayer(cfg, i, is_sum[i], self._layer_window(i), max(cfg.get_layer_sliding_window(i), 0))
            for i in range(cfg.num_layers)])
        self.norm = RMSNormParam(cfg.embed_dim, cfg.norm_eps)
        self.output = None if cfg.tie_word_embeddings else FusedLinear(cfg.embed_dim, cfg.vocab_size)
        self.summary_embedding = None
        self._meta_cache: Dict[tuple, BatchMeta] = {}
        self.skip_output_layer = False
        self.loss_chunk_tokens = 2048
        self.drop_partial_summary = False   # inference: a trailing partial chunk gets no summary tokens
        self.cp = None                      # parallel.cp.CpContext: ``forward`` then takes this rank's sequence shard
        self.tp = None                      # parallel.tp.TpContext: this module holds one tensor-parallel shard

    # ---- configuration helpers ----------------------------------------------------
    def _layer_is_summary(self) -> List[bool]:
        return [False] * self.config.num_layers

    def _layer_window(self, i: int) -> int:
        return 0

    def _layout(self, L: int) -> Optional[SummaryLayout]:
        return None

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.tok_embeddings.weight if self.output is None else self.output.weight

    def get_initializer(self):
        """N(0, 0.02) for matrices, ones for norm scales (the benchmark initialisation)."""
        return super().get_initializer()

    def reference_init(self, seed: Optional[int] = None) -> None:
        """The reference's scheme: xavier-uniform attention/MLP linears, LeCun-normal lm_head, N(0, 0.02)
        embeddings, ones for norms (``muse/models/qwen3_sa/modeling.py:401-470``)."""
        if seed is not None:
            torch.manual_seed(seed)
        cfg = self.config
        Hq, Hkv, Dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        with torch.no_grad():
            nn.init.normal_(self.tok_embeddings.weight, 0.0, 0.02)
            if self.summary_embedding is not None:
                nn.init.normal_(self.summary_embedding.weight, 0.0, 0.02)
            if self.output is not None:
                nn.init.normal_(self.output.weight, 0.0, 1.0 / math.sqrt(cfg.embed_dim))
            for layer in self.layers:
                for lin in (layer.attn.wqkv, layer.attn.wqkv_summary):
                    if lin is None:
                        continue
                    for lo, hi in ((0, Hq * Dh), (Hq * Dh, (Hq + Hkv) * Dh), ((Hq + Hkv) * Dh, (Hq + 2 * Hkv) * Dh)):
                        nn.init.xavier_uniform_(lin.weight[lo:hi])
                nn.init.xavier_uniform_(layer.attn.output_proj.weight)
                F = cfg.intermediate_dim
                nn.init.xavier_uniform_(layer.mlp.w13.weight[:F])
                nn.init.xavier_uniform_(layer.mlp.w13.weight[F:])
                nn.init.xavier_uniform_(layer.mlp.w2.weight)
            for m in self.modules():
                if isinstance(m, RMSNormParam):
                    nn.init.ones_(m.scale)

    # ---- forward ----------------------------------------------------------------
    def _meta(self, B: int, L: int, device, position_ids, use_summary: bool = True) -> BatchMeta:
        if self.cp is not None:
            if position_ids is not None:
                raise NotImplementedError("explicit position ids are not combined with context parallelism")
            if L != self.cp.shape.local_len or B != self.cp.batch:
                raise ValueError(f"context-parallel shard is [{self.cp.batch}, {self.cp.shape.local_len}], got [{B}, {L}]")
            key = ("cp", id(self.cp), B, L, str(device), use_summary)
            if key not in self._meta_cache:
                layout = self._layout(self.cp.shape.seq_len) if use_summary else None
                self._meta_cache[key] = BatchMeta(B, L, layout, device, self.config.rope_impl == "llama", cp=self.cp)
            return self._meta_cache[key]
        layout = self._layout(L) if use_summary else None
        if position_ids is not None:
            return BatchMeta(B, L, layout, device, self.config.rope_impl == "llama", position_ids)
        key = (B, L, str(device), self.drop_partial_summary, use_summary)
        if key not in self._meta_cache:
            self._meta_cache[key] = BatchMeta(B, L, layout, device, self.config.rope_impl == "llama")
        return self._meta_cache[key]

    def embed(self, tokens: torch.Tensor, meta: BatchMeta) -> torch.Tensor:
        x = ops.embedding(tokens.reshape(-1), self.tok_embeddings.weight)
        if meta.Ns > 0:
            x = torch.cat([x, self._summary_rows(meta, x.dtype)], dim=0)
        return x

    def _summary_rows(self, meta: BatchMeta, dtype) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, tokens: torch.Tensor, labels: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, return_hidden: bool = False,
                collect_attn: bool = False, ignore_index: int = -100, kv_sink=None, last_token_only: bool = False,
                use_summary: bool = True, cu_seqlens: Optional[torch.Tensor] = None):
        """``tokens`` ``[B, L]`` -> loss (with ``labels``), hidden ``[B, L, D]`` or logits ``[B, L, V]``.

        ``cu_seqlens`` (token offsets of documents packed into the sequence, the same for every sequence of the batch):
        full-attention layers keep every query inside its own document (the reference's varlen FlashAttention-2 path,
        ``muse/models/qwen3/_layers.py:331-334``); summary-attention layers ignore document boundaries, as the
        reference's summary insertion does (``muse/layers/summary_utils.py:26-27``).

        ``labels`` are already shifted (label of position t is token t+1) with ``ignore_index`` where masked,
        as the reference trainer builds them (``recipes/pretrain_kai_summary_unified.py:867-873``).
        """
        B, L = tokens.shape
        # use_summary=False runs every layer as plain causal attention on the base projections (the distillation
        # teacher: same weights, no summary tokens, recipes/pretrain_kai_summary_unified.py:967-997)
        meta = self._meta(B, L, tokens.device, position_ids, use_summary)
        meta.kv_sink = kv_sink
        meta.cu_seqlens = cu_seqlens if cu_seqlens is not None and cu_seqlens.numel() > 2 else None
        tp = meta.tp = self.tp
        x = self.embed(tokens, meta)
        collect = [] if collect_attn else None
        delta = None
        for layer in self.layers:
            x, delta = layer(x, delta, meta, collect)
        if tp is not None:
            tp.flush()      # the residual rows are read directly below
        meta.kv_sink = None
        n_text = B * L
        if last_token_only:   # prefill: only the last position of every sequence feeds the head
            rows = torch.arange(B, device=x.device) * L + (L - 1)
            xl = x[rows]
            dl = delta[rows] if delta is not None else None
            _, h = _add_norm(tp, xl, dl, self.norm.scale, self.config.norm_eps)
            logits = ops.linear(h, self.lm_head_weight)
            if tp is not None and logits.shape[-1] != self.config.vocab_size:
                logits = tp.gather_logits(logits)
            return logits.view(B, 1, -1)
        # summary rows are dropped before the final norm and the head (modeling.py:243-249)
        _, h = _add_norm(tp, x[:n_text], delta[:n_text] if delta is not None else None, self.norm.scale,
                         self.config.norm_eps)
        self.last_attn_outputs = collect
        if labels is not None and not self.skip_output_layer:
            return ops.linear_cross_entropy(h, self.lm_head_weight, labels.reshape(-1), ignore_index,
                                            self.loss_chunk_tokens)
        if return_hidden or self.skip_output_layer:
            return h.view(B, L, -1)
        logits = ops.linear(h, self.lm_head_weight)
        if tp is not None and logits.shape[-1] != self.config.vocab_size:
            logits = tp.gather_logits(logits)
        return logits.view(B, L, -1)

    # ---- Muse / HF parameter names ---------------------------------------------------
    def muse_state_dict(self, state: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
        """State dict under the reference's parameter names (fused projections split)."""
        cfg = self.config
        Hq, Hkv, Dh, F = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.intermediate_dim
        src = state if state is not None else self.state_dict()
        out: Dict[str, torch.Tensor] = {}
        for k, v in src.items():
            if k == "tok_embeddings.weight":
                out["model.tok_embeddings.weight"] = v
            elif k == "norm.scale":
                out["model.norm.scale"] = v
            elif k == "output.weight":
                out["model.output.weight"] = v
            elif k == "summary_embedding.weight":
                out["summary_embedding.weight"] = v
            elif k.startswith("layers."):
                _, i, rest = k.split(".", 2)
                p = f"model.layers.{i}."
                if rest in ("attn.wqkv.weight", "attn.wqkv_summary.weight"):
                    suf = "_summary" if "summary" in rest else ""
                    out[p + f"attn.q_proj{suf}.weight"] = v[:Hq * Dh]
                    out[p + f"attn.k_proj{suf}.weight"] = v[Hq * Dh:(Hq + Hkv) * Dh]
                    out[p + f"attn.v_proj{suf}.weight"] = v[(Hq + Hkv) * Dh:]
                elif rest == "mlp.w13.weight":
                    out[p + "mlp.w1.weight"] = v[:F]
                    out[p + "mlp.w3.weight"] = v[F:]
                else:
                    out[p + rest] = v
            else:
                out[k] = v
        return out

    def from_muse_state_dict(self, muse: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Inverse of :meth:`muse_state_dict` (fuses q|k|v and w1|w3)."""
        out: Dict[str, torch.Tensor] = {}
        groups: Dict[str, Dict[str, torch.Tensor]] = {}
        for k, v in muse.items():
            k2 = k[len("model."):] if k.startswith("model.") else k
            if k2.startswith("layers."):
                _, i, rest = k2.split(".", 2)
                for names, fused in ((("attn.q_proj.weight", "attn.k_proj.weight", "attn.v_proj.weight"),
                                      "attn.wqkv.weight"),
                                     (("attn.q_proj_summary.weight", "attn.k_proj_summary.weight",
                                       "attn.v_proj_summary.weight"), "attn.wqkv_summary.weight"),
                                     (("mlp.w1.weight", "mlp.w3.weight"), "mlp.w13.weight")):
                    if rest in names:
                        groups.setdefault(f"layers.{i}.{fused}", {})[rest] = v
                        break
                else:
                    out[k2] = v
            else:
                out[k2] = v
        order = ["attn.q_proj.weight", "attn.k_proj.weight", "attn.v_proj.weight",
                 "attn.q_proj_summary.weight", "attn.k_proj_summary.weight", "attn.v_proj_summary.weight",
                 "mlp.w1.weight", "mlp.w3.weight"]
        for fused, parts in groups.items():
            out[fused] = torch.cat([parts[n] for n in order if n in parts], dim=0)
        return out

    def load_muse_state_dict(self, muse: Dict[str, torch.Tensor], strict: bool = True):
        return self.load_state_dict(self.from_muse_state_dict(muse), strict=strict)

    _MUSE_TO_HF = [
        ("sa_norm_summary.scale", "input_layernorm_summary.weight"), ("sa_norm.scale", "input_layernorm.weight"),
        ("mlp_norm.scale", "post_attention_layernorm.weight"), ("attn.output_proj", "self_attn.o_proj"),
        ("attn.q_norm_summary.scale", "self_attn.q_norm_summary.weight"),
        ("attn.k_norm_summary.scale", "self_attn.k_norm_summary.weight"),
        ("attn.q_norm.scale", "self_attn.q_norm.weight"), ("attn.k_norm.scale", "self_attn.k_norm.weight"),
        ("attn.", "self_attn."), ("mlp.w1.", "mlp.gate_proj."), ("mlp.w3.", "mlp.up_proj."),
        ("mlp.w2.", "mlp.down_proj."),
    ]

    @classmethod
    def muse_to_hf_keys(cls, muse: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Reference key names -> HF names; the summary embedding is appended to ``embed_tokens`` and ``lm_head``
        is zero-padded to the same vocabulary (``examples/pretrain/convert/checkpoint.py:20-109``)."""
        out: Dict[str, torch.Tensor] = {}
        summary = None
        top = {"model.tok_embeddings.weight": "model.embed_tokens.weight", "model.norm.scale": "model.norm.weight",
               "model.output.weight": "lm_head.weight"}
        for k, v in muse.items():
            if k in top:
                out[top[k]] = v
            elif k == "summary_embedding.weight":
                summary = v
            elif k.startswith("model.layers."):
                _, _, i, rest = k.split(".", 3)
                for a, b in cls._MUSE_TO_HF:
                    if rest.startswith(a) or (a.endswith(".scale") and rest == a):
                        rest = b + rest[len(a):]
                        break
                out[f"model.layers.{i}.{rest}"] = v
            else:
                out[k] = v
        if summary is not None and "model.embed_tokens.weight" in out:
            emb = out["model.embed_tokens.weight"]
            out["model.embed_tokens.weight"] = torch.cat([emb, summary.to(emb.dtype)], dim=0)
            if "lm_head.weight" in out and out["lm_head.weight"].shape[0] < emb.shape[0] + summary.shape[0]:
                lm = out["lm_head.weight"]
                pad = lm.new_zeros(emb.shape[0] + summary.shape[0] - lm.shape[0], lm.shape[1])
                out["lm_head.weight"] = torch.cat([lm, pad], dim=0)
        return out

    @classmethod
    def hf_to_muse_keys(cls, hf: Dict[str, torch.Tensor], vocab_size: int, n_summary: int) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        top = {"model.embed_tokens.weight": "model.tok_embeddings.weight", "model.norm.weight": "model.norm.scale",
               "lm_head.weight": "model.output.weight"}
        for k, v in hf.items():
            if k in top:
                if k == "model.embed_tokens.weight" and v.shape[0] >= vocab_size + n_summary > vocab_size:
                    out["summary_embedding.weight"] = v[vocab_size:vocab_size + n_summary]
                    v = v[:vocab_size]
                if k == "lm_head.weight":
                    v = v[:vocab_size]
                out[top[k]] = v
            elif k.startswith("model.layers."):
                _, _, i, rest = k.split(".", 3)
                for a, b in cls._MUSE_TO_HF:
                    if rest.startswith(b) or rest == b:
                        rest = a + rest[len(b):]
                        break
                out[f"model.layers.{i}.{rest}"] = v
            else:
                out[k] = v
        return out

    def convert_hf_state_dict(self, hf_state):
        cfg = self.config
        n_sum = getattr(cfg, "summary_token_num", 0) if getattr(cfg, "summary_independent_parameters", False) else 0
        return self.from_muse_state_dict(self.hf_to_muse_keys(hf_state, cfg.vocab_size, n_sum))

    def revert_hf_state_dict(self, state):
        return self.muse_to_hf_keys(self.muse_state_dict(state))

    # ---- generation (greedy / sampling) on the training graph, for sanity checks ------------
    @torch.no_grad()
    def generate(self, tokens: torch.Tensor, max_new_tokens: int, temperature: float = 0.0,
                 top_p: float = 1.0, eos_id: Optional[int] = None) -> torch.Tensor:
        """Recompute-everything generation (no cache); the serving path is ``ksa_b200.inference``."""
        out = tokens
        for _ in range(max_new_tokens):
            logits = self.forward(out)[:, -1].float()
            if temperature <= 0:
                nxt = logits.argmax(-1, keepdim=True)
            else:
                probs = torch.softmax(logits / temperature, -1)
                sp, si = probs.sort(-1, descending=True)
                keep = sp.cumsum(-1) - sp < top_p
                sp = sp * keep
                nxt = si.gather(-1, torch.multinomial(sp / sp.sum(-1, keepdim=True), 1))
            out = torch.cat([out, nxt], dim=1)
            if eos_id is not None and bool((nxt == eos_id).all()):
                break
        return out


@register_model("Qwen3SummaryModel")
class Qwen3SummaryModel(Qwen3Model):
    """Qwen3 with Kwai Summary Attention; per layer summary attention or full attention (hybrid stacks)."""

    config_class = Qwen3SummaryAttentionConfig

    def __init__(self, config: Qwen3SummaryAttentionConfig):
        super().__init__(config)
        cfg = config
        if cfg.summary_enabled and cfg.summary_independent_parameters:
            self.summary_embedding = nn.Embedding(cfg.summary_token_num, cfg.embed_dim)

    def _layer_is_summary(self) -> List[bool]:
        cfg = self.config
        return cfg.get_layer_is_summary() if cfg.summary_enabled else [False] * cfg.num_layers

    def _layer_window(self, i: int) -> int:
        cfg = self.config
        return cfg.get_layer_sliding_chunk_num(i) if cfg.summary_enabled else 0

    def _layout(self, L: int) -> Optional[SummaryLayout]:
        cfg = self.config
        if not cfg.summary_enabled:
            return None
        return get_layout(L, cfg.summary_chunk_size, cfg.summary_token_num, cfg.summary_chunk_position_ids_type,
                          cfg.summary_token_position_ids_type, self.drop_partial_summary)

    def _summary_rows(self, meta: BatchMeta, dtype) -> torch.Tensor:
        cfg = self.config
        n_chunks = meta.Ns // meta.n_sum
        if self.summary_embedding is not None:
            rows = self.summary_embedding.weight
        else:  # summary tokens are ordinary vocabulary entries starting at summary_token_begin
            ids = torch.arange(cfg.summary_token_begin, cfg.summary_token_begin + meta.n_sum,
                               device=self.tok_embeddings.weight.device)
            rows = ops.embedding(ids, self.tok_embeddings.weight)
        return rows.to(dtype).repeat(meta.B * n_chunks, 1)

    def set_mix_coeff(self, iteration: int) -> float:
        """Linear anneal of the summary projections towards the base ones (``_layers.py:83-93``)."""
        cfg = self.config
        if not cfg.summary_mix_qkv:
            coeff = 1.0
        elif iteration <= cfg.summary_mix_start_iter:
            coeff = 1.0
        elif iteration >= cfg.summary_mix_end_iter:
            coeff = 0.0
        else:
            coeff = 1.0 - (iteration - cfg.summary_mix_start_iter) / max(
                1, cfg.summary_mix_end_iter - cfg.summary_mix_start_iter)
        dev = self.tok_embeddings.weight.device
        if cfg.summary_mix_qkv:
            if getattr(self, "_mix_coeff_dev", None) is None or self._mix_coeff_dev.device != dev:
                self._mix_coeff_dev = torch.ones((), dtype=torch.float32, device=dev)
            self._mix_coeff_dev.fill_(coeff)
        for layer in self.layers:
            layer.attn.mix_coeff = coeff
            layer.attn.mix_coeff_dev = self._mix_coeff_dev if cfg.summary_mix_qkv else None
        return coeff
