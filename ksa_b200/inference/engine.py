"""Prefill + decode engine for Qwen3-KSA with the ring-buffer KV cache (batch >= 1).

Prefill runs the training graph once over the prompt (block-sparse KSA attention for summary layers, causal
attention for full layers), with a trailing partial chunk receiving no summary tokens, and files every layer's
rotated K/V into the caches.  A decode step feeds one text token per sequence; when that token completes a chunk the
step also carries the chunk's ``S`` summary tokens (summary embedding, summary projections, position ids of the
``last_chunk_slice_right`` rule) and afterwards flushes the chunk into the ring and appends the summary K/V
(``examples/pretrain/hf_template/modeling_qwen3sa.py:1040-1325,1473-1560``).  The reference's decode path supports
batch 1 only (``:753-754``); here all sequences of a batch advance together and may sit at different chunk phases.

Chunk phases are mirrored on the host (they are a deterministic function of prompt length and steps taken), so a step
never reads device memory back; slice bounds and slots are computed on the device from the counters.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from .. import ops
from ..models.qwen3_ksa import _add_norm, _row_linear
from ..ops import _lib, reference as ref
from .cache import (CacheSpec, CacheState, FullLayerCache, KsaLayerCache, flush_plan, summary_step_slices,
                    text_step_slices)


def _decode_attention(q, k_cache, v_cache, start, length, scale, counters=None):
    """q ``[B, Tq, Hq, D]``; every (b, t) attends cache slots ``[start, start+length)``."""
    if not q.is_cuda:
        outs = [ref.decode_attention(q[:, t:t + 1], k_cache, v_cache, length[:, t].long(), start[:, t].long(), scale)
                for t in range(q.shape[1])]
        return torch.cat(outs, dim=1)
    B, Tq, Hq, D = q.shape
    Hkv, cap = k_cache.shape[1], k_cache.shape[2]
    # short slices (the ring + summaries of a summary layer) are latency-bound: cut them into many small splits so
    # that every SM holds several CTAs; long caches get at most 64 splits
    keys_per_split = 128
    splits = max(1, min(64, (cap + keys_per_split - 1) // keys_per_split))
    keys_per_split = ((cap + splits - 1) // splits + 63) // 64 * 64
    part_o = torch.empty((B, Tq, Hq, splits, D), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((B, Tq, Hq, splits, 2), dtype=torch.float32, device=q.device)
    out = torch.empty_like(q)
    # the split that finishes last merges the splits itself and puts its counter back to zero, so launches that
    # follow one another on a stream can share ``counters`` (``[B * Hkv]`` int32 zeros; a fresh array when not given)
    if counters is None:
        counters = torch.zeros(B * Hkv, dtype=torch.int32, device=q.device)
    _lib.call("ksa_decode_attn", q.contiguous(), k_cache, v_cache, start.contiguous(), length.contiguous(), part_o,
              part_ml, out, B, Tq, Hq, Hkv, D, cap, splits, keys_per_split, float(scale), counters)
    return out


def _cache_append(k_new, v_new, k_cache, v_cache, slots):
    """``k_new``/``v_new`` ``[B, T, H, D]`` (views allowed) -> cache ``[B, H, cap, D]`` at ``slots[B, T]`` (< 0: skip)."""
    if not k_new.is_cuda:
        B, T, H, D = k_new.shape
        for b in range(B):
            for t in range(T):
                s = int(slots[b, t])
                if s >= 0:
                    k_cache[b, :, s] = k_new[b, t]
                    v_cache[b, :, s] = v_new[b, t]
        return
    B, T, H, D = k_new.shape
    assert k_new.stride(3) == 1 and k_new.stride(2) == D and v_new.stride() == k_new.stride()
    _lib.call("ksa_kv_cache_append", k_new, v_new, k_cache, v_cache, slots.contiguous(), B, T, H, D, k_cache.shape[2],
              k_new.stride(1), k_new.stride(0))


def _cache_move(k_cache, v_cache, src, dst, enable, rows):
    if rows == 0:
        return
    if not k_cache.is_cuda:
        for b in range(k_cache.shape[0]):
            if int(enable[b]):
                s, d = int(src[b]), int(dst[b])
                k_cache[b, :, d:d + rows] = k_cache[b, :, s:s + rows].clone()
                v_cache[b, :, d:d + rows] = v_cache[b, :, s:s + rows].clone()
        return
    B, H, cap, D = k_cache.shape
    _lib.call("ksa_kv_cache_move", k_cache, v_cache, src.contiguous(), dst.contiguous(), enable.contiguous(), B, H, D,
              cap, rows)


class KsaInferenceEngine:
    def __init__(self, model, max_len: int, batch: int, device=None, dtype=None, cuda_graph: bool = True):
        self.model = model.eval()
        # steps that do not cross a chunk boundary replay one captured CUDA graph (all indices come from device
        # counters, so the launch sequence is the same every step); boundary steps (1 in ``chunk``) run eagerly
        self.cuda_graph = cuda_graph
        self._graphs = {}            # any sequence at a chunk boundary? -> (graph, logits)
        self._graph_tokens = None
        self._boundary_dev = None    # [B] int32: which sequences close a chunk in this step (read inside the graphs)
        self._plain_steps = {False: 0, True: 0}
        self.model.drop_partial_summary = True
        cfg = model.config
        self.cfg = cfg
        p = next(model.parameters())
        self.device = device or p.device
        self.dtype = dtype or p.dtype
        self.batch = batch
        self.max_len = max_len
        self.C = cfg.summary_chunk_size if cfg.summary_enabled else max_len
        self.S = cfg.summary_token_num if cfg.summary_enabled else 0
        Hkv, Dh = cfg.num_kv_heads, cfg.head_dim
        self.layer_caches: List[object] = []
        self.specs: List[Optional[CacheSpec]] = []
        for layer in model.layers:
            if layer.is_summary_layer:
                spec = CacheSpec(self.C, self.S, layer.window_chunks, max_len // self.C + 1)
                self.specs.append(spec)
                self.layer_caches.append(KsaLayerCache(spec, batch, Hkv, Dh, self.dtype, self.device))
            else:
                self.specs.append(None)
                self.layer_caches.append(FullLayerCache(max_len, batch, Hkv, Dh, self.dtype, self.device))
        self.state = CacheState(batch, self.device)
        self.host_len = [0] * batch
        self._boundary_dev = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self._merge_counters = torch.zeros(batch * Hkv, dtype=torch.int32, device=self.device)

    def reserve(self, max_len: int) -> None:
        """Grow every layer's cache so that sequences may reach ``max_len`` tokens; contents are kept.  The cache layout
        puts the region that grows (text of full-attention layers, summaries of summary layers) last, so the old
        buffers are prefixes of the new ones.  Captured decode graphs hold the old addresses and are dropped."""
        if max_len <= self.max_len:
            return
        cfg = self.cfg
        Hkv, Dh = cfg.num_kv_heads, cfg.head_dim
        for li, old in enumerate(self.layer_caches):
            if self.specs[li] is not None:
                sp = self.specs[li]
                spec = CacheSpec(sp.chunk, sp.n_sum, sp.window, max_len // self.C + 1)
                new = KsaLayerCache(spec, self.batch, Hkv, Dh, self.dtype, self.device)
                self.specs[li] = spec
            else:
                new = FullLayerCache(max_len, self.batch, Hkv, Dh, self.dtype, self.device)
            cap = old.k.shape[2]
            new.k[:, :, :cap] = old.k
            new.v[:, :, :cap] = old.v
            self.layer_caches[li] = new
        self.max_len = max_len
        self._graphs = {}

    def cache_bytes(self) -> int:
        return sum(c.k.numel() * c.k.element_size() * 2 for c in self.layer_caches)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, lengths: Optional[List[int]] = None,
                batch_chunk: Optional[int] = None) -> torch.Tensor:
        """``tokens`` ``[B, L]`` -> logits of every sequence's last prompt position ``[B, V]``; caches are filled.

        ``lengths``: prompt length of every sequence when they differ (``tokens`` is then padded on the right; the
        padding is never read).  Sequences of equal length are prefilled together, at most ``batch_chunk`` at a time
        (bounds the activation memory of long prompts in large batches); afterwards the sequences decode together,
        each at its own chunk phase."""
        B, Lmax = tokens.shape
        assert B == self.batch
        lengths = [Lmax] * B if lengths is None else [int(l) for l in lengths]
        assert len(lengths) == B and all(0 < l <= Lmax for l in lengths), "bad prompt lengths"
        if max(lengths) > self.max_len:
            self.reserve(max(lengths))
        groups = {}
        for i, l in enumerate(lengths):
            groups.setdefault(l, []).append(i)
        out = None
        for L, idx in sorted(groups.items()):
            step = batch_chunk or len(idx)
            for j in range(0, len(idx), step):
                rows = idx[j:j + step]
                logits = self._prefill_rows(tokens[rows, :L] if rows != list(range(B)) or L != Lmax else tokens, rows)
                if out is None:
                    out = torch.empty(B, logits.shape[-1], dtype=torch.float32, device=logits.device)
                out[rows] = logits
        self.host_len = list(lengths)
        return out

    def _prefill_rows(self, tokens: torch.Tensor, rows: List[int]) -> torch.Tensor:
        """Prefill the sequences ``rows`` of the batch (all of length ``tokens.shape[1]``) in one pass of the model."""
        B, L = tokens.shape
        cfg, C, S = self.cfg, self.C, self.S
        Hq, Hkv, Dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        n_full = L // C if S > 0 else 0      # complete chunks
        tail = L - n_full * C if S > 0 else L
        Ns = n_full * S
        contiguous = rows == list(range(rows[0], rows[0] + B))
        sel = slice(rows[0], rows[0] + B) if contiguous else None

        def put(dst, slots, src):
            """``src`` ``[B, n, H, D]`` -> cache ``dst[rows, :, slots]`` (``slots``: slice or index tensor)."""
            if contiguous:
                dst[sel, :, slots] = src.transpose(1, 2)
            else:
                for i, r in enumerate(rows):
                    dst[r, :, slots] = src[i].transpose(0, 1)

        def sink(layer_idx, qkv, is_summary_layer):
            cache = self.layer_caches[layer_idx]
            k_t = qkv[:B * L, Hq * Dh:(Hq + Hkv) * Dh].view(B, L, Hkv, Dh)
            v_t = qkv[:B * L, (Hq + Hkv) * Dh:].view(B, L, Hkv, Dh)
            if not is_summary_layer:
                put(cache.k, slice(0, L), k_t)
                put(cache.v, slice(0, L), v_t)
                return
            spec = self.specs[layer_idx]
            W = spec.window
            # ring: the last min(W, n_full) complete chunks, chunk c at ring slot (c mod W)
            for c in range(max(0, n_full - W), n_full):
                dst = spec.text0 + (c % max(W, 1)) * C
                put(cache.k, slice(dst, dst + C), k_t[:, c * C:(c + 1) * C])
                put(cache.v, slice(dst, dst + C), v_t[:, c * C:(c + 1) * C])
            # current (partial) chunk, right to left: chunk offset o -> slot S + C - 1 - o
            if tail > 0:
                lo = n_full * C
                slots = torch.arange(S + C - 1, S + C - 1 - tail, -1, device=qkv.device)
                put(cache.k, slots, k_t[:, lo:lo + tail])
                put(cache.v, slots, v_t[:, lo:lo + tail])
            if Ns > 0:
                k_s = qkv[B * L:, Hq * Dh:(Hq + Hkv) * Dh].view(B, Ns, Hkv, Dh)
                v_s = qkv[B * L:, (Hq + Hkv) * Dh:].view(B, Ns, Hkv, Dh)
                put(cache.k, slice(spec.sum0, spec.sum0 + Ns), k_s)
                put(cache.v, slice(spec.sum0, spec.sum0 + Ns), v_s)

        logits = self.model(tokens, kv_sink=sink, last_token_only=True)
        where = sel if contiguous else torch.tensor(rows, device=self.device)
        self.state.text_len[where] = L
        self.state.cbl[where] = tail if S > 0 else 0
        self.state.chunks[where] = n_full
        return logits[:, -1].float()

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """``tokens`` ``[B]``: the next text token of every sequence -> logits ``[B, V]``."""
        C, S = self.C, self.S
        if max(self.host_len) + 1 > self.max_len:
            self.reserve(2 * self.max_len)
        boundary_host = [S > 0 and (l % C) == C - 1 for l in self.host_len]
        anyb = any(boundary_host)
        tp = getattr(self.model, "tp", None)
        # Two graphs: steps in which no sequence closes a chunk, and steps in which some do (those carry the summary
        # rows as well; WHICH sequences close one is data, read from ``_boundary_dev``).  With tensor parallelism only
        # the first kind is captured, and the graph ends at the final norm: the vocabulary-parallel head and the
        # gather of its logits (a library collective) run after the replay.
        graphable = self.cuda_graph and tokens.is_cuda and (not anyb or tp is None)
        head_in_graph = tp is None
        if anyb:
            self._boundary_dev.copy_(torch.tensor(boundary_host, dtype=torch.int32), non_blocking=False)
        if not graphable:
            logits = self._decode_impl(tokens, anyb)
        elif anyb not in self._graphs and self._plain_steps[anyb] == 0:
            self._plain_steps[anyb] += 1    # first-call set-up of the kernels happens outside a capture
            logits = self._decode_impl(tokens, anyb)
        else:
            if self._graph_tokens is None:
                self._graph_tokens = tokens.reshape(self.batch).clone()
            if anyb not in self._graphs:
                torch.cuda.synchronize(self.device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out = self._decode_impl(self._graph_tokens, anyb, head_in_graph)
                self._graphs[anyb] = (graph, out)
            graph, out = self._graphs[anyb]
            self._graph_tokens.copy_(tokens.reshape(self.batch))
            graph.replay()
            logits = out.clone() if head_in_graph else self._head(out)
        self.host_len = [l + 1 for l in self.host_len]
        return logits

    def _head(self, hidden: torch.Tensor) -> torch.Tensor:
        model, tp = self.model, getattr(self.model, "tp", None)
        logits = ops.linear(hidden, model.lm_head_weight)
        if tp is not None and logits.shape[-1] != self.cfg.vocab_size:
            logits = tp.gather_logits(logits)
        return logits.float()

    def _decode_impl(self, tokens: torch.Tensor, any_boundary: bool, with_head: bool = True) -> torch.Tensor:
        """Device work of one decode step (launches only; the host mirror of the lengths is advanced by the caller).
        ``any_boundary``: some sequence closes a chunk in this step; which ones is read from ``_boundary_dev``."""
        if not tokens.is_cuda or os.environ.get("KSA_DEPENDENT_LAUNCH", "1") == "0":
            return self._decode_body(tokens, any_boundary, with_head)
        # a step is a chain of some four hundred kernels of a few microseconds each: launched dependently, each may
        # start (and the projections fetch their first weights) while its predecessor is still running
        before = _lib.set_dependent_launch(True)
        try:
            return self._decode_body(tokens, any_boundary, with_head)
        finally:
            _lib.set_dependent_launch(before)

    def _decode_body(self, tokens: torch.Tensor, any_boundary: bool, with_head: bool = True) -> torch.Tensor:
        model, cfg = self.model, self.cfg
        tp = getattr(model, "tp", None)      # tensor-parallel shard: cfg holds the local head counts
        B, C, S = self.batch, self.C, self.S
        Hq, Hkv, Dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        scale = Dh ** -0.5
        st = self.state
        dev = self.device
        pos_t = st.text_len.clone()                              # position of the new text token
        x = ops.embedding(tokens.reshape(B), model.tok_embeddings.weight)      # [B, D]
        if any_boundary:
            boundary = self._boundary_dev
            xs = model._summary_rows(_OneChunk(B, S), x.dtype)                 # [B*S, D]
            x = torch.cat([x, xs], dim=0)
            chunk_start = st.text_len - (C - 1)
            j = torch.arange(S, device=dev, dtype=torch.int32)
            if cfg.summary_token_position_ids_type == "zeros":
                pos_s = torch.zeros(B, S, dtype=torch.int32, device=dev)
            elif cfg.summary_token_position_ids_type == "last_chunk_slice_right":
                pos_s = torch.maximum(chunk_start[:, None] + ((j[None, :] + 1) * C) // S - 1, chunk_start[:, None])
            else:
                pos_s = torch.maximum(chunk_start[:, None] + (j[None, :] * C) // S - 1, chunk_start[:, None])
            pos_all = torch.cat([pos_t, pos_s.reshape(-1).to(torch.int32)])
        else:
            pos_all = pos_t
        if cfg.summary_enabled and cfg.summary_chunk_position_ids_type == "inner_chunk":
            pos_all = pos_all.clone()
            pos_all[:B] = st.cbl
        delta = None
        slices_of = {}      # layers with the same cache geometry share the step's slot / slice tensors
        # ordinary steps without tensor parallelism: residual add + norm live inside the projection that follows them
        fuse_norm = tp is None and not any_boundary and B <= 4
        for li, layer in enumerate(model.layers):
            a = layer.attn
            cache = self.layer_caches[li]
            if fuse_norm:
                x, qkv = ops.norm_linear(x, delta, layer.sa_norm.scale, cfg.norm_eps, a.wqkv.weight)
                h = None
            else:
                x, h = _add_norm(tp, x, delta, layer.sa_norm.scale, cfg.norm_eps)
            if layer.is_summary_layer:
                spec = self.specs[li]
                if fuse_norm:
                    pass
                elif any_boundary:
                    if layer.sa_norm_summary is not None:
                        h = torch.cat([h[:B], ops.rms_norm(x[B:], layer.sa_norm_summary.scale, cfg.norm_eps)])
                    w_s = a.wqkv_summary.weight if a.wqkv_summary is not None else a.wqkv.weight
                    qkv = ops.dual_linear(h, a.wqkv.weight, w_s, B)
                else:
                    qkv = ops.linear(h, a.wqkv.weight)
                skey = (spec.chunk, spec.n_sum, spec.window, spec.max_chunks)
                if skey not in slices_of:
                    slot_t, start_t, len_t = text_step_slices(spec, st)
                    slices_of[skey] = (slot_t.view(B, 1).to(torch.int32).contiguous(),
                                       start_t.view(B, 1).to(torch.int32).contiguous(),
                                       len_t.view(B, 1).to(torch.int32).contiguous(), start_t, len_t)
                slot_t1, start_t1, len_t1, start_t, len_t = slices_of[skey]
                # norm + rotation of q / k, and the text tokens' K / V go into the cache in the same kernel
                qkv = ops.qk_norm_rope_decode(qkv, a._norm_w(a.q_norm), a._norm_w(a.k_norm), pos_all, Hq, Hkv, Dh,
                                              cfg.rope_base, cfg.norm_eps, cfg.rope_impl == "llama", cache.k, cache.v,
                                              slot_t1)
                q_t = qkv[:B, :Hq * Dh].view(B, 1, Hq, Dh)
                if any_boundary:
                    slot_s, start_s, len_s = summary_step_slices(spec, B, dev)
                    off = torch.where(boundary[:, None] > 0, slot_s, torch.full_like(slot_s, -1))
                    q_s = qkv[B:, :Hq * Dh].view(B, S, Hq, Dh)
                    k_s = qkv[B:, Hq * Dh:(Hq + Hkv) * Dh].view(B, S, Hkv, Dh)
                    v_s = qkv[B:, (Hq + Hkv) * Dh:].view(B, S, Hkv, Dh)
                    _cache_append(k_s, v_s, cache.k, cache.v, off)
                    q_all = torch.cat([q_t, q_s], dim=1)
                    starts = torch.cat([start_t.view(B, 1), start_s], dim=1).to(torch.int32)
                    lens = torch.cat([len_t.view(B, 1), len_s * boundary[:, None]], dim=1).to(torch.int32)
                    att = _decode_attention(q_all, cache.k, cache.v, starts, lens, scale,
                                            self._merge_counters)                             # [B, 1+S, Hq, Dh]
                    att = torch.cat([att[:, 0].reshape(B, Hq * Dh), att[:, 1:].reshape(B * S, Hq * Dh)], dim=0)
                    # flush: chunk text -> ring, scratch summaries -> summary region (boundary sequences only)
                    src_t, dst_t, src_s, dst_s = flush_plan(spec, st)
                    if spec.window > 0:
                        _cache_move(cache.k, cache.v, src_t, dst_t, boundary, C)
                    _cache_move(cache.k, cache.v, src_s, dst_s, boundary, S)
                else:
                    att = _decode_attention(q_t, cache.k, cache.v, start_t1, len_t1, scale,
                                            self._merge_counters).reshape(B, Hq * Dh)
                attn_out = _row_linear(tp, att, a.output_proj.weight)
                if fuse_norm:
                    x, delta = layer.mlp.forward_after_norm(x, attn_out, layer.mlp_norm.scale, cfg.norm_eps)
                else:
                    x, h2 = _add_norm(tp, x, attn_out, layer.mlp_norm.scale, cfg.norm_eps)
                    delta = layer.mlp(h2, tp)
            else:
                if not fuse_norm:
                    qkv = ops.linear(h[:B], a.wqkv.weight)
                qkv = ops.qk_norm_rope_decode(qkv, a._norm_w(a.q_norm), a._norm_w(a.k_norm), pos_all[:B], Hq, Hkv, Dh,
                                              cfg.rope_base, cfg.norm_eps, cfg.rope_impl == "llama", cache.k, cache.v,
                                              st.text_len)
                q_t = qkv[:, :Hq * Dh].view(B, 1, Hq, Dh)
                zeros = torch.zeros(B, 1, dtype=torch.int32, device=dev)
                att = _decode_attention(q_t, cache.k, cache.v, zeros, (st.text_len + 1).view(B, 1).to(torch.int32),
                                        scale, self._merge_counters).reshape(B, Hq * Dh)
                attn_out = _row_linear(tp, att, a.output_proj.weight)
                if fuse_norm:
                    x, delta = layer.mlp.forward_after_norm(x, attn_out, layer.mlp_norm.scale, cfg.norm_eps)
                else:
                    x, h2 = _add_norm(tp, x, attn_out, layer.mlp_norm.scale, cfg.norm_eps)
                    delta = layer.mlp(h2[:B], tp)
        _, hN = _add_norm(tp, x[:B], delta[:B], model.norm.scale, cfg.norm_eps)
        # advance the counters
        st.text_len += 1
        if S > 0:
            if any_boundary:
                st.chunks += boundary
                st.cbl.copy_(torch.where(boundary > 0, torch.zeros_like(st.cbl), st.cbl + 1))
            else:
                st.cbl += 1
        return self._head(hN) if with_head else hN

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, eos_id: Optional[int] = None,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Decode ``max_new_tokens`` tokens; returns ``[B, L + new]``.  ``temperature == 0`` is greedy decoding;
        otherwise tokens are sampled from the temperature-scaled distribution restricted to the ``top_k`` most likely
        tokens and / or the smallest set whose probability mass reaches ``top_p``
        (``muse/models/qwen3/modeling.py:473-605``)."""
        logits = self.prefill(prompt)
        out = [prompt]
        done = torch.zeros(prompt.shape[0], dtype=torch.bool, device=prompt.device)
        nxt = sample_next(logits, temperature, top_k, top_p, generator)
        for i in range(max_new_tokens):
            if eos_id is not None:
                nxt = torch.where(done, torch.full_like(nxt, eos_id), nxt)
                done = done | (nxt == eos_id)
            out.append(nxt.view(-1, 1))
            if i + 1 == max_new_tokens or (eos_id is not None and bool(done.all())):
                break
            nxt = sample_next(self.decode_step(nxt), temperature, top_k, top_p, generator)
        return torch.cat(out, dim=1)


def sample_next(logits: torch.Tensor, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """``logits`` ``[B, V]`` -> token ids ``[B]`` (greedy when ``temperature <= 0``)."""
    if temperature <= 0.0:
        return logits.argmax(-1)
    logits = logits.float() / temperature
    if top_k and top_k < logits.shape[-1]:
        kth = logits.topk(top_k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, order = logits.sort(dim=-1, descending=True)
        probs = sorted_logits.softmax(-1)
        drop = probs.cumsum(-1) - probs >= top_p            # keep tokens until the mass before them reaches top_p
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, order, sorted_logits)
    return torch.multinomial(logits.softmax(-1), 1, generator=generator).squeeze(-1)


class _OneChunk:
    """Shape record for ``_summary_rows``: the summary rows of one chunk per sequence."""

    def __init__(self, B: int, S: int):
        self.B, self.Ns, self.n_sum = B, S, S
