"""Model configs: Qwen3 and Qwen3 + Kwai Summary Attention (KSA).

Field names match the reference JSON (``muse/config/model_config.py:79-437``,
``examples/pretrain/model_config/model_config_1b9_hybrid.json``) so shipped
model JSONs load as they are.  Per-layer lists may be written as pattern
strings such as ``"([1]*3+[0]*1)*7"``; they are parsed by a small grammar
here, never by ``eval``.
"""
from __future__ import annotations

from typing import Dict, List, Literal, Optional, Union

from pydantic import Field, field_validator, model_validator

from .base import BaseConfig, register_config


# --------------------------------------------------------------------------
# pattern strings:   expr := term ('+' term)* ; term := atom ('*' int)* ;
#                    atom := '[' ints ']' | '(' expr ')'
# --------------------------------------------------------------------------
class _PatternParser:
    def __init__(self, text: str):
        self.s = "".join(text.split())
        self.i = 0

    def _peek(self) -> str:
        return self.s[self.i] if self.i < len(self.s) else ""

    def _eat(self, ch: str) -> None:
        if self._peek() != ch:
            raise ValueError(f"pattern {self.s!r}: expected {ch!r} at offset {self.i}")
        self.i += 1

    def _int(self) -> int:
        j = self.i
        while self._peek().isdigit():
            self.i += 1
        if j == self.i:
            raise ValueError(f"pattern {self.s!r}: expected a number at offset {j}")
        return int(self.s[j:self.i])

    def _atom(self) -> List[int]:
        if self._peek() == "[":
            self._eat("[")
            vals: List[int] = []
            if self._peek() != "]":
                vals.append(self._int())
                while self._peek() == ",":
                    self._eat(",")
                    if self._peek() == "]":
                        break
                    vals.append(self._int())
            self._eat("]")
            return vals
        if self._peek() == "(":
            self._eat("(")
            vals = self._expr()
            self._eat(")")
            return vals
        raise ValueError(f"pattern {self.s!r}: unexpected {self._peek()!r} at offset {self.i}")

    def _term(self) -> List[int]:
        vals = self._atom()
        while self._peek() == "*":
            self._eat("*")
            vals = vals * self._int()
        return vals

    def _expr(self) -> List[int]:
        vals = self._term()
        while self._peek() == "+":
            self._eat("+")
            vals = vals + self._term()
        return vals

    def parse(self) -> List[int]:
        vals = self._expr()
        if self.i != len(self.s):
            raise ValueError(f"pattern {self.s!r}: trailing text at offset {self.i}")
        return vals


def parse_layer_pattern(text: str) -> List[int]:
    """``"([128]*3+[1024]*1)*6"`` -> a list of 24 ints."""
    if not isinstance(text, str):
        raise ValueError(f"expected a pattern string, got {type(text).__name__}")
    return _PatternParser(text).parse()


def _maybe_pattern(v):
    if isinstance(v, str) and "[" in v:
        return parse_layer_pattern(v)
    return v


class ModelConfig(BaseConfig):
    model_class: str = Field(default="", description="registered model class name")


@register_config
class Qwen3Config(ModelConfig):
    model_class: str = "Qwen3Model"
    vocab_size: int = 151936
    embed_dim: int = 4096
    num_layers: int = 32
    tie_word_embeddings: bool = True
    hidden_act: str = "silu"
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    attn_dropout: float = Field(default=0.0, ge=0.0, le=1.0)
    attention_function: Literal["eager", "flash_attention_2", "b200"] = "b200"
    q_proj_bias: bool = False
    k_proj_bias: bool = False
    v_proj_bias: bool = False
    attention_bias: bool = False
    intermediate_dim: int = 11008
    max_seq_len: int = 32768
    rope_base: float = 10000.0
    rope_impl: Literal["llama", "hf"] = "hf"
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    layer_sliding_window: Optional[Union[int, List[int]]] = None
    norm_eps: float = 1e-6
    rms_norm_eps: float = 1e-6
    q_norm: bool = True
    k_norm: bool = True
    eos_token_id: Optional[int] = 151645

    @field_validator("layer_sliding_window", mode="before")
    @classmethod
    def _parse_lsw(cls, v):
        return _maybe_pattern(v)

    @model_validator(mode="after")
    def _check_heads(self):
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(
                f"num_heads ({self.num_heads}) must be divisible by num_kv_heads ({self.num_kv_heads})")
        return self

    @property
    def sliding_window_enabled(self) -> bool:
        if self.layer_sliding_window is not None:
            return True
        return bool(self.use_sliding_window and self.sliding_window and self.sliding_window > 0)

    def get_layer_sliding_window(self, layer_idx: int) -> int:
        """Token window of a layer, or -1 for full causal attention."""
        if not self.sliding_window_enabled:
            return -1
        val = self.layer_sliding_window
        if isinstance(val, list):
            if len(val) != self.num_layers:
                raise ValueError("layer_sliding_window list length != num_layers")
            w = val[layer_idx]
        elif isinstance(val, int):
            w = val
        else:
            w = self.sliding_window
        return int(w) if w and w > 0 else -1

    # derived sizes ---------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    def num_parameters(self) -> int:
        d, f = self.embed_dim, self.intermediate_dim
        per_layer = d * (self.q_dim + 2 * self.kv_dim) + self.q_dim * d + 3 * d * f + 2 * d
        if self.q_norm:
            per_layer += self.head_dim
        if self.k_norm:
            per_layer += self.head_dim
        total = self.num_layers * per_layer + d + self.vocab_size * d
        if not self.tie_word_embeddings:
            total += self.vocab_size * d
        return total


@register_config
class Qwen3SummaryAttentionConfig(Qwen3Config):
    model_class: str = "Qwen3SummaryModel"
    use_summary_attention: bool = False
    summary_chunk_size: int = 0
    summary_token_num: int = 0
    summary_sliding_chunk_num: Union[int, List[int]] = 0
    summary_token_begin: Optional[int] = None
    summary_layer_freq: Union[int, List[int]] = 0
    summary_independent_parameters: bool = False
    summary_independent_qkv: Optional[bool] = None
    summary_independent_attention_layernorm: bool = False
    summary_independent_qk_norm: bool = False
    summary_mix_qkv: bool = False
    summary_mix_start_iter: int = 0
    summary_mix_end_iter: int = 0
    summary_chunk_position_ids_type: Literal["inner_chunk", "origin"] = "inner_chunk"
    summary_token_position_ids_type: Literal[
        "zeros", "last_chunk_slice_right", "last_chunk_slice_left"] = "zeros"
    summary_attention_mode: Literal["kernel", "mask", "block"] = "kernel"
    enable_summary_distill_attention: bool = False
    summary_distill_attention_norm: bool = False

    @field_validator("summary_layer_freq", "summary_sliding_chunk_num", mode="before")
    @classmethod
    def _parse_patterns(cls, v):
        return _maybe_pattern(v)

    @property
    def summary_enabled(self) -> bool:
        return bool(self.use_summary_attention and self.summary_chunk_size > 0
                    and self.summary_token_num > 0)

    @property
    def use_independent_qkv(self) -> bool:
        if self.summary_independent_qkv is not None:
            return self.summary_independent_qkv
        return self.summary_independent_parameters

    def get_layer_is_summary(self) -> List[bool]:
        """Per layer: True = summary-attention layer, False = full causal layer.

        ``0`` = every layer; int ``N`` = layers with ``i % N == 0``; a list is a
        bitmask (``muse/config/model_config.py:408-423``).
        """
        freq = self.summary_layer_freq
        if isinstance(freq, list):
            if len(freq) != self.num_layers:
                raise ValueError(
                    f"summary_layer_freq has {len(freq)} entries for {self.num_layers} layers")
            return [bool(x) for x in freq]
        if freq == 0:
            return [True] * self.num_layers
        return [(i % freq == 0) for i in range(self.num_layers)]

    def get_layer_sliding_chunk_num(self, layer_idx: int) -> int:
        val = self.summary_sliding_chunk_num
        if isinstance(val, list):
            if len(val) != self.num_layers:
                raise ValueError(
                    f"summary_sliding_chunk_num has {len(val)} entries for {self.num_layers} layers")
            return int(val[layer_idx])
        return int(val)

    def num_parameters(self) -> int:
        total = super().num_parameters()
        if not self.summary_enabled:
            return total
        d = self.embed_dim
        if self.summary_independent_parameters:
            total += self.summary_token_num * d
        n_sa = sum(self.get_layer_is_summary())
        if self.use_independent_qkv:
            total += n_sa * d * (self.q_dim + 2 * self.kv_dim)
            if self.summary_independent_attention_layernorm:
                total += n_sa * d
            if self.summary_independent_qk_norm:
                total += n_sa * 2 * self.head_dim
        return total


# --------------------------------------------------------------------------
# Named shapes used by the benchmarks and tests.
# --------------------------------------------------------------------------
def _ksa(**kw) -> Qwen3SummaryAttentionConfig:
    base = dict(
        use_summary_attention=True, summary_token_num=1, summary_independent_parameters=True,
        summary_chunk_position_ids_type="origin",
        summary_token_position_ids_type="last_chunk_slice_right",
        tie_word_embeddings=False, q_norm=True, k_norm=True, rope_impl="hf",
    )
    base.update(kw)
    base.setdefault("summary_token_begin", base["vocab_size"])
    return Qwen3SummaryAttentionConfig(**base)


def qwen3_ksa_tiny() -> Qwen3SummaryAttentionConfig:
    """4 layers (3 summary : 1 full), hidden 256, 4Q/2KV x 64, FFN 768, chunk 64, window 4."""
    return _ksa(vocab_size=4096, embed_dim=256, num_layers=4, num_heads=4, num_kv_heads=2,
                head_dim=64, intermediate_dim=768, max_seq_len=8192, rope_base=1e6,
                summary_chunk_size=64, summary_sliding_chunk_num=4,
                summary_layer_freq="([1]*3+[0]*1)*1")


def qwen3_ksa_1b9() -> Qwen3SummaryAttentionConfig:
    """28 layers (3:1), hidden 2048, 16Q/8KV x 128, FFN 6144, vocab 151936, chunk 128, window 8."""
    return _ksa(vocab_size=151936, embed_dim=2048, num_layers=28, num_heads=16, num_kv_heads=8,
                head_dim=128, intermediate_dim=6144, max_seq_len=131072, rope_base=1e6,
                summary_chunk_size=128, summary_sliding_chunk_num=8,
                summary_layer_freq="([1]*3+[0]*1)*7")


def qwen3_ksa_4b() -> Qwen3SummaryAttentionConfig:
    """Qwen3-4B shape: 36 layers (3:1), hidden 2560, 32Q/8KV x 128, FFN 9728."""
    return _ksa(vocab_size=151936, embed_dim=2560, num_layers=36, num_heads=32, num_kv_heads=8,
                head_dim=128, intermediate_dim=9728, max_seq_len=131072, rope_base=1e6,
                summary_chunk_size=128, summary_sliding_chunk_num=8,
                summary_layer_freq="([1]*3+[0]*1)*9")


def qwen3_ksa_shipped_1b9() -> Qwen3SummaryAttentionConfig:
    """The shape of the reference's shipped JSON: 24 layers, 16/16 heads, chunk 8, all-SA."""
    return _ksa(vocab_size=151936, embed_dim=2048, num_layers=24, num_heads=16, num_kv_heads=16,
                head_dim=128, intermediate_dim=6144, max_seq_len=131072, rope_base=10000,
                summary_chunk_size=8, summary_sliding_chunk_num="([128]*3+[1024]*1)*6")


PRESETS: Dict[str, object] = {
    "qwen3-ksa-tiny": qwen3_ksa_tiny,
    "qwen3-1.9b-ksa": qwen3_ksa_1b9,
    "ksa-4b": qwen3_ksa_4b,
    "qwen3-1.9b-ksa-shipped": qwen3_ksa_shipped_1b9,
}


def get_preset(name: str) -> Qwen3SummaryAttentionConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: {sorted(PRESETS)}")
    return PRESETS[name]()
