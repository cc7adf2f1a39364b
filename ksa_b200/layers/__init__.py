"""Generic building blocks (the reference's ``muse/layers`` package): norms, rotary embeddings, feed-forward,
tied linear, KV cache, attention back ends, multi-head attention and a generic transformer decoder.

The Qwen3 / Qwen3-KSA models use fused parameter layouts of their own (``ksa_b200.models``); these modules give the
same capabilities as stand-alone ``nn.Module`` blocks.  On CUDA bf16 tensors they run this package's sm_100a kernels,
elsewhere the fp32 PyTorch statements of the same math.
"""
from .attention import MultiHeadAttention
from .attention_utils import ATTENTION_BACKENDS, EagerAttention, TensorCoreAttention, get_attention_backend
from .feed_forward import FeedForward
from .kv_cache import KVCache
from .layer_norm import Fp32LayerNorm
from .linear import TiedLinear
from .position_embeddings import LlamaRotaryPositionalEmbeddings, RotaryPositionalEmbeddings
from .rms_norm import RMSNorm
from .summary_utils import SummaryBatch, build_summary_batch
from .transformer import TransformerCrossAttentionLayer, TransformerDecoder, TransformerSelfAttentionLayer

__all__ = ["MultiHeadAttention", "ATTENTION_BACKENDS", "EagerAttention", "TensorCoreAttention", "get_attention_backend",
           "FeedForward", "KVCache", "Fp32LayerNorm", "TiedLinear", "LlamaRotaryPositionalEmbeddings",
           "RotaryPositionalEmbeddings", "RMSNorm", "SummaryBatch", "build_summary_batch",
           "TransformerCrossAttentionLayer", "TransformerDecoder", "TransformerSelfAttentionLayer"]
