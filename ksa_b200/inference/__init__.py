from .cache import CacheSpec, CacheState, FullLayerCache, KsaLayerCache
from .engine import KsaInferenceEngine

__all__ = ["CacheSpec", "CacheState", "FullLayerCache", "KsaLayerCache", "KsaInferenceEngine"]
