"""ksa_b200: Blackwell-native training and inference for Qwen3 + Kwai Summary Attention."""
__version__ = "0.1.0"
