from .base import Model, get_model_class, list_models, register_model
from .qwen3_ksa import Qwen3Model, Qwen3SummaryModel

__all__ = ["Model", "get_model_class", "list_models", "register_model", "Qwen3Model", "Qwen3SummaryModel"]
