from .ce import CrossEntropyLoss
from .distill import attention_cosine_loss, attention_mse_loss, kl_divergence_loss
from .chunked import ChunkedDistillLossComputer

__all__ = ["CrossEntropyLoss", "attention_mse_loss", "attention_cosine_loss", "kl_divergence_loss",
           "ChunkedDistillLossComputer"]
