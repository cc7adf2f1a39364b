"""Model / hardware FLOPs utilisation from the config alone (``muse/utils/mfu.py:32-146``).

Per token and layer the forward costs ``2h(hq+2hkv) + 2*s*hq + 2*hq*h + 6*h*ffn`` FLOPs (projections, attention
scores+values at context ``s``, output projection, SwiGLU) and the logits ``2hV``; a training step costs 3x the
forward (4x in hardware terms with full activation recomputation); distillation adds a teacher forward.  The
reference's peak table stops at Hopper, which silently disables MFU on B200; this one knows Blackwell and prefers a
measured peak when one is given."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

PEAK_BF16_TFLOPS = {
    "A100": 312.0, "A800": 312.0, "H100": 989.0, "H800": 989.0, "H20": 148.0, "H200": 989.0,
    "B200": 2250.0, "B100": 1800.0, "GB200": 2500.0,
}


def device_peak_tflops(name: Optional[str] = None, measured: Optional[float] = None) -> Optional[float]:
    """Dense bf16 peak for a device name (substring match); ``measured`` (e.g. a cuBLAS burst) wins when given."""
    if measured:
        return float(measured)
    if name is None:
        try:
            import torch
            name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else None
        except Exception:
            name = None
    if not name:
        return None
    for key, val in PEAK_BF16_TFLOPS.items():
        if key in name.upper():
            return val
    return None


@dataclass
class FlopsModel:
    hidden: int
    q_dim: int
    kv_dim: int
    ffn: int
    vocab: int
    layers: int
    summary_chunk: int = 0
    summary_tokens: int = 0

    @classmethod
    def from_config(cls, cfg) -> "FlopsModel":
        enabled = bool(getattr(cfg, "summary_enabled", False))
        return cls(cfg.embed_dim, cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim,
                   cfg.intermediate_dim, cfg.vocab_size, cfg.num_layers,
                   cfg.summary_chunk_size if enabled else 0, cfg.summary_token_num if enabled else 0)

    def expanded_len(self, seq_len: int) -> int:
        if self.summary_chunk <= 0:
            return seq_len
        return seq_len + -(-seq_len // self.summary_chunk) * self.summary_tokens

    def forward_flops(self, seq_len: int, with_summary: bool = True) -> float:
        """Forward FLOPs of one sequence, dense-attention accounting like the reference (context = sequence)."""
        s = self.expanded_len(seq_len) if with_summary else seq_len
        h = self.hidden
        per_token_layer = 2 * h * (self.q_dim + 2 * self.kv_dim) + 2 * s * self.q_dim + 2 * self.q_dim * h + 6 * h * self.ffn
        return s * self.layers * per_token_layer + seq_len * 2 * h * self.vocab

    def step_flops(self, seq_len: int, grad_checkpointing: bool = False, distill: bool = False):
        """(model FLOPs, hardware FLOPs) of one training sequence."""
        fwd = self.forward_flops(seq_len)
        teacher = self.forward_flops(seq_len, with_summary=False) if distill else 0.0
        model = 3 * fwd + teacher
        hardware = (4 if grad_checkpointing else 3) * fwd + teacher
        return model, hardware


def mfu(tokens_per_sec_per_gpu: float, cfg, seq_len: int, peak_tflops: Optional[float] = None,
        grad_checkpointing: bool = False, distill: bool = False) -> dict:
    fm = FlopsModel.from_config(cfg)
    model, hw = fm.step_flops(seq_len, grad_checkpointing, distill)
    seqs_per_sec = tokens_per_sec_per_gpu / seq_len
    peak = device_peak_tflops(measured=peak_tflops)
    out = {"tflops_per_gpu": model * seqs_per_sec / 1e12, "hw_tflops_per_gpu": hw * seqs_per_sec / 1e12}
    if peak:
        out["mfu"] = out["tflops_per_gpu"] / peak
        out["hfu"] = out["hw_tflops_per_gpu"] / peak
    return out
