"""Losses, train-loop utilities, metrics and the FLOP model on CPU."""
import csv
import math
import os

import pytest
import torch
import torch.nn.functional as F
from torch import nn

from ksa_b200.config import get_preset
from ksa_b200.losses import ChunkedDistillLossComputer, CrossEntropyLoss
from ksa_b200.losses.distill import attention_cosine_loss, attention_mse_loss, kl_divergence_loss, rms_normalize
from ksa_b200.training.common import (GradNormLogger, clip_grad_by_value, compute_grad_norm, freeze_params_by_pattern,
                                      set_default_dtype, to_dtype)
from ksa_b200.utils.metrics import CSVBackend, DerivedSeries, Metrics, Series, SimpleMetrics, initialize_metrics


# ------------------------------------------------------------------------------------------------ losses
def test_cross_entropy_modes():
    torch.manual_seed(0)
    logits, labels = torch.randn(2, 7, 11), torch.randint(0, 11, (2, 7))
    labels[0, 2] = -100
    ref = F.cross_entropy(logits.reshape(-1, 11), labels.reshape(-1), ignore_index=-100)
    torch.testing.assert_close(CrossEntropyLoss()(logits, labels), ref)
    per_tok = CrossEntropyLoss(reduction="none")(logits, labels)
    assert per_tok.shape == (2, 7) and per_tok[0, 2] == 0
    shifted = CrossEntropyLoss(shift_labels=True)(logits, labels)
    ref_s = F.cross_entropy(logits[:, :-1].reshape(-1, 11), labels[:, 1:].reshape(-1), ignore_index=-100)
    torch.testing.assert_close(shifted, ref_s)
    assert float(CrossEntropyLoss()(logits, torch.full((2, 7), -100))) == 0.0       # nothing to predict: no NaN


@pytest.mark.parametrize("enable_kl", [False, True])
def test_chunked_loss_computer_matches_direct_computation(enable_kl):
    torch.manual_seed(1)
    B, L, D, V = 2, 9, 16, 37
    w = nn.Parameter(torch.randn(V, D) * 0.3)
    h = (torch.randn(B, L, D)).requires_grad_(True)
    th = torch.randn(B, L, D)
    labels = torch.randint(0, V, (B, L))
    labels[1, 3:5] = -100
    # direct
    logits = h.reshape(-1, D) @ w.t()
    ce = F.cross_entropy(logits, labels.reshape(-1), ignore_index=-100)
    total = 1.5 * ce
    if enable_kl:
        valid = labels.reshape(-1) != -100
        kl = kl_divergence_loss(logits[valid], (th.reshape(-1, D) @ w.t())[valid])
        total = total + 0.7 * kl
    gh, gw = torch.autograd.grad(total, [h, w])
    # chunked, 4 tokens at a time
    h2 = h.detach().clone().requires_grad_(True)
    w2 = nn.Parameter(w.detach().clone())
    comp = ChunkedDistillLossComputer(w2, minibatch_size=4, lm_factor=1.5, kl_factor=0.7, enable_kl=enable_kl)
    out = comp.forward_and_backward(h2, th if enable_kl else None, labels)
    torch.testing.assert_close(out["total_loss"], total.detach(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(h2.grad, gh, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(w2.grad, gw, atol=1e-5, rtol=1e-4)
    # gradient accumulation scales the gradients, not the reported loss
    h3 = h.detach().clone().requires_grad_(True)
    w3 = nn.Parameter(w.detach().clone())
    out3 = ChunkedDistillLossComputer(w3, 4, 1.5, 0.7, enable_kl).forward_and_backward(h3, th if enable_kl else None, labels,
                                                                                      gradient_accumulation_steps=2)
    torch.testing.assert_close(out3["total_loss"], out["total_loss"])
    torch.testing.assert_close(h3.grad, gh / 2, atol=1e-5, rtol=1e-4)


def test_attention_matching_losses():
    s = [torch.randn(4, 8), torch.randn(4, 8)]
    t = [x + 0.01 * torch.randn_like(x) for x in s]
    assert float(attention_mse_loss(s, t)) < 1e-3 and float(attention_cosine_loss(s, t)) < 1e-3
    far = [x + 10.0 for x in s]
    assert float(attention_mse_loss(s, far)) == pytest.approx(0.1)          # clamped per layer
    assert float(attention_mse_loss([], [])) == 0.0
    x = torch.randn(3, 5) * 7
    torch.testing.assert_close(rms_normalize(x).pow(2).mean(-1), torch.ones(3), atol=1e-4, rtol=1e-4)
    same = kl_divergence_loss(torch.randn(6, 9).requires_grad_(True), torch.randn(6, 9))
    assert float(same.detach()) > 0 and float(kl_divergence_loss(s[0], s[0])) == pytest.approx(0.0, abs=1e-6)


# ------------------------------------------------------------------------------------------------ train-loop utilities
def test_clip_norm_freeze_and_dtype_helpers(tmp_path):
    model = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    for i, p in enumerate(model.parameters()):
        p.grad = torch.full_like(p, 3.0 * (-1) ** i)
    norm = compute_grad_norm(model.parameters())
    n_el = sum(p.numel() for p in model.parameters())
    assert float(norm) == pytest.approx(3.0 * math.sqrt(n_el))
    clip_grad_by_value(model, 0.5)
    assert all(float(p.grad.abs().max()) == 0.5 for p in model.parameters())
    clip_grad_by_value(model, None)                                          # no range: untouched
    stats = freeze_params_by_pattern(model, ["1.weight"])
    assert stats["trainable"] == 8 and stats["frozen"] == n_el - 8
    assert [n for n, p in model.named_parameters() if p.requires_grad] == ["1.weight"]
    assert to_dtype("bfloat16") is torch.bfloat16 and to_dtype(torch.float16) is torch.float16
    with set_default_dtype("bfloat16"):
        assert torch.zeros(1).dtype == torch.bfloat16
    assert torch.zeros(1).dtype == torch.float32
    log = GradNormLogger(str(tmp_path / "gn.csv"), every=2)
    for step in range(4):
        log.log(step, [(n, p.grad) for n, p in model.named_parameters()])
    rows = list(csv.reader(open(tmp_path / "gn.csv")))
    assert len(rows) >= 2


def test_activation_checkpointing_keeps_gradients():
    from ksa_b200.models import get_model_class
    from ksa_b200.training.activations import set_activation_checkpointing
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 128, "head_dim": 16,
                                               "summary_chunk_size": 16})
    grads = []
    for ckpt in (False, True):
        torch.manual_seed(0)
        m = get_model_class(cfg.model_class)(cfg)
        m.init_weights(seed=0)
        m = m.float()
        if ckpt:
            assert set_activation_checkpointing(m, m.get_checkpointable_module_classes()) == 2
        toks = torch.randint(0, 128, (2, 65), generator=torch.Generator().manual_seed(3))
        m(toks[:, :-1], toks[:, 1:]).backward()
        grads.append({n.replace("_checkpoint_wrapped_module.", ""): p.grad.clone() for n, p in m.named_parameters()})
    assert grads[0].keys() == grads[1].keys()
    for n in grads[0]:
        torch.testing.assert_close(grads[0][n], grads[1][n], atol=1e-6, rtol=1e-5)


def test_selective_recomputation_of_the_feed_forward_blocks_keeps_gradients_and_saves_less():
    """``mode="mlp"``: same loss and gradients; the tensors autograd keeps alive shrink by the gate/up projection and
    the SwiGLU output of every layer, and no layer is wrapped (parameter names stay as they are)."""
    from ksa_b200.models import get_model_class
    from ksa_b200.training.activations import set_activation_checkpointing
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 256, "vocab_size": 128, "head_dim": 16,
                                               "summary_chunk_size": 16})
    out = []
    for mode in (None, "mlp", "full"):
        m = get_model_class(cfg.model_class)(cfg)
        m.init_weights(seed=0)
        m = m.float()
        if mode:
            assert set_activation_checkpointing(m, m.get_checkpointable_module_classes(), mode=mode) == 2
        toks = torch.randint(0, 128, (2, 65), generator=torch.Generator().manual_seed(3))
        kept = {}

        def pack(t):
            kept[(t.data_ptr(), t.shape)] = t.numel() * t.element_size()
            return t
        with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
            loss = m(toks[:, :-1], toks[:, 1:])
        loss.backward()
        params = {p.data_ptr() for p in m.parameters()}
        saved = sum(v for (ptr, _), v in kept.items() if ptr not in params)
        out.append((float(loss.detach()), {n.replace("_checkpoint_wrapped_module.", ""): p.grad.clone()
                                  for n, p in m.named_parameters()}, saved, [n for n, _ in m.named_parameters()]))
    (l0, g0, s0, n0), (l1, g1, s1, n1), (l2, g2, s2, _) = out
    assert l0 == l1 == l2 and n0 == n1
    for n in g0:
        torch.testing.assert_close(g0[n], g1[n], atol=1e-6, rtol=1e-5)
    rows = 2 * 64                                 # text rows; the summary rows only add to the saving
    assert s0 - s1 >= 2 * rows * 3 * 256 * 4      # two layers x (gate | up | activation) in fp32
    assert s2 < s1 < s0
    with pytest.raises(ValueError):
        set_activation_checkpointing(m, None, mode="attention")


# ------------------------------------------------------------------------------------------------ metrics
def test_series_algebra_is_lazy_and_exact():
    s = Series("x")
    s.extend([1, 2, torch.tensor(3.0), 4])
    assert s.values() == [1.0, 2.0, 3.0, 4.0] and s.latest() == 4.0
    avg2 = s.avg(2)
    assert avg2.values() == [3.5]
    s.append(6)
    assert avg2.values() == [5.0]                                   # derived views are computed when read
    assert s.cumsum().values() == [1, 3, 6, 10, 16] and s.diff().values() == [1, 1, 1, 2]
    assert s.shift(2, fill=-1).values() == [-1, -1, 1, 2, 3] and s[1:3].values() == [2, 3] and s.last(2).values() == [4, 6]
    t = Series("t")
    t.extend([2, 2, 2, 2, 3])
    assert (s / t).values() == [0.5, 1, 1.5, 2, 2] and ((s + 1) * 2).values() == [4, 6, 8, 10, 14]
    assert s.sum(3).values() == [13] and (s - t).latest() == 3
    with pytest.raises(TypeError):
        avg2.append(1)


def test_metrics_reports_and_backends(tmp_path):
    m = initialize_metrics(seq_length=64, world_size=4, log_every=2, backends=[CSVBackend(str(tmp_path / "m.csv"))])
    for step in range(4):
        m.loss.append(torch.tensor(4.0 - step))
        m.tokens.append(128)
        m.samples.append(2)
        m.grad_norm.append(1.0 + step)
        m.learning_rate.append(1e-3)
        m.step_time.append(0.5)
        m.step()
        if step % 2 == 1:
            out = m.write(step + 1)
    assert out["loss"] == pytest.approx(1.5) and out["grad_norm"] == 4.0
    assert out["total_tokens"] == 512 and out["tokens_per_sec_per_gpu"] == pytest.approx(256.0)
    assert out["tokens_per_day"] == pytest.approx(256.0 * 86400 * 4)
    m.close()
    rows = list(csv.DictReader(open(tmp_path / "m.csv")))
    assert len(rows) == 2 and float(rows[-1]["loss"]) == pytest.approx(1.5)
    sm = SimpleMetrics()
    sm.update(loss=2.0, lr=1.0)
    sm.update(loss=4.0)
    summary = sm.summary()
    assert summary["loss"] == 3.0 and summary["lr"] == 1.0 and "elapsed" in summary


def test_flops_model_and_mfu():
    from ksa_b200.utils.mfu import FlopsModel, device_peak_tflops, mfu
    cfg = get_preset("qwen3-1.9b-ksa")
    fm = FlopsModel.from_config(cfg)
    h, q, kv, ffn, V, L = cfg.embed_dim, cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim, \
        cfg.intermediate_dim, cfg.vocab_size, 8192
    s = L + (L // cfg.summary_chunk_size) * cfg.summary_token_num            # the student sequence includes summary tokens
    assert fm.expanded_len(L) == s
    per_tok = 2 * h * (q + 2 * kv) + 2 * s * q + 2 * q * h + 6 * h * ffn     # the reference's per-token, per-layer formula
    assert fm.forward_flops(L) == pytest.approx(s * cfg.num_layers * per_tok + L * 2 * h * V)
    model, hw = fm.step_flops(L)
    assert model == hw == pytest.approx(3 * fm.forward_flops(L))
    model_d, hw_d = fm.step_flops(L, grad_checkpointing=True, distill=True)
    teacher = fm.forward_flops(L, with_summary=False)
    assert model_d == pytest.approx(3 * fm.forward_flops(L) + teacher) and hw_d == pytest.approx(4 * fm.forward_flops(L) + teacher)
    assert device_peak_tflops("NVIDIA B200") is not None and device_peak_tflops("NVIDIA H100 80GB") == pytest.approx(989)
    assert device_peak_tflops("some other device") is None
    rep = mfu(60000.0, cfg, L, peak_tflops=2250.0)
    assert 0.2 < rep["mfu"] < 0.6 and rep["tflops_per_gpu"] > 500
    rep_ckpt = mfu(60000.0, cfg, L, peak_tflops=2250.0, grad_checkpointing=True)
    assert rep_ckpt["hfu"] > rep["hfu"] and rep_ckpt["mfu"] == pytest.approx(rep["mfu"])


def test_small_helpers():
    import time
    from ksa_b200.utils.common import Timer, dist_reduce_dict, get_rank, get_world_size, set_random_seed, to_cuda
    from ksa_b200.utils.tracing import StepTimer, nvtx_range
    set_random_seed(5)
    a = torch.rand(3)
    set_random_seed(5)
    assert torch.equal(a, torch.rand(3))
    assert get_rank() == 0 and get_world_size() == 1
    assert dist_reduce_dict({"a": 2.0, "b": 4.0}) == {"a": 2.0, "b": 4.0}          # single process: unchanged
    nested = to_cuda({"x": torch.ones(2), "y": [torch.zeros(1), "s"]}, device="cpu")
    assert nested["y"][1] == "s" and nested["x"].device.type == "cpu"
    with Timer("block") as t:
        time.sleep(0.01)
    assert t.elapsed >= 0.01
    st = StepTimer(device="cpu")
    for _ in range(3):
        with nvtx_range("step"):
            time.sleep(0.002)
        st.tick()
    s = st.summary()
    assert s["steps"] == 3 and s["min_ms"] >= 1.0


def test_benchmark_flags_survive_the_torchrun_parser():
    """``torch.distributed.run`` parses abbreviations of its own options before the script's arguments are split off
    (``--m`` is ambiguous there): the multi-GPU benchmark modes are documented with spellings that pass through."""
    from torch.distributed.run import get_args_parser
    from ksa_b200.tools import infer_bench, kernel_bench
    launcher = get_args_parser()
    for module, argv in (
            ("ksa_b200.tools.kernel_bench", ["ag-gemm", "--gemm-m", "33024", "--gemm-n", "1536", "--gemm-k", "2560"]),
            ("ksa_b200.tools.kernel_bench", ["gemm-rs", "--gemm-m", "33024", "--gemm-k", "2048", "--dim", "2560"]),
            ("ksa_b200.tools.kernel_bench", ["cp-attn", "--seq", "32768", "--bwd"]),
            ("ksa_b200.tools.infer_bench", ["--prompt-len", "32768", "--decode", "0", "--tp-two-phase-min", "2",
                                            "--tp-separate-gather", "--tp-pull-partials"])):
        a = launcher.parse_args(["--nproc-per-node", "2", "--master-addr", "127.0.0.1", "-m", module] + argv)
        assert a.training_script == module and a.training_script_args == argv
    k = kernel_bench.build_parser().parse_args(["ag-gemm", "--gemm-m", "33024", "--gemm-n", "1536", "--gemm-k", "2560"])
    assert (k.m, k.n, k.k) == (33024, 1536, 2560)
    k = kernel_bench.build_parser().parse_args(["gemm", "--m", "128", "--pair", "--scatter-world", "4"])
    assert k.m == 128 and k.pair and k.scatter_world == 4
    assert infer_bench is not None


def test_bench_clock_sampler_parses_nvidia_smi_lines(tmp_path, monkeypatch):
    """The benchmark's clock record: median SM clock, maximum clock and the throttle reasons seen while it ran, read
    from ``nvidia-smi`` query lines (here produced by a stand-in executable; the sampler only reads)."""
    import os
    import stat
    import sys
    import time
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    try:
        import bench
    finally:
        sys.path.remove(root)
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/bash\n"
                    "echo '0, 1650, 1965, 990.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1710, 1965, 985.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1965, 1965, 400.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo 'garbage line'\n"
                    "sleep 30\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}:{os.environ['PATH']}")
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.5)
    rec = s.stop()
    assert rec["samples"] == 3 and rec["sm_mhz"] == 1710.0 and rec["sm_max_mhz"] == 1965.0
    assert rec["reasons"] == ["sw_power_cap"]
    # without the tool the record says so instead of failing the benchmark
    monkeypatch.setenv("PATH", str(tmp_path / "empty"))
    s = bench.ClockSampler(0)
    s.start()
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]
