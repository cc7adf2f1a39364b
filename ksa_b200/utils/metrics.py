"""Training metrics: lazy series algebra, device-side accumulation, rank reduction at log cadence, pluggable sinks.

Feature parity with ``muse/utils/metrics.py`` (``Series`` / ``DerivedSeries`` with avg/sum/cumsum/diff/shift/slicing,
``Metrics.step()``, Stdout / CSV / TensorBoard / W&B back ends) and ``muse/training/simple_metrics.py``.  What differs
on purpose: the reference runs ``all_gather_object`` over every series on every micro-step
(``muse/utils/metrics.py:2143``) and reads losses with ``.item()`` each step; here a value may be a device scalar that
is appended without synchronising, and ranks are reduced with ONE tensor all-reduce when the metrics are written.
"""
from __future__ import annotations

import csv
import math
import os
import time
from typing import Callable, Dict, List, Optional, Sequence, Union

import torch
import torch.distributed as dist

Number = Union[int, float, torch.Tensor]


def _to_float(v: Number) -> float:
    if torch.is_tensor(v):
        return float(v.detach().float().item())
    return float(v)


class Series:
    """A named, growing sequence of scalars with lazy derived views."""

    def __init__(self, name: str, reduce: str = "mean"):
        self.name = name
        self.reduce = reduce            # how ranks are combined: "mean" | "sum" | "max" | "none"
        self._values: List[Number] = []

    # ---- recording
    def append(self, v: Number) -> None:
        self._values.append(v.detach() if torch.is_tensor(v) else v)

    def extend(self, vs: Sequence[Number]) -> None:
        for v in vs:
            self.append(v)

    def __len__(self) -> int:
        return len(self._values)

    def values(self) -> List[float]:
        """Materialise (device scalars are read here, in one batch per device)."""
        tensors = [(i, v) for i, v in enumerate(self._values) if torch.is_tensor(v)]
        if tensors:
            stacked = torch.stack([v.float().reshape(()) for _, v in tensors]).cpu().tolist()
            for (i, _), f in zip(tensors, stacked):
                self._values[i] = f
        return [float(v) for v in self._values]

    # ---- lazy algebra
    def _derive(self, fn: Callable[[List[float]], List[float]], label: str) -> "DerivedSeries":
        return DerivedSeries(f"{label}({self.name})", [self], lambda xs: fn(xs[0]), self.reduce)

    def __getitem__(self, key) -> "DerivedSeries":
        if isinstance(key, slice):
            return self._derive(lambda v: v[key], f"slice[{key.start}:{key.stop}:{key.step}]")
        return self._derive(lambda v: [v[key]], f"item[{key}]")

    def last(self, n: int = 1) -> "DerivedSeries":
        return self._derive(lambda v: v[-n:], f"last{n}")

    def avg(self, window: Optional[int] = None) -> "DerivedSeries":
        def f(v):
            w = v if window is None else v[-window:]
            return [sum(w) / len(w)] if w else []
        return self._derive(f, f"avg{window or ''}")

    def sum(self, window: Optional[int] = None) -> "DerivedSeries":
        return self._derive(lambda v: [math.fsum(v if window is None else v[-window:])], f"sum{window or ''}")

    def cumsum(self) -> "DerivedSeries":
        def f(v):
            out, acc = [], 0.0
            for x in v:
                acc += x
                out.append(acc)
            return out
        return self._derive(f, "cumsum")

    def diff(self) -> "DerivedSeries":
        return self._derive(lambda v: [b - a for a, b in zip(v[:-1], v[1:])], "diff")

    def shift(self, n: int = 1, fill: float = 0.0) -> "DerivedSeries":
        return self._derive(lambda v: ([fill] * n + v)[:len(v)] if n >= 0 else v[-n:] + [fill] * (-n), f"shift{n}")

    def _binary(self, other, op, sym) -> "DerivedSeries":
        if isinstance(other, Series):
            return DerivedSeries(f"({self.name}{sym}{other.name})", [self, other],
                                 lambda xs: [op(a, b) for a, b in zip(xs[0], xs[1])], self.reduce)
        return self._derive(lambda v: [op(a, other) for a in v], f"{sym}{other}")

    def __add__(self, o): return self._binary(o, lambda a, b: a + b, "+")
    def __sub__(self, o): return self._binary(o, lambda a, b: a - b, "-")
    def __mul__(self, o): return self._binary(o, lambda a, b: a * b, "*")
    def __truediv__(self, o): return self._binary(o, lambda a, b: a / b if b else float("nan"), "/")

    def latest(self) -> Optional[float]:
        v = self.values()
        return v[-1] if v else None

    def clear(self) -> None:
        self._values = []


class DerivedSeries(Series):
    """A view computed from parent series when read."""

    def __init__(self, name: str, parents: List[Series], fn: Callable[[List[List[float]]], List[float]], reduce="mean"):
        super().__init__(name, reduce)
        self._parents, self._fn = parents, fn

    def append(self, v):
        raise TypeError("a derived series is read-only")

    def values(self) -> List[float]:
        return list(self._fn([p.values() for p in self._parents]))

    def __len__(self) -> int:
        return len(self.values())


# ------------------------------------------------------------------------------------------------------- sinks
class MetricsBackend:
    def write(self, step: int, scalars: Dict[str, float]) -> None:
        raise NotImplementedError

    def close(self) -> None:
        pass


class StdoutBackend(MetricsBackend):
    def write(self, step, scalars):
        body = " | ".join(f"{k}={v:.6g}" for k, v in scalars.items())
        print(f"[Metrics] step={step} | {body}", flush=True)


class CSVBackend(MetricsBackend):
    def __init__(self, path: str):
        self.path = path
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self._fields: Optional[List[str]] = None

    def write(self, step, scalars):
        row = {"step": step, **scalars}
        new = not os.path.exists(self.path) or self._fields is None
        if self._fields is None or any(k not in self._fields for k in row):
            self._fields = list(row) if self._fields is None else self._fields + [k for k in row if k not in self._fields]
            new = True
        mode = "a" if os.path.exists(self.path) and not new else "a"
        with open(self.path, mode, newline="") as f:
            w = csv.DictWriter(f, fieldnames=self._fields)
            if new:
                w.writeheader()
            w.writerow(row)


class TensorBoardBackend(MetricsBackend):
    def __init__(self, log_dir: str):
        from torch.utils.tensorboard import SummaryWriter
        self.writer = SummaryWriter(log_dir=log_dir)

    def write(self, step, scalars):
        for k, v in scalars.items():
            self.writer.add_scalar(k, v, step)

    def close(self):
        self.writer.close()


class WandbBackend(MetricsBackend):
    def __init__(self, **init_kwargs):
        import wandb  # optional dependency
        self._wandb = wandb
        wandb.init(**init_kwargs)

    def write(self, step, scalars):
        self._wandb.log(scalars, step=step)

    def close(self):
        self._wandb.finish()


# ------------------------------------------------------------------------------------------------------- registry
class Metrics:
    """Named series + derived reports + sinks.  ``metrics.loss.append(x)`` creates series on first use."""

    def __init__(self, backends: Optional[List[MetricsBackend]] = None, group=None, rank0_only: bool = True):
        object.__setattr__(self, "_series", {})
        object.__setattr__(self, "_reports", {})
        object.__setattr__(self, "_backends", backends or [])
        object.__setattr__(self, "_group", group)
        object.__setattr__(self, "_rank0_only", rank0_only)
        object.__setattr__(self, "_step", 0)

    def __getattr__(self, name: str) -> Series:
        series = object.__getattribute__(self, "_series")
        if name.startswith("_"):
            raise AttributeError(name)
        if name not in series:
            series[name] = Series(name)
        return series[name]

    def add_series(self, name: str, reduce: str = "mean") -> Series:
        self._series[name] = Series(name, reduce)
        return self._series[name]

    def report(self, name: str, series: Series) -> None:
        """Register what ``write()`` emits under ``name`` (the latest value of ``series`` at that time)."""
        self._reports[name] = series

    def step(self) -> None:
        """Advance the metrics step; nothing is communicated here."""
        object.__setattr__(self, "_step", self._step + 1)

    def collect(self) -> Dict[str, float]:
        local = {}
        for name, s in self._reports.items():
            v = s.latest()
            if v is not None:
                local[name] = (v, s.reduce)
        if not local:
            return {}
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self._group) > 1:
            keys = sorted(local)
            dev = "cuda" if dist.get_backend(self._group) == "nccl" else "cpu"
            t_sum = torch.tensor([local[k][0] for k in keys], dtype=torch.float64, device=dev)
            t_max = t_sum.clone()
            dist.all_reduce(t_sum, group=self._group)
            dist.all_reduce(t_max, op=dist.ReduceOp.MAX, group=self._group)
            w = dist.get_world_size(self._group)
            out = {}
            for i, k in enumerate(keys):
                r = local[k][1]
                out[k] = {"mean": t_sum[i].item() / w, "sum": t_sum[i].item(), "max": t_max[i].item(),
                          "none": local[k][0]}[r]
            return out
        return {k: v for k, (v, _) in local.items()}

    def write(self, step: Optional[int] = None) -> Dict[str, float]:
        scalars = self.collect()
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        if scalars and (rank == 0 or not self._rank0_only):
            for b in self._backends:
                b.write(self._step if step is None else step, scalars)
        return scalars

    def close(self) -> None:
        for b in self._backends:
            b.close()


def initialize_metrics(seq_length: int, world_size: int = 1, log_every: int = 1,
                       backends: Optional[List[MetricsBackend]] = None, group=None) -> Metrics:
    """The trainer's standard set (``muse/training/common.py:449-526``): loss, grad_norm, learning_rate,
    seconds_per_step, total_tokens, total_samples, tokens/samples per second per GPU, tokens per day."""
    m = Metrics(backends, group)
    for name, red in (("loss", "mean"), ("grad_norm", "mean"), ("learning_rate", "mean"), ("step_time", "max"),
                      ("tokens", "sum"), ("samples", "sum")):
        m.add_series(name, red)
    m.report("loss", m.loss.avg(log_every))
    m.report("grad_norm", m.grad_norm.last())
    m.report("learning_rate", m.learning_rate.last())
    m.report("seconds_per_step", m.step_time.avg(log_every))
    m.report("total_tokens", m.tokens.cumsum().last())
    m.report("total_samples", m.samples.cumsum().last())
    tps = DerivedSeries("tokens_per_sec_per_gpu", [m.tokens, m.step_time],
                        lambda xs: [math.fsum(xs[0][-log_every:]) / max(math.fsum(xs[1][-log_every:]), 1e-9)], "mean")
    sps = DerivedSeries("samples_per_sec_per_gpu", [m.samples, m.step_time],
                        lambda xs: [math.fsum(xs[0][-log_every:]) / max(math.fsum(xs[1][-log_every:]), 1e-9)], "mean")
    m.report("tokens_per_sec_per_gpu", tps)
    m.report("samples_per_sec_per_gpu", sps)
    m.report("tokens_per_day", DerivedSeries("tokens_per_day", [tps], lambda xs: [x * 86400.0 * world_size for x in xs[0]], "mean"))
    return m


class SourceLossMonitor:
    """Loss per data domain and per data source between two log steps
    (``recipes/pretrain_kai_summary_unified.py:308-324,1029-1040,1091-1120``): every micro-batch adds
    ``loss * valid_tokens`` and ``valid_tokens`` under its domain and its source; at log time the window is summed
    over ranks and reported as ``domain_loss/<d>``, ``domain_tokens/<d>``, ``datasource_loss/<s>``,
    ``datasource_tokens/<s>``.  Losses may be device tensors: they are read back once per window, not per step."""

    def __init__(self):
        self._pending: List[tuple] = []

    @staticmethod
    def _name(value) -> str:
        if isinstance(value, str):
            return value
        if isinstance(value, (list, tuple)) and value:
            uniq = list(dict.fromkeys(value))
            return uniq[0] if len(uniq) == 1 else "mixed"
        return "unknown"

    @staticmethod
    def source_alias(name: str) -> str:
        parts = str(name).rstrip("/").rsplit("/", 2)
        return "/".join(parts[-2:]) if len(parts) >= 2 else (parts[-1] or "unknown")

    def add(self, batch: dict, loss, valid_tokens: int) -> None:
        source = self._name(batch.get("data_source"))
        domain = self._name(batch.get("data_domain")) if batch.get("data_domain") is not None else source
        if valid_tokens > 0:
            self._pending.append((domain, source, loss, int(valid_tokens)))

    def window(self, group=None) -> Dict[str, float]:
        """Scalars of the window since the last call, summed over the ranks of ``group``; clears the window."""
        losses = [p[2] for p in self._pending]
        if losses and any(torch.is_tensor(x) for x in losses):
            vals = torch.stack([x.detach().float().reshape(()) if torch.is_tensor(x) else torch.tensor(float(x))
                                for x in losses]).tolist()
        else:
            vals = [float(x) for x in losses]
        local: Dict[str, List[float]] = {}
        for (domain, source, _, n), v in zip(self._pending, vals):
            for key in (f"domain/{domain}", f"source/{self.source_alias(source)}"):
                acc = local.setdefault(key, [0.0, 0.0])
                acc[0] += v * n
                acc[1] += n
        self._pending = []
        merged = local
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            parts: List[Optional[dict]] = [None] * dist.get_world_size(group)
            dist.all_gather_object(parts, local, group=group)      # keys differ between ranks; once per log step
            merged = {}
            for part in parts:
                for k, (a, b) in (part or {}).items():
                    acc = merged.setdefault(k, [0.0, 0.0])
                    acc[0] += a
                    acc[1] += b
        out: Dict[str, float] = {}
        for k in sorted(merged):
            loss_sum, tokens = merged[k]
            if tokens <= 0:
                continue
            kind, name = k.split("/", 1)
            prefix = "domain" if kind == "domain" else "datasource"
            out[f"{prefix}_loss/{name}"] = loss_sum / tokens
            out[f"{prefix}_tokens/{name}"] = tokens
        return out


class SimpleMetrics:
    """Running means between logs, no series history (``muse/training/simple_metrics.py:14-158``)."""

    def __init__(self):
        self._sum: Dict[str, float] = {}
        self._n: Dict[str, int] = {}
        self._t0 = time.perf_counter()

    def update(self, **values: Number) -> None:
        for k, v in values.items():
            self._sum[k] = self._sum.get(k, 0.0) + _to_float(v)
            self._n[k] = self._n.get(k, 0) + 1

    def summary(self, reset: bool = True) -> Dict[str, float]:
        out = {k: self._sum[k] / max(self._n[k], 1) for k in self._sum}
        out["elapsed"] = time.perf_counter() - self._t0
        if reset:
            self._sum, self._n, self._t0 = {}, {}, time.perf_counter()
        return out
