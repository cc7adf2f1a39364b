"""Memory-mapped token corpora, weighted blending with resumable state, and the trainer's batch adapter.

File formats and batch contract follow the reference (``muse/data/datasets/kai_mmap.py:44-147,167-281,436-618``):

* a corpus is ``<prefix>.bin`` (flat token ids) + ``<prefix>.bin.meta`` (numpy dtype name, e.g. ``uint32``) and an
  optional ``<prefix>_loss_mask.bin`` (QA corpora); sample ``i`` is tokens ``[i*L, i*L + L + 1)``;
* a mixture is a recipe file with ``weight path`` or ``domain weight path`` per line;
* every global batch draws ``global_batch_size`` source names with the mixture weights from a private, seeded
  RNG; each source hands out its samples in order and wraps around at the end of an epoch; rank/worker ``k``
  takes positions ``k, k+stride, ...`` of the draw;
* ``state_dict`` holds per-source cursors, epochs, consumed tokens and the RNG state; cursors are rescaled when
  the sequence length changes between stages (8k -> 32k -> ...); a draw that was handed out only in part is part of
  the state, so a resume continues with exactly the next sample;
* batches are ``{"input_ids" [1,L], "loss_mask" [1,L], "position_ids" [1,L], "cu_seqlens" [0,L], "data_source",
  "data_domain"}``.

Differences by intent: the RNG is a private ``numpy.random.Generator`` (the reference reseeds and saves the global
numpy state), and cursor state lives in the object (no ``multiprocessing.Manager`` dictionaries), so a dataset can be
iterated in-process or inside one DataLoader worker with identical results.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch


def data_file_path(prefix: str) -> str:
    return prefix + ".bin"


def meta_file_path(prefix: str) -> str:
    return prefix + ".bin.meta"


def loss_mask_file_path(prefix: str) -> str:
    return prefix + "_loss_mask.bin"


def write_corpus(prefix: str, tokens: np.ndarray, dtype: str = "uint32", loss_mask: Optional[np.ndarray] = None) -> None:
    """Write a corpus in the on-disk format (used by tests, the synthetic-data tool and the baseline harness)."""
    os.makedirs(os.path.dirname(os.path.abspath(prefix)), exist_ok=True)
    np.asarray(tokens, dtype=getattr(np, dtype)).tofile(data_file_path(prefix))
    with open(meta_file_path(prefix), "w") as f:
        f.write(dtype)
    if loss_mask is not None:
        np.asarray(loss_mask, dtype=getattr(np, dtype)).tofile(loss_mask_file_path(prefix))


class MMapDataset(torch.utils.data.Dataset):
    """One pre-tokenised corpus; ``self[i]`` is ``{"text": int64[L+1]}`` (or tokens||loss_mask, ``2L``, for QA)."""

    def __init__(self, path: str, chunk_size: int):
        with open(meta_file_path(path)) as r:
            self._dtype = np.dtype(getattr(np, r.read().strip()))
        self._path = self.name = path
        self._chunk_size = int(chunk_size)
        self._total_bytes = os.path.getsize(data_file_path(path))
        if self._total_bytes % self._dtype.itemsize:
            raise ValueError(f"{data_file_path(path)}: size is not a multiple of {self._dtype.itemsize} bytes")
        self._open()

    def _open(self) -> None:
        self._tokens = np.memmap(data_file_path(self._path), dtype=self._dtype, mode="r")
        self._mask = (np.memmap(loss_mask_file_path(self._path), dtype=self._dtype, mode="r")
                      if self.is_qa_dataset else None)

    def __getstate__(self):
        return {"path": self._path, "chunk_size": self._chunk_size}

    def __setstate__(self, state):
        self.__init__(state["path"], state["chunk_size"])

    @property
    def is_qa_dataset(self) -> bool:
        return os.path.exists(loss_mask_file_path(self._path))

    @property
    def size(self) -> int:
        return self._total_bytes // self._dtype.itemsize

    @property
    def num_sample(self) -> int:
        # a sample needs L+1 tokens (input + shifted target) unless the corpus carries its own loss mask
        if self.is_qa_dataset:
            return self.size // self._chunk_size
        return max(0, (self.size - 1) // self._chunk_size)

    def __len__(self) -> int:
        return self.num_sample

    def __getitem__(self, i: int) -> Dict[str, np.ndarray]:
        L = self._chunk_size
        if self.is_qa_dataset:
            return {"text": np.concatenate([self._tokens[i * L:(i + 1) * L], self._mask[i * L:(i + 1) * L]]).astype(np.int64)}
        return {"text": np.asarray(self._tokens[i * L:i * L + L + 1], dtype=np.int64)}

    @staticmethod
    def exists(path: str) -> bool:
        return os.path.exists(meta_file_path(path)) and os.path.exists(data_file_path(path))


def parse_data_prefix(data_prefix) -> Tuple[List[str], Optional[Dict[str, str]]]:
    """A prefix, a recipe file (2 or 3 columns) or a flat ``[w1, p1, w2, p2, ...]`` list -> (flat list, {path: domain})."""
    if isinstance(data_prefix, str):
        if os.path.isfile(data_prefix) and not data_prefix.endswith((".bin", ".meta")):
            flat: List[str] = []
            domains: Dict[str, str] = {}
            base = os.path.dirname(os.path.abspath(data_prefix))
            with open(data_prefix) as f:
                for line in f:
                    line = line.strip()
                    if not line or line[0] in "#\"" or "=" in line:
                        continue
                    parts = line.split(None, 2)
                    if len(parts) == 3:
                        try:
                            w = float(parts[1])
                        except ValueError:
                            w = None
                        if w is not None:
                            if w > 0:
                                flat += [parts[1], parts[2].strip()]
                                domains[parts[2].strip()] = parts[0]
                            continue
                    parts = line.split(None, 1)
                    if len(parts) == 2:
                        try:
                            w = float(parts[0])
                        except ValueError:
                            continue
                        if w > 0:
                            flat += [parts[0], parts[1].strip()]
            if not flat:
                raise ValueError(f"recipe file {data_prefix} holds no weight/path pairs")
            # paths in a recipe may be relative to the working directory (reference behaviour) or to the recipe file
            for i in range(1, len(flat), 2):
                if not MMapDataset.exists(flat[i]):
                    for cand in (os.path.join(base, flat[i]), os.path.join(os.path.dirname(base), flat[i])):
                        if MMapDataset.exists(cand):
                            if flat[i] in domains:
                                domains[cand] = domains.pop(flat[i])
                            flat[i] = cand
                            break
            return flat, domains or None
        return [data_prefix], None
    return list(data_prefix), None


def get_datasets_weights(flat: Sequence[str]) -> Tuple[List[str], List[float]]:
    if len(flat) == 1:
        return [flat[0]], [1.0]
    if len(flat) % 2:
        raise ValueError("expected weight/prefix pairs")
    weights = [float(w) for w in flat[0::2]]
    total = sum(weights)
    return [p.strip() for p in flat[1::2]], [w / total for w in weights]


class BlendableWeightedSamplingDataset(torch.utils.data.IterableDataset):
    """Weighted sampling over corpora with per-source cursors, epoch wrap, rank/worker striding and resumable state."""

    def __init__(self, datasets: Sequence[MMapDataset], weights: Sequence[float], *, seed: int, global_batch_size: int,
                 num_workers: int = 1, dp_rank: int = 0, dp_world_size: int = 1):
        if len(datasets) != len(weights):
            raise ValueError("one weight per dataset")
        self._datasets = OrderedDict((d.name, d) for d in datasets)
        w = np.asarray(weights, dtype=np.float64)
        if w.sum() <= 0:
            raise ValueError("mixture weights must sum to a positive number")
        self.weights = w / w.sum()
        self.seed = seed
        self.global_bs = int(global_batch_size)
        self._num_workers = max(1, int(num_workers))
        self._dp_rank, self._dp_world_size = dp_rank, dp_world_size
        if self.global_bs % (self._num_workers * self._dp_world_size):
            raise ValueError("global_batch_size must be a multiple of num_workers * dp_world_size")
        self._rng = np.random.default_rng(seed)
        self.consume_sample = {n: 0 for n in self._datasets}
        self.consume_token = {n: 0 for n in self._datasets}
        self.past_epoch = {n: 0 for n in self._datasets}
        self._pending = None   # (names, indices, samples handed out) of a draw that has been handed out only in part

    @property
    def size(self) -> int:
        return sum(d.size for d in self._datasets.values())

    def state_dict(self) -> dict:
        out = OrderedDict()
        for name, d in self._datasets.items():
            out[name] = {"past_epoch": self.past_epoch[name], "c_sample": self.consume_sample[name],
                         "c_token": self.consume_token[name], "num_tokens": d.size}
        out["rng_state"] = self._rng.bit_generator.state
        out["pending_draw"] = self._pending
        return out

    def load_state_dict(self, state: dict, old_seq_length: Optional[int] = None, seq_length: Optional[int] = None) -> None:
        if "rng_state" in state:
            self._rng.bit_generator.state = state["rng_state"]
        same_length = not (old_seq_length and seq_length and old_seq_length != seq_length)
        self._pending = state.get("pending_draw") if same_length else None
        for name in self._datasets:
            if name not in state:
                continue  # a corpus added since the checkpoint starts from zero
            c = state[name]["c_sample"]
            if old_seq_length and seq_length and old_seq_length != seq_length:
                c = (c * old_seq_length + seq_length - 1) // seq_length
            self.consume_sample[name] = int(c)
            self.consume_token[name] = int(state[name]["c_token"])
            self.past_epoch[name] = int(state[name]["past_epoch"])

    def _draw(self) -> Tuple[List[str], List[int]]:
        names = list(self._datasets)
        picks = self._rng.choice(len(names), size=self.global_bs, p=self.weights)
        chosen, index = [], []
        for k in picks:
            n = names[int(k)]
            d = self._datasets[n]
            if self.consume_sample[n] >= d.num_sample:
                self.consume_sample[n] = 0
                self.past_epoch[n] += 1
            index.append(self.consume_sample[n])
            self.consume_sample[n] += 1
            self.consume_token[n] += d._chunk_size
            chosen.append(n)
        return chosen, index

    def __iter__(self) -> Iterator[Tuple[dict, str]]:
        info = torch.utils.data.get_worker_info()
        worker = 0 if info is None else info.id
        stride = self._num_workers * self._dp_world_size
        first = self._dp_rank + worker * self._dp_world_size
        per_reader = self.global_bs // stride          # samples of one draw that this (rank, worker) hands out
        while True:
            # `_pending` counts samples already handed out of the current draw, not a position: the saved state is
            # written by one rank and read by all, and every reader re-adds its own first position.
            if self._pending is not None:
                names, index, done = self._pending
            else:
                names, index = self._draw()
                done = 0
            for k in range(done, per_reader):
                pos = first + k * stride
                self._pending = (names, index, k + 1) if k + 1 < per_reader else None
                yield self._datasets[names[pos]][index[pos]], names[pos]
            self._pending = None


class KaiMMapDataset(torch.utils.data.IterableDataset):
    """Adapter producing the trainer's batch dicts from a corpus or a weighted mixture."""

    def __init__(self, data_prefix, seq_length: int, seed: int = 1024, rank: int = 0, world_size: int = 1,
                 num_workers: int = 1, global_batch_size: int = 1, skip_warmup: bool = True, **_unused):
        flat, self._domain_map = parse_data_prefix(data_prefix)
        paths, weights = get_datasets_weights(flat)
        missing = [p for p in paths if not MMapDataset.exists(p)]
        if missing:
            raise FileNotFoundError(f"corpus files missing (.bin / .bin.meta): {missing}")
        corpora = [MMapDataset(p, seq_length) for p in paths]
        self.seq_length = int(seq_length)
        self.loader_workers = max(0, int(num_workers))     # worker processes a trainer puts in front of this dataset
        if len(corpora) == 1 and len(flat) == 1:
            self.dataset = corpora[0]
            self._rank, self._world = rank, world_size
        else:
            self.dataset = BlendableWeightedSamplingDataset(
                corpora, weights, seed=seed, global_batch_size=global_batch_size, num_workers=num_workers,
                dp_rank=rank, dp_world_size=world_size)

    @property
    def supports_dataloader_resume(self) -> bool:
        return isinstance(self.dataset, BlendableWeightedSamplingDataset)

    def state_dict(self) -> dict:
        if not self.supports_dataloader_resume:
            raise RuntimeError("dataloader resume needs a blended (recipe-file) dataset")
        return {"state_type": "kai_mmap", "seq_length": self.seq_length, "dataset_state": self.dataset.state_dict()}

    def load_state_dict(self, state: dict) -> None:
        if not self.supports_dataloader_resume:
            raise RuntimeError("dataloader resume needs a blended (recipe-file) dataset")
        if isinstance(state, dict) and state.get("state_type") == "kai_mmap":
            self.dataset.load_state_dict(state["dataset_state"], old_seq_length=state.get("seq_length"),
                                         seq_length=self.seq_length)
        else:
            self.dataset.load_state_dict(state, seq_length=self.seq_length)

    def __iter__(self):
        if isinstance(self.dataset, BlendableWeightedSamplingDataset):
            for sample, source in self.dataset:
                yield self._to_batch(sample, source)
        else:
            while True:
                for i in range(self._rank, self.dataset.num_sample, self._world):
                    yield self._to_batch(self.dataset[i], self.dataset.name)

    def _to_batch(self, sample: dict, source: str) -> dict:
        text = torch.from_numpy(np.ascontiguousarray(sample["text"])).long()
        L = self.seq_length
        if text.shape[0] == 2 * L:
            ids, mask = text[:L], text[L:]
            nxt = None
        else:
            ids, mask = text[:L], torch.ones(L, dtype=torch.long)
            nxt = text[L] if text.shape[0] > L else None
        batch = {"input_ids": ids.unsqueeze(0), "loss_mask": mask.unsqueeze(0),
                 "position_ids": torch.arange(L, dtype=torch.int32).unsqueeze(0),
                 "cu_seqlens": torch.tensor([0, L], dtype=torch.int32), "data_source": [source]}
        if nxt is not None:
            batch["next_token"] = nxt.reshape(1)
        if self._domain_map and source in self._domain_map:
            batch["data_domain"] = [self._domain_map[source]]
        return batch


class SyntheticTokenDataset(torch.utils.data.IterableDataset):
    """Uniform-random token ids of a fixed shape (the benchmark inputs); deterministic per (seed, rank)."""

    def __init__(self, vocab_size: int, seq_length: int, seed: int = 0, rank: int = 0, batch_size: int = 1):
        self.vocab_size, self.seq_length, self.batch_size = vocab_size, seq_length, batch_size
        self._gen = torch.Generator().manual_seed(seed * 1000003 + rank)

    def __iter__(self):
        L = self.seq_length
        while True:
            ids = torch.randint(0, self.vocab_size, (self.batch_size, L), generator=self._gen)
            yield {"input_ids": ids, "loss_mask": torch.ones_like(ids),
                   "position_ids": torch.arange(L, dtype=torch.int32).unsqueeze(0).expand(self.batch_size, -1),
                   "cu_seqlens": torch.tensor([0, L], dtype=torch.int32), "data_source": ["synthetic"]}


def make_labels(input_ids: torch.Tensor, loss_mask: torch.Tensor, ignore_index: int = -100) -> Tuple[torch.Tensor, torch.Tensor]:
    """Shifted labels from the original ids and mask: label[t] = id[t+1], ``ignore_index`` where masked; the last
    position has no target (``recipes/pretrain_kai_summary_unified.py:867-873``)."""
    ids = torch.nn.functional.pad(input_ids[:, 1:], (0, 1), value=0)
    m = torch.nn.functional.pad(loss_mask[:, 1:], (0, 1), value=0)
    return ids * m + ignore_index * (1 - m), m.contiguous()
