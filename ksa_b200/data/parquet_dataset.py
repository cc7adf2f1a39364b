"""Parquet sample pipeline (``muse/data/datasets/base.py:118-316,316-619``): ordered and window-shuffled readers,
sharding of files or samples over data-parallel ranks and loader workers, a ``process`` hook and token packing.

The pre-training recipe reads mmap token corpora only (as the reference's does); this pipeline serves tokenised or
raw-text parquet shards, e.g. for fine-tuning data.  Unlike the reference's, iteration order is a pure function of
``(seed, epoch, rank, worker)`` and the position is resumable: ``state_dict()`` records the epoch and how many
samples this shard has produced, and ``load_state_dict`` fast-forwards without touching the skipped rows' payload.
"""
from __future__ import annotations

import glob
import os
import random
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Union

import torch
from torch.utils.data import IterableDataset, get_worker_info


def _worker() -> tuple:
    info = get_worker_info()
    return (0, 1) if info is None else (info.id, info.num_workers)


def expand_sources(sources: Union[str, Sequence[str]]) -> List[str]:
    """Files, directories (every ``*.parquet`` inside) and glob patterns -> sorted file list."""
    if isinstance(sources, str):
        sources = [sources]
    out: List[str] = []
    for s in sources:
        if os.path.isdir(s):
            out += sorted(glob.glob(os.path.join(s, "**", "*.parquet"), recursive=True))
        elif any(ch in s for ch in "*?["):
            out += sorted(glob.glob(s))
        else:
            out.append(s)
    return out


class ParquetReader:
    """Rows of the files in order, each tagged with ``__file__``, ``__index__``, ``__total__``.  Unreadable files are
    reported and skipped, as the reference does."""

    def __init__(self, sources: Union[str, Sequence[str]], columns: Optional[List[str]] = None):
        self.sources = expand_sources(sources)
        self.columns = columns

    def _rows(self, fn: str) -> Iterator[Dict[str, Any]]:
        import pyarrow.parquet as pq
        try:
            pf = pq.ParquetFile(fn)
        except Exception as e:  # noqa: BLE001
            print(f"[parquet] cannot open {fn}: {type(e).__name__}: {e}")
            return
        total, idx = pf.metadata.num_rows, 0
        for batch in pf.iter_batches(batch_size=1024, columns=self.columns):
            for row in batch.to_pylist():
                row["__file__"], row["__index__"], row["__total__"] = fn, idx, total
                idx += 1
                yield row

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        for fn in self.sources:
            yield from self._rows(fn)


def window_shuffle(rows: Iterator[Dict[str, Any]], buffer_size: int, seed: int) -> Iterator[Dict[str, Any]]:
    """Keep ``buffer_size`` rows; for every further row read, a random buffered row leaves."""
    rng = random.Random(seed)
    buf: List[Dict[str, Any]] = []
    for row in rows:
        if len(buf) < buffer_size:
            buf.append(row)
            continue
        j = rng.randrange(len(buf))
        buf[j], row = row, buf[j]
        yield row
    rng.shuffle(buf)
    yield from buf


class ShuffledParquetReader(ParquetReader):
    """Window shuffle: a buffer of ``buffer_size`` rows is kept and a random element leaves for every row read."""

    def __init__(self, sources, columns=None, buffer_size: int = 16384, seed: int = 0):
        super().__init__(sources, columns)
        self.buffer_size, self.seed = buffer_size, seed

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        return window_shuffle(super().__iter__(), self.buffer_size, self.seed)


class DistributedParquetDataset(IterableDataset):
    """Parquet samples sharded over data-parallel ranks and loader workers.

    ``shard_by="file"`` gives every (rank, worker) its own files (needs at least as many files as shards);
    ``"sample"`` lets everyone read every file and keep rows ``i % shards == shard``.  ``process`` maps a row to the
    training sample (tokenise, build masks); returning ``None`` drops the row.  With ``pack_to`` token rows
    (``input_ids`` lists) are concatenated and cut into fixed-length samples with ``cu_seqlens`` document bounds.
    """

    def __init__(self, sources, rank: int = 0, world_size: int = 1, shard_by: str = "file", shuffle: bool = True,
                 shuffle_buffer_size: int = 16384, seed: int = 0, num_epochs: int = 1, columns: Optional[List[str]] = None,
                 process: Optional[Callable[[Dict[str, Any]], Optional[Dict[str, Any]]]] = None,
                 pack_to: Optional[int] = None):
        if shard_by not in ("file", "sample"):
            raise ValueError("shard_by must be 'file' or 'sample'")
        self.files = expand_sources(sources)
        if not self.files:
            raise FileNotFoundError(f"no parquet files under {sources}")
        self.rank, self.world_size, self.shard_by = rank, world_size, shard_by
        self.shuffle, self.buffer, self.seed, self.num_epochs = shuffle, shuffle_buffer_size, seed, num_epochs
        self.columns, self.process, self.pack_to = columns, process, pack_to
        self.epoch, self.produced = 0, 0
        self._skip = 0

    # ------------------------------------------------------------------ resume
    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "produced": self.produced, "seed": self.seed}

    def load_state_dict(self, state: Dict[str, int]) -> None:
        self.epoch, self._skip = int(state["epoch"]), int(state["produced"])
        self.produced = 0

    # ------------------------------------------------------------------ iteration
    def _epoch_rows(self, epoch: int) -> Iterator[Dict[str, Any]]:
        wid, nw = _worker()
        shard, shards = self.rank * nw + wid, self.world_size * nw
        files = list(self.files)
        if self.shuffle:
            random.Random(self.seed * 1000003 + epoch).shuffle(files)
        if self.shard_by == "file":
            if len(files) < shards:
                raise ValueError(f"{len(files)} files cannot be split over {shards} shards; use shard_by='sample'")
            files = files[shard::shards]
        rows: Iterator[Dict[str, Any]] = iter(ParquetReader(files, self.columns))
        if self.shard_by == "sample":      # the same file order everywhere, so the modulo partitions the rows
            rows = (row for i, row in enumerate(rows) if i % shards == shard)
        if self.shuffle:
            rows = window_shuffle(rows, self.buffer, self.seed * 7919 + epoch * 31 + shard)
        return rows

    def _samples(self, epoch: int) -> Iterator[Dict[str, Any]]:
        pending: List[int] = []
        bounds: List[int] = [0]
        for row in self._epoch_rows(epoch):
            sample = self.process(row) if self.process is not None else row
            if sample is None:
                continue
            if self.pack_to is None:
                yield sample
                continue
            ids = list(sample["input_ids"])
            while ids:
                take = min(self.pack_to - len(pending), len(ids))
                pending += ids[:take]
                ids = ids[take:]
                bounds.append(len(pending))
                if len(pending) == self.pack_to:
                    yield {"input_ids": torch.tensor(pending, dtype=torch.long)[None],
                           "cu_seqlens": torch.tensor(bounds, dtype=torch.int32)}
                    pending, bounds = [], [0]

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        while self.epoch < self.num_epochs:
            for sample in self._samples(self.epoch):
                if self._skip > 0:
                    self._skip -= 1
                    self.produced += 1
                    continue
                self.produced += 1
                yield sample
            self.epoch += 1
            self.produced = 0
