"""Worker-process data loading in front of the resumable token datasets.

The reference puts a ``DataLoader(batch_size=1, num_workers=1)`` in front of its dataset and shares the sampler state
with the worker through a ``multiprocessing.Manager`` dict (``recipes/pretrain_kai_summary_unified.py:636-642``,
``muse/data/datasets/kai_mmap.py:188-194``); a worker that has prefetched ahead then reports a state that is ahead of
what the trainer has consumed.  Here the state travels WITH every batch: the worker yields ``(batch, state after this
batch)``, and the loader remembers the state of the last batch the trainer actually took, so a checkpoint resumes at
the next unconsumed sample however far the worker had run ahead.
"""
from __future__ import annotations

from typing import Any, Iterator, Optional

import torch
from torch.utils.data import DataLoader, IterableDataset


class _WithState(IterableDataset):
    def __init__(self, dataset):
        self.dataset = dataset
        self.stateful = hasattr(dataset, "state_dict") and getattr(dataset, "supports_dataloader_resume", True)

    def __iter__(self):
        for batch in self.dataset:
            yield batch, (self.dataset.state_dict() if self.stateful else None)


class ResumableLoader:
    """Iterates ``dataset`` in ``num_workers`` worker processes (0: in this process) and keeps its resumable state in
    step with the batches handed out.  With more than one worker every worker strides the stream by its id (the
    datasets read ``torch.utils.data.get_worker_info``); the remembered state is then the one that came with the last
    batch, which is exact for one worker, the reference's setting."""

    def __init__(self, dataset, num_workers: int = 1, prefetch_factor: int = 2):
        self.dataset = dataset
        self.num_workers = int(num_workers)
        self.prefetch_factor = prefetch_factor
        self._state: Optional[Any] = None
        self._it: Optional[Iterator] = None
        for name in ("seq_length",):
            if hasattr(dataset, name):
                setattr(self, name, getattr(dataset, name))

    def __iter__(self):
        kw = dict(batch_size=None, shuffle=False, num_workers=self.num_workers)
        if self.num_workers > 0:
            kw["prefetch_factor"] = self.prefetch_factor
        self._it = iter(DataLoader(_WithState(self.dataset), **kw))
        return self

    def __next__(self):
        if self._it is None:
            iter(self)
        batch, state = next(self._it)
        if state is not None:
            self._state = state
        return batch

    def state_dict(self):
        """State after the last batch that ``__next__`` returned (before the first one: the dataset's own state)."""
        return self._state if self._state is not None else self.dataset.state_dict()

    def load_state_dict(self, state) -> None:
        if self._it is not None:
            raise RuntimeError("load the dataloader state before iteration starts (the workers copy the dataset then)")
        self.dataset.load_state_dict(state)
        self._state = None

    @property
    def supports_dataloader_resume(self) -> bool:
        return hasattr(self.dataset, "state_dict") and getattr(self.dataset, "supports_dataloader_resume", True)
