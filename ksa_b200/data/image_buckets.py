"""Aspect-ratio and resolution buckets for image samples of the parquet pipeline.

The reference carries these helpers next to its (vestigial) parquet datasets (``muse/data/utils.py:90-252``): an image
is assigned to a resolution level by the geometric mean of its sides, then to the bucket of that level whose aspect
ratio is closest, so that a batch holds images of one shape; a "resolution budget" gives the batch size per level.
The text pre-training recipe does not use them.  Here the bucket table of a level is generated instead of listed: all
shapes whose sides are multiples of ``size / 16``, whose aspect ratio lies in ``[1/4, 4]`` and whose area is the
largest that does not exceed ``size * size`` for their height (landscape shapes mirror the portrait ones).
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import Dict, List, Optional, Sequence, Tuple

RESOLUTION_LEVELS: Tuple[int, ...] = (256, 512, 768, 1024, 1536, 2048)


def _ratio_key(h: int, w: int) -> str:
    """``h / w`` with two decimals, trailing zeros dropped but one kept ("0.25", "1.0", "4.0")."""
    text = f"{h / w:.2f}"
    return text[:-1] if text.endswith("0") else text


@lru_cache(maxsize=None)
def aspect_ratio_buckets(image_size: int) -> Dict[str, Tuple[int, int]]:
    """``{"h/w rounded to 2 digits": (height, width)}`` for images of about ``image_size ** 2`` pixels.

    Sizes between two levels use the next level up; sizes above the largest level scale its table."""
    level = next((r for r in RESOLUTION_LEVELS if image_size <= r), None)
    if level is None:
        scale = image_size / RESOLUTION_LEVELS[-1]
        return {k: (int(h * scale), int(w * scale)) for k, (h, w) in aspect_ratio_buckets(RESOLUTION_LEVELS[-1]).items()}
    step, area = level // 16, level * level
    out: Dict[str, Tuple[int, int]] = {}
    h = level // 2
    while h <= level:                                   # portrait half, the square included: h <= w
        w = min(area // h // step * step, 4 * h)
        if w >= h:
            out.setdefault(_ratio_key(h, w), (h, w))
        h += step
    for k, (ph, pw) in list(out.items()):               # landscape half
        if ph != pw:
            out.setdefault(_ratio_key(pw, ph), (pw, ph))
    return dict(sorted(out.items(), key=lambda kv: float(kv[0])))


def closest_ratio(height: int, width: int, buckets: Dict[str, Tuple[int, int]]) -> str:
    """Key of the bucket whose aspect ratio (height / width) is nearest to the image's."""
    ratio = height / width
    return min(buckets, key=lambda k: abs(float(k) - ratio))


def closest_size(height: int, width: int, buckets: Dict[str, Tuple[int, int]]) -> Tuple[int, int]:
    """``(height, width)`` of the bucket an image of this shape is resized to."""
    return buckets[closest_ratio(height, width, buckets)]


def resolution_level(height: int, width: int, levels: Optional[Sequence[int]] = None) -> int:
    """Largest level that does not exceed ``sqrt(height * width)`` (no upsampling); the smallest level for images
    below all of them."""
    levels = list(levels) if levels is not None else list(RESOLUTION_LEVELS)
    effective = (height * width) ** 0.5
    fitting = [r for r in levels if r <= effective]
    return max(fitting) if fitting else min(levels)


@dataclass
class ResolutionBudget:
    size: int          # resolution level
    batch_size: int    # images of that level per batch


@dataclass
class ResolutionBudgetConfig:
    """Levels in use and their batch sizes; samples are buffered per (level, aspect-ratio bucket) until a batch is full."""
    budgets: List[ResolutionBudget]

    def batch_size(self, size: int) -> int:
        for b in self.budgets:
            if b.size == size:
                return b.batch_size
        raise KeyError(f"no budget for resolution {size}")

    @property
    def levels(self) -> List[int]:
        return [b.size for b in self.budgets]


DEFAULT_RESOLUTION_BUDGETS = ResolutionBudgetConfig([ResolutionBudget(512, 32), ResolutionBudget(768, 16),
                                                     ResolutionBudget(1024, 8)])


def parse_resolution_budgets(text: str) -> ResolutionBudgetConfig:
    """``"512:32,768:16,1024:8"`` (level:batch size) -> ``ResolutionBudgetConfig``."""
    budgets = []
    for entry in text.split(","):
        entry = entry.strip()
        if not entry:
            continue
        size, _, batch = entry.partition(":")
        if not batch:
            raise ValueError(f"resolution budget {entry!r} is not of the form size:batch_size")
        budgets.append(ResolutionBudget(int(size), int(batch)))
    if not budgets:
        raise ValueError("no resolution budgets given")
    return ResolutionBudgetConfig(budgets)


class BucketBatcher:
    """Groups samples by (resolution level, aspect-ratio bucket) and releases a group when it has reached the batch
    size of its level (what the reference's multi-scale image loader does with the helpers above)."""

    def __init__(self, config: ResolutionBudgetConfig = DEFAULT_RESOLUTION_BUDGETS):
        self.config = config
        self._pending: Dict[Tuple[int, str], list] = {}

    def add(self, sample, height: int, width: int):
        """Returns ``(level, (h, w), samples)`` when a batch is complete, else ``None``."""
        level = resolution_level(height, width, self.config.levels)
        buckets = aspect_ratio_buckets(level)
        key = closest_ratio(height, width, buckets)
        group = self._pending.setdefault((level, key), [])
        group.append(sample)
        if len(group) >= self.config.batch_size(level):
            del self._pending[(level, key)]
            return level, buckets[key], group
        return None

    def flush(self):
        """Incomplete groups, for the end of an epoch."""
        out = [(level, aspect_ratio_buckets(level)[key], group) for (level, key), group in self._pending.items()]
        self._pending = {}
        return out
