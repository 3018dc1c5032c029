"""Sparse memory fine-tuning (SMFT) bookkeeping of the memory transformer: row-access counts, TF-IDF row
masks, and the conservative projection of a slot mask onto the two half-key tables.

Host-side mirror of `MemoryAccessCounts`, `SmftRowScore`, `SmftRowMask` and
`SmftProductKeyMaskProjection` (src/memory_transformer.rs:103-442, sort order :2045-2055).  Counting runs on
the device (`hl_memory_access_count_rows_i64_u64`); scoring and sorting touch one number per memory slot and
stay on the host, as in the reference.  Error texts follow the reference's.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Sequence

import numpy as np

from ._lib import HeirloomError


def product_key_side(memory_slots: int) -> int:
    side = math.isqrt(int(memory_slots))
    if side * side != memory_slots:
        raise HeirloomError(f"product-key SMFT mask projection requires square memory_slots, got {memory_slots}")
    return side


@dataclass
class SmftRowScore:
    row: int
    foreground_count: int
    background_count: int
    score: float


def sort_smft_scores(scores: List[SmftRowScore]) -> None:
    """Descending score, then descending foreground count, ascending background count, ascending row
    (src/memory_transformer.rs:2045-2055).  NaN scores compare equal to everything there; none arise from
    counts."""
    scores.sort(key=lambda s: (-s.score, -s.foreground_count, s.background_count, s.row))


@dataclass
class MemoryAccessCounts:
    memory_slots: int
    total_events: int
    unique_rows: int
    row_counts: np.ndarray  # uint64 [memory_slots]

    @staticmethod
    def empty(memory_slots: int) -> "MemoryAccessCounts":
        return MemoryAccessCounts(memory_slots, 0, 0, np.zeros(memory_slots, np.uint64))

    @staticmethod
    def from_rows(memory_slots: int, rows: Iterable[int]) -> "MemoryAccessCounts":
        rows = np.asarray(list(rows) if not isinstance(rows, np.ndarray) else rows, np.int64).reshape(-1)
        bad = rows[(rows < 0) | (rows >= memory_slots)]
        if bad.size:
            raise HeirloomError(f"memory access row {int(bad[0])} is out of range for memory_slots {memory_slots}")
        counts = np.bincount(rows, minlength=memory_slots).astype(np.uint64)
        return MemoryAccessCounts(memory_slots, int(rows.size), int(np.count_nonzero(counts)), counts)

    @staticmethod
    def from_row_counts(memory_slots: int, row_counts: Sequence[int]) -> "MemoryAccessCounts":
        counts = np.asarray(row_counts, np.uint64).reshape(-1)
        out = MemoryAccessCounts(memory_slots, int(counts.sum(dtype=np.uint64)), int(np.count_nonzero(counts)), counts)
        out.validate()
        return out

    def validate(self) -> None:
        if len(self.row_counts) != self.memory_slots:
            raise HeirloomError(f"MemoryAccessCounts row_counts length {len(self.row_counts)} does not match "
                                f"memory_slots {self.memory_slots}")
        total = int(np.asarray(self.row_counts, np.uint64).sum(dtype=np.uint64))
        if self.total_events != total:
            raise HeirloomError(f"MemoryAccessCounts total_events {self.total_events} does not match row_counts sum {total}")
        unique = int(np.count_nonzero(self.row_counts))
        if self.unique_rows != unique:
            raise HeirloomError(f"MemoryAccessCounts unique_rows {self.unique_rows} does not match non-zero row count {unique}")

    def merge_in(self, other: "MemoryAccessCounts") -> None:
        self.validate()
        other.validate()
        if self.memory_slots != other.memory_slots:
            raise HeirloomError(f"MemoryAccessCounts merge memory_slots mismatch: {self.memory_slots} vs {other.memory_slots}")
        a = np.asarray(self.row_counts, np.uint64)
        b = np.asarray(other.row_counts, np.uint64)
        merged = a + b
        if np.any(merged < a):
            raise HeirloomError("MemoryAccessCounts merge overflow")
        self.row_counts = merged
        self.total_events = int(merged.sum(dtype=np.uint64))
        self.unique_rows = int(np.count_nonzero(merged))

    def top_rows(self, limit: int) -> List[SmftRowScore]:
        rows = [SmftRowScore(int(r), int(self.row_counts[r]), 0, float(self.row_counts[r]))
                for r in np.flatnonzero(self.row_counts)]
        sort_smft_scores(rows)
        return rows[:limit]

    def smft_mask_against(self, background: "MemoryAccessCounts", trainable_fraction: float, min_rows: int) -> "SmftRowMask":
        """TF-IDF ranking of the rows this count set touched against a background set
        (src/memory_transformer.rs:273-327): tf = fg/total_fg, idf = ln((total_bg + slots)/(bg + 1))."""
        if self.memory_slots != background.memory_slots:
            raise HeirloomError(f"SMFT foreground/background memory_slots mismatch: {self.memory_slots} vs "
                                f"{background.memory_slots}")
        if not (math.isfinite(trainable_fraction) and 0.0 <= trainable_fraction <= 1.0):
            raise HeirloomError(f"SMFT trainable_fraction must be finite in [0, 1], got {trainable_fraction}")
        fg_total = float(max(self.total_events, 1))
        bg_total = float(max(background.total_events, 1))
        slots = float(max(self.memory_slots, 1))
        scores = []
        for r in np.flatnonzero(self.row_counts):
            fg, bg = int(self.row_counts[r]), int(background.row_counts[r])
            tf = float(fg) / fg_total
            idf = math.log((bg_total + slots) / (float(bg) + 1.0))
            scores.append(SmftRowScore(int(r), fg, bg, tf * idf))
        sort_smft_scores(scores)
        requested = int(math.ceil(float(self.unique_rows) * trainable_fraction))
        trainable_count = min(max(requested, min(min_rows, self.unique_rows)), len(scores))
        trainable = [s.row for s in scores[:trainable_count]]
        return SmftRowMask(self.memory_slots, trainable, max(self.memory_slots - trainable_count, 0), trainable_fraction, scores)


@dataclass
class SmftProductKeyMaskProjection:
    side: int
    value_trainable_rows: int
    left_trainable_rows: List[int]
    right_trainable_rows: List[int]
    policy: str = "conservative_all_slots"
    half_key_rows_are_conservative: bool = True

    def _mask(self, rows: Sequence[int]) -> np.ndarray:
        mask = np.zeros(self.side, np.uint8)
        for r in rows:
            if r >= self.side:
                raise HeirloomError(f"product-key SMFT projected row {r} is out of range for side {self.side}")
            mask[r] = 1
        return mask

    def left_mask(self) -> np.ndarray:
        return self._mask(self.left_trainable_rows)

    def right_mask(self) -> np.ndarray:
        return self._mask(self.right_trainable_rows)


@dataclass
class SmftRowMask:
    memory_slots: int
    trainable_rows: List[int]
    frozen_rows: int
    trainable_fraction: float
    scores: List[SmftRowScore] = field(default_factory=list)

    def validate(self) -> None:
        if not (math.isfinite(self.trainable_fraction) and 0.0 <= self.trainable_fraction <= 1.0):
            raise HeirloomError(f"SMFT trainable_fraction must be finite and between 0 and 1, got {self.trainable_fraction}")
        seen = set()
        for row in self.trainable_rows:
            if row < 0 or row >= self.memory_slots:
                raise HeirloomError(f"SMFT trainable row {row} is out of range for memory_slots {self.memory_slots}")
            if row in seen:
                raise HeirloomError(f"SMFT trainable row {row} appears more than once")
            seen.add(row)
        expected = max(self.memory_slots - len(self.trainable_rows), 0)
        if self.frozen_rows != expected:
            raise HeirloomError(f"SMFT frozen_rows {self.frozen_rows} does not match memory_slots {self.memory_slots} "
                                f"minus trainable rows {len(self.trainable_rows)}")

    def to_mask(self) -> np.ndarray:
        """Byte per memory slot, 1 = trainable (`SmftRowMask::to_tensor`, src/memory_transformer.rs:404-417)."""
        self.validate()
        mask = np.zeros(self.memory_slots, np.uint8)
        mask[np.asarray(self.trainable_rows, np.int64)] = 1
        return mask

    def product_key_projection(self) -> SmftProductKeyMaskProjection:
        """A half-key row is trainable only when every slot it takes part in is trainable
        (src/memory_transformer.rs:366-402)."""
        self.validate()
        side = product_key_side(self.memory_slots)
        grid = self.to_mask().reshape(side, side).astype(bool)
        left = [int(i) for i in np.flatnonzero(grid.all(axis=1))]
        right = [int(i) for i in np.flatnonzero(grid.all(axis=0))]
        return SmftProductKeyMaskProjection(side, len(self.trainable_rows), left, right)


@dataclass
class SmftAccessReport:
    counts: MemoryAccessCounts
    top_rows: List[SmftRowScore]
