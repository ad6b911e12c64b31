"""Label-space padding and sharding rule.

Parity: reference main.py:76-97.  ``L`` labels are padded to ``Lp`` so that every one of the
``G`` ranks owns the same number ``Ls`` of classifier rows and ``Ls`` is a multiple of 16
(tensor-core friendly).  Rank ``r`` owns global labels ``[r*Ls, (r+1)*Ls)``; padded labels have
no positives and are clipped to ``L-1`` at prediction time (reference dl_base.py:768-769,782).

The kernels of this package tile labels in blocks of ``LABEL_TILE`` rows; a shard whose ``Ls`` is
not a multiple of the tile is handled by the kernels' bounds checks (TMA zero-fill on loads,
predicated stores), so the on-disk layout keeps the reference's multiple-of-16 rule.
"""
from __future__ import annotations

from dataclasses import dataclass

LABEL_TILE = 128


@dataclass(frozen=True)
class LabelSharding:
    num_labels: int        # L, true label count
    world_size: int        # G
    padded_labels: int     # Lp
    labels_per_rank: int   # Ls

    def shard_range(self, rank: int) -> tuple[int, int]:
        return rank * self.labels_per_rank, (rank + 1) * self.labels_per_rank

    def owner(self, label: int) -> int:
        return label // self.labels_per_rank


def shard_labels(num_labels: int, world_size: int) -> LabelSharding:
    """Pad ``num_labels`` the way the reference does: first to a multiple of ``world_size``,
    then so that the per-rank count is a multiple of 16."""
    if num_labels <= 0 or world_size <= 0:
        raise ValueError("num_labels and world_size must be positive")
    padded = num_labels
    if padded % world_size != 0:
        padded = world_size * ((num_labels + world_size - 1) // world_size)
    per = padded // world_size
    if per % 16 != 0:
        padded = world_size * 16 * ((per + 15) // 16)
        per = padded // world_size
    return LabelSharding(num_labels, world_size, padded, per)


def batch_row_range(global_batch: int, world_size: int, rank: int) -> tuple[int, int]:
    """Rows of the global batch that ``rank`` encodes.  A remainder ``global_batch % G`` is spread
    over the first ranks, one extra row each (reference dl_base.py:348-358, 920-928)."""
    per = global_batch // world_size
    rem = global_batch % world_size
    start = rank * per + min(rank, rem)
    end = start + per + (1 if rank < rem else 0)
    return start, end
