"""Expert-parallel partitioning helpers (host logic shared by bench.py and the tests).

Experts are split into contiguous equal ranges, one per rank; the router is replicated, so every rank knows every
token's experts and computes only the (token, rank) rows of the experts it owns.  Summing the per-rank row buffers
(zeros for rows owned elsewhere) reproduces the one-GPU buffer bit for bit: each row has exactly one non-zero
contributor."""
from __future__ import annotations

import numpy as np


def expert_range(E: int, rank: int, size: int) -> tuple[int, int]:
    if size < 1 or E % size or not (0 <= rank < size):
        raise ValueError("experts (%d) must divide evenly over %d ranks" % (E, size))
    per = E // size
    return rank * per, (rank + 1) * per


def owner_of(E: int, size: int, expert_ids: np.ndarray) -> np.ndarray:
    return np.asarray(expert_ids) // (E // size)


def scaling_bound(step_bytes_total: float, moe_bytes: float, n: int) -> float:
    """Upper bound on the speed-up from sharding only the expert weights over n GPUs (HBM bytes per GPU)."""
    return step_bytes_total / (step_bytes_total - moe_bytes + moe_bytes / n)
