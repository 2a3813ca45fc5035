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


def row_order(sids, nranks: int, rank: int):
    """Device row order under slot sharding (slot s belongs to rank s mod nranks), through the C ABI (host logic, no device):
    returns (perm, lo, hi) -- perm[j] = caller's index of device row j, [lo, hi) = this rank's rows."""
    import ctypes as C
    from . import lib
    L = lib.load()
    s = np.ascontiguousarray(sids, np.int32)
    perm = np.empty(len(s), np.int32)
    lo, hi = C.c_int(), C.c_int()
    L.qw_ep_row_order.restype = C.c_int
    L.qw_ep_row_order.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    if L.qw_ep_row_order(s.ctypes.data, len(s), nranks, rank, perm.ctypes.data, C.addressof(lo), C.addressof(hi)) != 0:
        raise ValueError("bad rank / nranks")
    return perm, lo.value, hi.value
