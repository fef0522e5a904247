"""Host-side statement of the expert-parallel row layout.

The device computes this layout itself every forward (``ep_exchange_kernel`` in
``csrc/ep.cu``); this module states the same rules in numpy so a host can size
``recv_rows_max`` and so the rules can be tested without a GPU.

Rank q owns experts ``[q*e_local, (q+1)*e_local)``.  In q's dispatch buffer the
rows of local expert ``le`` start at a multiple of ``ROW_ALIGN`` and hold the
picks of source rank 0 first, then rank 1, ...; inside one source the picks keep
the order of their flat index ``t*k+j``.
"""
from __future__ import annotations

import numpy as np

ROW_ALIGN = 128


def round_up(a, b):
    return (a + b - 1) // b * b


def owner_layout(counts_all: np.ndarray, q: int, e_local: int):
    """Layout of owner q's buffer. ``counts_all[s, e]`` = picks of expert e on source rank s.
    Returns (ex_counts[e_local], ex_poffsets[e_local+1])."""
    tot = counts_all[:, q * e_local:(q + 1) * e_local].sum(0)
    poff = np.zeros(e_local + 1, np.int64)
    poff[1:] = np.cumsum(round_up(tot, ROW_ALIGN))
    return tot.astype(np.int32), poff.astype(np.int32)


REFUSED_BASE = -(1 << 30)  # dst_base of every expert in a refused step: every row position becomes negative


def rows_capacity(rows_in: int, e_local: int) -> int:
    """Row capacity of a rank's dispatch buffer: ``rows_in`` is ``recv_rows_max`` of the handle's configuration
    (default ``t_max * top_k * world``); every local expert's segment may need rounding up to ROW_ALIGN."""
    return (round_up(rows_in, ROW_ALIGN) // ROW_ALIGN + e_local) * ROW_ALIGN


def step_refused(counts_all: np.ndarray, e_local: int, rows_cap: int) -> bool:
    """A step is refused when the padded rows of ANY owner exceed the capacity.  Every rank evaluates this on the
    same count matrix, so all of them refuse together; a refused step moves no row (dispatch, combine and the
    backward kernels skip picks whose position is negative) and raises the bounds bit of the device error word."""
    return rows_needed(counts_all, e_local) > rows_cap


def dst_base(counts_all: np.ndarray, r: int, e_local: int, rows_cap: int | None = None) -> np.ndarray:
    """First row, in the owner's buffer, of source rank r's picks of every expert (REFUSED_BASE everywhere when
    ``rows_cap`` is given and the step does not fit it)."""
    W, E = counts_all.shape
    out = np.zeros(E, np.int32)
    if rows_cap is not None and step_refused(counts_all, e_local, rows_cap):
        out[:] = REFUSED_BASE
        return out
    for q in range(W):
        _, poff = owner_layout(counts_all, q, e_local)
        for le in range(e_local):
            e = q * e_local + le
            out[e] = poff[le] + counts_all[:r, e].sum()
    return out


def rows_needed(counts_all: np.ndarray, e_local: int) -> int:
    """Largest padded row count any owner receives (compare with the handle's capacity)."""
    W = counts_all.shape[0]
    return int(max(owner_layout(counts_all, q, e_local)[1][-1] for q in range(W)))


def shard_tokens(T: int, world: int, rank: int):
    """Token slice of one rank when a global batch of T tokens is split evenly (the remainder goes to the last ranks' predecessors)."""
    base, rem = divmod(T, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)
