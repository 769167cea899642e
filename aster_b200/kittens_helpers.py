"""Helpers shared by the GEMM generators of the reference, restated for this package:
the direct-B weight preshuffle, the pipeline-strategy table and the cooperative-load split
(contrib/kittens/test/kittens_helpers.py:90-169, contrib/kittens/test/coop.py:12-27).
"""

from __future__ import annotations

import math

import numpy as np

# Stage of each pipelined operation per strategy.  Columns, in order:
_STAGE_KEYS = ("A_LOAD", "A_LDS_WRITE", "A_LDS_READ", "B_LOAD", "B_LDS_WRITE", "B_LDS_READ", "COMPUTE")
_STAGE_ROWS = {
    0: (0, 0, 0, 0, 0, 0, 0),
    1: (0, 1, 1, 1, 1, 1, 1),
    2: (0, 0, 1, 0, 1, 1, 1),
    3: (0, 1, 2, 0, 1, 2, 2),
    4: (0, 2, 2, 0, 1, 2, 2),
    5: (0, 1, 2, 2, 2, 2, 3),
    6: (0, 2, 2, 1, 1, 2, 3),
    7: (0, 2, 3, 0, 2, 3, 4),
    8: (0, 1, 3, 0, 2, 3, 4),
    9: (0, 3, 4, 0, 3, 4, 5),
    10: (0, 2, 4, 0, 3, 4, 5),
    11: (0, 1, 3, 0, 1, 4, 4),
    12: (0, 1, 3, 1, 2, 4, 4),
    13: (0, 1, 3, 0, 2, 4, 4),
}
#: strategy -> {operation: stage}; the table of kittens_helpers.py:137-157.  On B200 only the
#: depth ``max(stage) + 1`` matters: it is the shared-memory ring depth.
PIPELINE_STRATEGIES = {k: dict(zip(_STAGE_KEYS, row)) for k, row in _STAGE_ROWS.items()}


def pipeline_strategy_stages(strategy: int) -> tuple[int, int]:
    """``(a_stages, b_stages)`` = max stage + 1 over each operand's operations and COMPUTE
    (kittens_helpers.py:161-169)."""
    s = PIPELINE_STRATEGIES[strategy]
    a = max(s[k] for k in ("A_LOAD", "A_LDS_WRITE", "A_LDS_READ", "COMPUTE"))
    b = max(s[k] for k in ("B_LOAD", "B_LDS_WRITE", "B_LDS_READ", "COMPUTE"))
    return a + 1, b + 1


def shuffle_weight(B: np.ndarray) -> np.ndarray:
    """Preshuffle ``B[N, K]`` into the reference's direct-B order (kittens_helpers.py:90-119).

    Within every 16-row x 32-column block, the element at (row r, column 16*h + 4*g + w) moves
    to position ``((g * 16 + r) * 2 + h) * 4 + w`` of the block's 512 elements, and blocks are
    stored n-block-major, k-block-minor.  Same shape and dtype as ``B``.
    """
    N, K = B.shape
    assert N % 16 == 0, f"N={N} must be multiple of 16"
    assert K % 32 == 0, f"K={K} must be multiple of 32"
    blocks = B.reshape(N // 16, 16, K // 32, 2, 4, 4)  # (nb, r, kb, h, g, w)
    return np.ascontiguousarray(blocks.transpose(0, 2, 4, 1, 3, 5)).reshape(N, K)  # (nb, kb, g, r, h, w)


def coop_2d_split(num_tiles: int, num_waves: int, kt: int) -> tuple[int, int, int, int]:
    """``(waves_s, waves_k, coop_s, coop_k)``: how ``num_waves`` share ``num_tiles x kt``
    transfer tiles with the least padding (coop.py:12-27).  TMA makes the split moot on B200;
    it is kept because the resource accounting of the operator surface refers to it."""
    best_key, best = None, None
    for ws in (d for d in range(1, num_waves + 1) if num_waves % d == 0):
        wk = num_waves // ws
        cs, ck = math.ceil(num_tiles / ws), math.ceil(kt / wk)
        key = (ws * wk * cs * ck - num_tiles * kt, max(0, ws - num_tiles) + max(0, wk - kt), -ws)
        if best_key is None or key < best_key:
            best_key, best = key, (ws, wk, cs, ck)
    return best
