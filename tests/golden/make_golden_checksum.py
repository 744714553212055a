"""The order-sensitive CSR checksum stored in ``geometry_counts.npz`` (shared by
the fixture generator and the tests)."""

from __future__ import annotations

import numpy as np


def csr_checksum(row_ptr: np.ndarray, source: np.ndarray) -> int:
    with np.errstate(over="ignore"):
        idx = np.arange(1, source.shape[0] + 1, dtype=np.uint64)
        a = np.sum(source.astype(np.uint64) * (idx * np.uint64(0x9E3779B97F4A7C15) + np.uint64(1)), dtype=np.uint64)
        idp = np.arange(1, row_ptr.shape[0] + 1, dtype=np.uint64)
        b = np.sum(row_ptr.astype(np.uint64) * (idp * np.uint64(0xC2B2AE3D27D4EB4F) + np.uint64(1)), dtype=np.uint64)
    return int(a ^ b)
