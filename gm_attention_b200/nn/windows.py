"""Aggregation windows and the cutoff comparison they share with the edge search.

Semantics of the reference's ``nn/convolution.py:47-91`` (windows) and
``discretization/edge_geometry.py:399-462`` (tolerant comparison): the hard
window is the indicator of ``r <= cutoff + slack`` (slack 1e-10 for float64
distances, 1e-5 otherwise) under the default ``whole-shell`` rule and a strict
``r <= cutoff`` under ``legacy``; the quartic window is
``relu(1 - (r / cutoff)^2)^2``.  ``GM_CUTOFF_RULE`` is read once at import.
"""

from __future__ import annotations

import math
import os

import torch
from torch import Tensor

CUTOFF_RULES = ("whole-shell", "legacy")
CUTOFF_RULE = os.environ.get("GM_CUTOFF_RULE", "whole-shell")
if CUTOFF_RULE not in CUTOFF_RULES:
    raise ValueError(f"GM_CUTOFF_RULE must be one of {CUTOFF_RULES}, got {CUTOFF_RULE!r}.")

#: slack of a membership decision made from float64 lattice coordinates
EXACT_SLACK = 1e-10


def cutoff_tolerance(dtype: torch.dtype) -> float:
    return 1e-10 if dtype == torch.float64 else 1e-5


def within_cutoff(distances: Tensor, cutoff: float) -> Tensor:
    if CUTOFF_RULE == "legacy":
        return distances <= float(cutoff)
    return distances <= float(cutoff) + cutoff_tolerance(distances.dtype)


def evaluate_aggregation_window(distances: Tensor, radius: float, kind: str) -> Tensor:
    if not (math.isfinite(radius) and radius > 0.0):
        raise ValueError(f"radius must be finite and positive, got {radius}.")
    if kind == "hard":
        return within_cutoff(distances, radius).to(distances.dtype)
    if kind == "quartic":
        return torch.relu(1.0 - (distances / radius) ** 2) ** 2
    raise ValueError(f"window must be 'hard' or 'quartic', got {kind!r}.")
