"""Host driver of the fused pair terms of the general steerable kernel.

Mirror of the reference's ``gm_attention/nn/fused_pairs.py``: ``MODE``,
``SUPPORTED``, ``Term``, ``plan``, ``enabled``, ``extension`` and the flags.
The reference compiles one CUDA extension per ``(a, b, trunk)``; here a single
kernel serves every ``a, b, trunk <= 16`` (runtime sizes, bounds unrolled), so
``extension()`` takes the sizes only for signature compatibility.
"""

from __future__ import annotations

import functools
import os
from dataclasses import dataclass
from typing import Any

import torch

MAX_MULT, MAX_TRUNK = 16, 16
#: every block size up to MAX_MULT is served (the reference's CPU build lists a fixed set)
SUPPORTED = tuple(range(1, MAX_MULT + 1))
MATRIX_COMPLEX, U_REAL, CONJ_U, OUT_REAL = 1, 2, 4, 8
MODE = os.environ.get("GM_FUSED_PAIRS", "0")


@functools.cache
def extension(a: int | None = None, b: int | None = None, trunk: int | None = None) -> Any:
    from gm_attention_b200 import _lib
    from gm_attention_b200.nn.ext import PairsExtension

    _lib.lib()
    return PairsExtension()


@dataclass(frozen=True)
class Term:
    """One (n, m, role) pair term: block shape, flags, rows of the readout, phase orders, radial power."""

    n: int
    m: int
    role: str
    flags: int
    a: int
    b: int
    real_head: bool
    rows: slice
    pre_order: int | None
    post_order: int | None
    power: int | None


def plan(kernel: Any) -> list[Term]:
    """The terms in the order of the general kernel's pair loop (reference ``fused_pairs.py:98-123``):
    for every output frequency m, for every input frequency n."""
    cached = kernel.__dict__.get("_fused_plan")
    if cached is not None:
        return cached  # type: ignore[no-any-return]
    terms: list[Term] = []
    for m in kernel.field_type_out.frequencies:
        b = kernel.field_type_out.multiplicity(m)
        for n in kernel.field_type_in.frequencies:
            a = kernel.field_type_in.multiplicity(n)
            if n == 0 and m == 0:
                terms.append(Term(n, m, "real", U_REAL | OUT_REAL, a, b, True, slice(0, a * b), None, None, None))
                continue
            rows, power = kernel._pair_ranges[(n, m, "linear")], kernel._pair_powers[(n, m, "linear")]
            if n == 0:
                terms.append(Term(n, m, "linear", MATRIX_COMPLEX | U_REAL, a, b, False, rows, None, m, power))
            elif m == 0:
                terms.append(Term(n, m, "linear", MATRIX_COMPLEX | CONJ_U | OUT_REAL, a, b, False, rows, n, None, power))
            else:
                terms.append(Term(n, m, "linear", MATRIX_COMPLEX, a, b, False, rows, m - n, None, power))
                terms.append(Term(n, m, "antilinear", MATRIX_COMPLEX | CONJ_U, a, b, False, kernel._pair_ranges[(n, m, "antilinear")],
                                  m + n, None, kernel._pair_powers[(n, m, "antilinear")]))
    kernel.__dict__["_fused_plan"] = terms
    return terms


def enabled(kernel: Any, x: Any, edges: Any) -> bool:
    if MODE == "0":
        return False
    if MODE == "cpu":
        raise RuntimeError("GM_FUSED_PAIRS=cpu is not provided by gm_attention_b200 (no CPU path)")
    if x.device.type != "cuda" or x.dtype not in (torch.float32, torch.float64):
        return False
    head = kernel.complex_head if kernel.complex_head is not None else kernel.real_head
    if not 1 <= head.in_features <= MAX_TRUNK:
        return False
    for term in plan(kernel):
        if not (1 <= term.a <= MAX_MULT and 1 <= term.b <= MAX_MULT):
            return False
        if any(o is not None and abs(o) > edges.max_frequency for o in (term.pre_order, term.post_order)):
            return False
    return True
