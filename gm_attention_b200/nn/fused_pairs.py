"""Host driver of the fused pair terms of the general steerable kernel.

Mirror of the reference's ``gm_attention/nn/fused_pairs.py``: ``MODE``,
``SUPPORTED``, ``Term``, ``plan``, ``enabled``, ``extension``, the flags, the
autograd function ``_FusedPairs`` (``fused_pairs.py:156-238``) and the driver
entry ``forward_general`` (``:247-295``).  The reference compiles one CUDA
extension per ``(a, b, trunk)``; here a single kernel serves every
``a, b, trunk <= 16`` (runtime sizes, bounds unrolled), so ``extension()``
takes the sizes only for signature compatibility.

``_FusedPairs.apply(hidden, complex_weight, complex_bias, real_weight, real_bias,
meta, phases, scales, *vectors)`` keeps the reference's argument order and
``meta`` keys (``terms``, ``tables``, ``in_index``, ``out_index``,
``out_frequencies``, ``out_multiplicity``): one launch per term forward, one per
term backward (input and trunk gradients accumulated in place, the term's
coefficient-major slab of the coefficient gradient written), then the readout
weight / bias gradients as ONE product of the coefficient gradient with
``[hidden | 1]``, summed over blocks of 16 384 edges like the reference's
``_blocked_weight_gradient`` (``nn/kernels.py:49-64``).
"""

from __future__ import annotations

import functools
import os
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

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


# ----------------------------------------------------------------------------- the autograd function

#: edges per block of the readout-gradient product (the reference's SPLIT_K_ROWS, ``nn/kernels.py:33``)
GRADIENT_BLOCK_ROWS = 16384


def _complex_of(real_dtype: torch.dtype) -> torch.dtype:
    return torch.complex128 if real_dtype == torch.float64 else torch.complex64


def _none(like: Tensor) -> Tensor:
    return like.new_empty(0)


def _head_rows(term: Term, cw: Tensor | None, cb: Tensor | None, rw: Tensor | None, rb: Tensor | None) -> tuple[Tensor, Tensor]:
    """The readout rows (and bias entries, or an empty tensor) that produce the term's block."""
    weight, bias = (rw, rb) if term.real_head else (cw, cb)
    if weight is None:
        raise RuntimeError(f"term ({term.n}, {term.m}, {term.role}) needs the {'real' if term.real_head else 'complex'} head")
    return weight[term.rows].contiguous(), (_none(weight) if bias is None else bias[term.rows].contiguous())


def _coefficient_product(grad_k: Tensor, operand: Tensor) -> Tensor:
    """``grad_k (width, E) @ operand (E, K) -> (width, K)``, summed over blocks of GRADIENT_BLOCK_ROWS edges (a batched
    product over the whole blocks, one more for the remainder): partial sums of bounded length, as the reference forms them."""
    width, e = grad_k.shape
    blocks = e // GRADIENT_BLOCK_ROWS
    if blocks < 2:
        return grad_k @ operand
    whole = blocks * GRADIENT_BLOCK_ROWS
    left = grad_k[:, :whole].reshape(width, blocks, GRADIENT_BLOCK_ROWS).permute(1, 0, 2)  # (blocks, width, rows): a view
    right = operand[:whole].reshape(blocks, GRADIENT_BLOCK_ROWS, operand.shape[1])
    total = torch.bmm(left, right).sum(0)
    if whole < e:
        total = total + grad_k[:, whole:] @ operand[whole:]
    return total


class _FusedPairs(torch.autograd.Function):
    """Every pair term of one general-kernel call (reference ``fused_pairs.py:156-238``)."""

    @staticmethod
    def forward(ctx: Any, hidden: Tensor, complex_weight: Tensor | None, complex_bias: Tensor | None, real_weight: Tensor | None,  # type: ignore[override]
                real_bias: Tensor | None, meta: dict[str, Any], phases: tuple[Tensor, ...], scales: tuple[Tensor, ...],
                *vectors: Tensor) -> tuple[Tensor, ...]:
        ext = extension()
        e = hidden.shape[0]
        outputs = [torch.zeros(e, meta["out_multiplicity"][m], dtype=hidden.dtype if m == 0 else _complex_of(hidden.dtype), device=hidden.device)
                   for m in meta["out_frequencies"]]
        for term, (pre, post, power) in zip(meta["terms"], meta["tables"], strict=True):
            weight, bias = _head_rows(term, complex_weight, complex_bias, real_weight, real_bias)
            ext.forward(hidden, weight, bias, vectors[meta["in_index"][term.n]],
                        _none(hidden) if pre is None else phases[pre], _none(hidden) if post is None else phases[post],
                        _none(hidden) if power is None else scales[power], outputs[meta["out_index"][term.m]], term.a, term.b, term.flags)
        ctx.save_for_backward(hidden, complex_weight, complex_bias, real_weight, real_bias, *phases, *scales, *vectors)
        ctx.meta, ctx.sizes = meta, (len(phases), len(scales))
        return tuple(outputs)

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Tensor | None) -> tuple[Any, ...]:  # type: ignore[override]
        meta = ctx.meta
        n_phases, n_scales = ctx.sizes
        hidden, cw, cb, rw, rb, *rest = ctx.saved_tensors
        phases, scales, vectors = rest[:n_phases], rest[n_phases:n_phases + n_scales], rest[n_phases + n_scales:]
        ext = extension()
        e = hidden.shape[0]
        upstream = []
        for g, m in zip(grad_outputs, meta["out_frequencies"], strict=True):
            if g is None:
                g = torch.zeros(e, meta["out_multiplicity"][m], dtype=hidden.dtype if m == 0 else _complex_of(hidden.dtype), device=hidden.device)
            upstream.append(g.contiguous())
        grad_hidden = torch.zeros_like(hidden)
        grad_vectors = [torch.zeros_like(v) for v in vectors]
        # coefficient gradients, coefficient-major (width, E): a term's rows are one contiguous slab
        slabs = {True: None if rw is None else hidden.new_empty(rw.shape[0], e), False: None if cw is None else hidden.new_empty(cw.shape[0], e)}
        for term, (pre, post, power) in zip(meta["terms"], meta["tables"], strict=True):
            weight, bias = _head_rows(term, cw, cb, rw, rb)
            slot = meta["in_index"][term.n]
            ext.backward(hidden, weight, bias, vectors[slot], _none(hidden) if pre is None else phases[pre],
                         _none(hidden) if post is None else phases[post], _none(hidden) if power is None else scales[power],
                         upstream[meta["out_index"][term.m]], grad_vectors[slot], grad_hidden, slabs[term.real_head][term.rows],
                         term.a, term.b, term.flags)
        # d weight = grad_k hidden, d bias = grad_k 1: one product against [hidden | 1]
        any_bias = cb is not None or rb is not None
        operand = torch.cat((hidden, hidden.new_ones(e, 1)), 1) if any_bias else hidden

        def readout_gradients(grad_k: Tensor | None, bias: Tensor | None) -> tuple[Tensor | None, Tensor | None]:
            if grad_k is None:
                return None, None
            product = _coefficient_product(grad_k, operand)
            if not any_bias:
                return product, None
            return product[:, :-1], (product[:, -1] if bias is not None else None)

        grad_cw, grad_cb = readout_gradients(slabs[False], cb)
        grad_rw, grad_rb = readout_gradients(slabs[True], rb)
        return (grad_hidden, grad_cw, grad_cb, grad_rw, grad_rb, None, None, None, *grad_vectors)


# ----------------------------------------------------------------------------- driver entry

def _trunk_output(kernel: Any, distances: Tensor) -> Tensor:
    """Radial basis then the Linear / SiLU trunk, ``(E, trunk width)`` (reference ``nn/kernels.py:108-117, 605-607``)."""
    hidden = kernel.radial_basis(distances)
    for layer in kernel.radial_trunk:
        hidden = layer(hidden)
    return hidden.contiguous()


def _transported_vectors(x: Any, edges: Any, frequencies: list[int]) -> tuple[Tensor, ...]:
    """Per input frequency the source node's coefficients in the TARGET gauge, per edge: ``e^{i n gamma} x_n[source]``
    as ``(E, a_n)`` complex, ``x_0[source]`` as ``(E, a_0)`` real (reference ``nn/kernels.py:156-189``).  ``x`` is an
    edge-level field when its leading size is the edge count, a node-level field otherwise."""
    out = []
    for n in frequencies:
        values = x[n]
        if values.shape[0] != edges.n_edges:
            values = values.index_select(0, edges.source_index)
        if n == 0:
            out.append(values.contiguous())
        else:
            z = torch.view_as_complex(values.contiguous()) if not values.is_complex() else values
            out.append((edges.transport_harmonic(n).unsqueeze(-1) * z).contiguous())
    return tuple(out)


def forward_general(kernel: Any, x: Any, edges: Any) -> Any:
    """``kernel._forward_general(x, edges)`` through the fused terms (reference ``fused_pairs.py:247-295``).

    ``kernel`` is the reference's ``SO2SteerableKernel`` or any object with its attributes (``field_type_in / _out``,
    ``radial_basis``, ``radial_trunk``, ``complex_head`` / ``real_head``, ``_pair_ranges``, ``_pair_powers``,
    ``_radial_powers``); ``x`` maps a frequency to ``(E or N, a_n[, 2])`` coefficients and carries ``field_type``; the
    result is built with ``type(x)(field_type_out, {m: coefficients})``."""
    terms = plan(kernel)
    with torch.profiler.record_function("gm::kernel/radial"):
        hidden = _trunk_output(kernel, edges.distances)
    in_frequencies, out_frequencies = list(kernel.field_type_in.frequencies), list(kernel.field_type_out.frequencies)
    with torch.profiler.record_function("gm::transport"):
        vectors = _transported_vectors(x, edges, in_frequencies)
    orders = sorted({o for t in terms for o in (t.pre_order, t.post_order) if o is not None})
    powers = sorted({t.power for t in terms if t.power is not None})
    phases = tuple(edges.angular_harmonic(o).contiguous() for o in orders)
    table = kernel._radial_powers(edges.distances) if powers else None
    scales = tuple(table[:, p].contiguous() for p in powers)
    where_order, where_power = {o: i for i, o in enumerate(orders)}, {p: i for i, p in enumerate(powers)}
    meta = {
        "terms": terms,
        "tables": [(where_order.get(t.pre_order), where_order.get(t.post_order), where_power.get(t.power)) for t in terms],
        "in_index": {n: i for i, n in enumerate(in_frequencies)},
        "out_index": {m: i for i, m in enumerate(out_frequencies)},
        "out_frequencies": out_frequencies,
        "out_multiplicity": {m: kernel.field_type_out.multiplicity(m) for m in out_frequencies},
    }
    heads = (kernel.complex_head, kernel.real_head)
    params = [p for head in heads for p in ((None, None) if head is None else (head.weight, head.bias))]
    with torch.profiler.record_function("gm::kernel/pairs"):
        outputs = _FusedPairs.apply(hidden, *params, meta, phases, scales, *vectors)
    return type(x)(kernel.field_type_out, {m: (out if m == 0 else torch.view_as_real(out)) for m, out in zip(out_frequencies, outputs, strict=True)})


__all__ = ["MODE", "SUPPORTED", "Term", "enabled", "extension", "forward_general", "plan"]
