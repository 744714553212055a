"""Host driver of the scores-and-softmax op and the depthwise convolution.

Mirror of the reference's ``gm_attention/nn/fused_attention.py`` for callers:
the same module globals (``MODE``, ``MAX_*``), planning helpers (``plan``,
``plan_depthwise``, ``plan_head``, ``descriptors``), per-edge-set constants
(``Geometry``, ``geometry``, chunk registry), enable predicates, the two
``torch.autograd.Function``s with their argument orders, and the module-level
entry points (``softmax``, ``softmax_head``, ``forward_depthwise``).  Owners
(attention / convolution modules) and edge sets are duck-typed: any object
with the attributes the reference's classes carry works.

What differs is underneath: ``extension()`` returns the ctypes-backed shim of
``libgmb200.so`` (:class:`gm_attention_b200.nn.ext.AttentionExtension`), the
kernels are the sm_100a ones, and the mode ``"cpu"`` is refused -- this build
has no CPU implementation.

``GM_FUSED_ATTENTION``: ``"0"`` off (callers take their eager path), ``"1"``
on for CUDA tensors.
"""

from __future__ import annotations

import functools
import os
import weakref
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any

import torch
from torch import Tensor

from gm_attention_b200.nn.windows import evaluate_aggregation_window

MAX_H, MAX_F, MAX_D, MAX_SLOTS, DESC = 8, 8, 512, 8192, 5
#: kept for callers that size by them; the sm_100a kernels take any neighbourhood
#: size (logits spill to the alpha buffer beyond the shared-memory budget)
THREADS, MAX_SMEM = 128, 96 * 1024
MODE = os.environ.get("GM_FUSED_ATTENTION", "0")


@functools.cache
def extension(cuda: bool = True) -> Any:
    """The extension-module stand-in.  ``cuda=False`` (the reference's CPU
    driver) does not exist in this build."""
    if not cuda:
        raise RuntimeError("gm_attention_b200 has no CPU driver: the fused ops run on CUDA tensors only")
    from gm_attention_b200 import _lib
    from gm_attention_b200.nn.ext import AttentionExtension

    _lib.lib()  # fail loudly now if libgmb200.so is missing
    return AttentionExtension()


# --------------------------------------------------------------------- plans


@dataclass(frozen=True)
class Plan:
    """Descriptor rows ``(n, a_n, flat offset, coefficient offset, dim)``, one
    per frequency of a head's type, with the sizes the kernels need."""

    rows: tuple[tuple[int, int, int, int, int], ...]
    heads: int
    width: int
    a_0: int
    complex_width: int
    max_order: int


_PLAN_KEY = "_fused_attention_plan"


def _plan(owner: Any, attn: Any, full: Any, heads: int) -> Plan:
    """Lay one head's type ``attn`` out inside the heads' direct sum ``full``
    (layout rule: reference ``fused_attention.py:98-114``)."""
    store = owner.__dict__
    if store.get(_PLAN_KEY) is not None:
        return store[_PLAN_KEY]  # type: ignore[no-any-return]
    starts = {n: s.start for n, s in full.slices().items()}
    rows = []
    coefficient_offset = 0
    for n, copies in attn.items():
        rows.append((n, copies, starts[n], 0 if n == 0 else coefficient_offset, 1 if n == 0 else 2))
        if n > 0:
            coefficient_offset += 4 * copies
    orders = [2 * n for n, _ in attn.items()]
    built = Plan(rows=tuple(rows), heads=heads, width=full.dimension, a_0=attn.multiplicity(0) if 0 in attn else 0,
                 complex_width=coefficient_offset, max_order=max(orders, default=0))
    store[_PLAN_KEY] = built
    return built


def plan(mhsa: Any) -> Plan:
    return _plan(mhsa, mhsa.field_type_attn, mhsa.field_type_in, mhsa.num_heads)


def plan_depthwise(conv: Any) -> Plan:
    return _plan(conv, conv.kernel.field_type, conv.kernel.field_type, 1)


def plan_head(head: Any) -> Plan:
    return _plan(head, head.field_type_attn, head.field_type_attn, 1)


def descriptors(owner: Any, p: Plan, device: torch.device) -> Tensor:
    """The plan's rows as an int64 ``(F, 5)`` tensor, cached on the owner per device."""
    key = ("_fused_attention_desc", str(device))
    if owner.__dict__.get(key) is None:
        owner.__dict__[key] = torch.tensor([list(r) for r in p.rows], dtype=torch.int64, device=device).reshape(-1, DESC)
    return owner.__dict__[key]  # type: ignore[no-any-return]


# --------------------------------------------------------------------- per-edge constants


def _segment_sum(values: Tensor, row_ptr: Tensor) -> Tensor:
    return torch.segment_reduce(values, "sum", offsets=row_ptr, axis=0)


@dataclass
class Geometry:
    """The constants of one edge set under one cutoff, window and dtype."""

    transport: Tensor  # (E, orders, 2)
    angular: Tensor  # (E, orders, 2)
    rho: Tensor  # (E,)  r / cutoff
    weights: Tensor  # (E,)  window * tangent quadrature weight
    bias: Tensor  # (E,)  log window + log tangent quadrature weight
    inside: Tensor  # (E,) uint8  window > 0
    row_ptr: Tensor  # (N + 1,) int64
    source: Tensor  # (E,) int64
    max_degree: int
    normalized: dict[float, Tensor] = field(default_factory=dict)
    base: Geometry | None = None
    span: tuple[int, int] | None = None
    chunk_degrees: dict[tuple[int, int], int] = field(default_factory=dict)

    def aggregation_weights(self, normalize: bool, eps: float) -> Tensor:
        """``weights``, or ``weights`` over each target's clamped window mass.
        A chunk (whole neighbourhoods of its parent) slices its parent's."""
        if self.base is not None and self.span is not None:
            lo, hi = self.span
            return self.base.aggregation_weights(normalize, eps)[lo:hi]
        if not normalize:
            return self.weights
        if eps not in self.normalized:
            mass = _segment_sum(self.weights, self.row_ptr).clamp_min(eps)
            degrees = self.row_ptr[1:] - self.row_ptr[:-1]
            self.normalized[eps] = (self.weights / torch.repeat_interleave(mass, degrees)).contiguous()
        return self.normalized[eps]


_GEOMETRIES: OrderedDict[tuple, tuple[Any, Geometry]] = OrderedDict()
_GEOMETRY_CACHE = 64
_CHUNKS: dict[int, tuple[Any, Any, int, int]] = {}


def _purge() -> None:
    for key in [k for k, (alive, _) in _GEOMETRIES.items() if alive() is None]:
        del _GEOMETRIES[key]
    for key in [k for k, (alive, *_rest) in _CHUNKS.items() if alive() is None]:
        del _CHUNKS[key]


def register_chunk(chunk: Any, parent: Any, first: int, last: int) -> None:
    """Declare ``chunk`` to be the edges ``first .. last`` of ``parent`` in
    order, so :func:`geometry` answers it with views of the parent's tables."""
    _purge()
    _CHUNKS[id(chunk.row_ptr)] = (weakref.ref(chunk.row_ptr), parent, int(first), int(last))


def chunk_of(edges: Any) -> tuple[Any, int, int] | None:
    entry = _CHUNKS.get(id(edges.row_ptr))
    if entry is None or entry[0]() is not edges.row_ptr:
        return None
    return entry[1], entry[2], entry[3]


def _largest_degree(row_ptr: Tensor) -> int:
    return int((row_ptr[1:] - row_ptr[:-1]).max()) if row_ptr.numel() > 1 else 0


def geometry(edges: Any, cutoff: float, window: str, dtype: torch.dtype) -> Geometry:
    """Per-edge constants of ``edges``, built once per (edge set, cutoff,
    window, dtype, device) and held while the edge set's ``row_ptr`` lives."""
    _purge()
    registered = chunk_of(edges)
    if registered is not None:
        parent, first, last = registered
        base = geometry(parent, cutoff, window, dtype)
        if (first, last) not in base.chunk_degrees:
            base.chunk_degrees[(first, last)] = _largest_degree(edges.row_ptr)
        return Geometry(base.transport[first:last], base.angular[first:last], base.rho[first:last], base.weights[first:last],
                        base.bias[first:last], base.inside[first:last], edges.row_ptr.contiguous(),
                        edges.source_index.contiguous(), base.chunk_degrees[(first, last)], base=base, span=(first, last))
    key = (id(edges.row_ptr), float(cutoff), window, dtype, str(edges.row_ptr.device))
    hit = _GEOMETRIES.get(key)
    if hit is not None and hit[0]() is edges.row_ptr:
        _GEOMETRIES.move_to_end(key)
        return hit[1]
    tiny = torch.finfo(dtype).tiny
    r = edges.distances.to(dtype)
    quadrature = edges.tangent_quadrature_weights.to(dtype)
    window_values = evaluate_aggregation_window(r, cutoff, window)
    row_ptr = edges.row_ptr.contiguous()
    built = Geometry(
        transport=torch.view_as_real(edges.transport_phases.contiguous()).to(dtype).contiguous(),
        angular=torch.view_as_real(edges.angular_phases.contiguous()).to(dtype).contiguous(),
        rho=(r / cutoff).contiguous(),
        weights=(window_values * quadrature).contiguous(),
        bias=(torch.log(window_values.clamp_min(tiny)) + torch.log(quadrature.clamp_min(tiny))).contiguous(),
        inside=(window_values > 0.0).to(torch.uint8).contiguous(),
        row_ptr=row_ptr,
        source=edges.source_index.contiguous(),
        max_degree=_largest_degree(row_ptr),
    )
    _GEOMETRIES[key] = (weakref.ref(edges.row_ptr), built)
    while len(_GEOMETRIES) > _GEOMETRY_CACHE:
        _GEOMETRIES.popitem(last=False)
    return built


# --------------------------------------------------------------------- enable predicates


def _mode_allows(x: Any) -> bool:
    if MODE == "0":
        return False
    if MODE == "cpu":
        raise RuntimeError("GM_FUSED_ATTENTION=cpu is not provided by gm_attention_b200 (no CPU path)")
    return x.device.type == "cuda" and x.dtype in (torch.float32, torch.float64)


def _layout_fits(p: Plan, highest_order: int, edges: Any) -> bool:
    return len(p.rows) <= MAX_F and p.width <= MAX_D and highest_order <= edges.max_frequency and edges.n_edges > 0


def softmax_enabled(mhsa: Any, x: Any, edges: Any) -> bool:
    """Whether the batched multi-head path takes :func:`softmax`."""
    if not _mode_allows(x) or mhsa.num_heads > MAX_H:
        return False
    p = plan(mhsa)
    return _layout_fits(p, max((r[0] for r in p.rows), default=0), edges)


def softmax_head_enabled(head: Any, x: Any, edges: Any) -> bool:
    """Whether the per-head path takes :func:`softmax_head`."""
    if not _mode_allows(x):
        return False
    p = plan_head(head)
    return _layout_fits(p, max((r[0] for r in p.rows), default=0), edges)


def enabled_depthwise(conv: Any, x: Any, edges: Any) -> bool:
    """Whether a depthwise convolution takes :func:`forward_depthwise`."""
    if not _mode_allows(x):
        return False
    p = plan_depthwise(conv)
    return _layout_fits(p, p.max_order, edges)


# --------------------------------------------------------------------- autograd functions


class Depthwise(torch.autograd.Function):
    """Depthwise convolution, differentiable in ``v``, ``rc`` and ``cc``."""

    @staticmethod
    def forward(ctx: Any, v: Tensor, rc: Tensor, cc: Tensor, transport: Tensor, angular: Tensor, rho: Tensor, weights: Tensor,
                desc: Tensor, row_ptr: Tensor, source: Tensor, a_0: int, complex_width: int) -> Tensor:
        with torch.profiler.record_function("gm::conv/fused"):
            out = extension(True).conv_forward(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, a_0, complex_width)
        ctx.save_for_backward(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source)
        ctx.widths = (a_0, complex_width)
        return out  # type: ignore[no-any-return]

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_out: Tensor) -> tuple:  # type: ignore[override]
        with torch.profiler.record_function("gm::conv/fused_backward"):
            dv, drc, dcc = extension(True).conv_backward(grad_out.contiguous(), *ctx.saved_tensors, *ctx.widths)
        return (dv, drc, dcc) + (None,) * 9


class Softmax(torch.autograd.Function):
    """Heads' scores and neighbourhood softmax, differentiable in ``q`` and ``k``."""

    @staticmethod
    def forward(ctx: Any, q: Tensor, k: Tensor, transport: Tensor, bias: Tensor, inside: Tensor, desc: Tensor, row_ptr: Tensor,
                source: Tensor, heads: int, scale: float, max_degree: int) -> Tensor:
        with torch.profiler.record_function("gm::attention/fused_softmax"):
            alpha = extension(True).softmax_forward(q, k, transport, bias, inside, desc, row_ptr, source, heads, scale, max_degree)
        ctx.save_for_backward(q, k, transport, bias, inside, desc, row_ptr, source, alpha)
        ctx.scalars = (heads, scale, max_degree)
        return alpha  # type: ignore[no-any-return]

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_alpha: Tensor) -> tuple:  # type: ignore[override]
        with torch.profiler.record_function("gm::attention/fused_softmax_backward"):
            dq, dk = extension(True).softmax_backward(grad_alpha.contiguous(), *ctx.saved_tensors, *ctx.scalars)
        return (dq, dk) + (None,) * 9


# --------------------------------------------------------------------- module-level entry points


def forward_depthwise(conv: Any, v: Tensor, real_coefficients: Tensor | None, complex_coefficients: Tensor | None,
                      edges: Any) -> Tensor:
    """Aggregate the flat node field ``v (N, D)`` over ``edges`` under the
    kernel's per-edge coefficients ``(1, E, a_0)`` / ``(1, E, W)``."""
    p = plan_depthwise(conv)
    g = geometry(edges, conv.cutoff, conv.window, v.dtype)
    none = v.new_zeros(0)
    rc = none if real_coefficients is None else real_coefficients.contiguous()
    cc = none if complex_coefficients is None else complex_coefficients.contiguous()
    weights = g.aggregation_weights(bool(conv.normalize), float(conv.eps))
    return Depthwise.apply(v.contiguous(), rc, cc, g.transport, g.angular, g.rho, weights, descriptors(conv, p, v.device),  # type: ignore[no-any-return]
                           g.row_ptr, g.source, p.a_0, p.complex_width)


def softmax(mhsa: Any, q: Tensor, k: Tensor, edges: Any) -> Tensor:
    """Attention weights ``(E, H)`` of a multi-head layer from its flat
    projected queries and keys."""
    p = plan(mhsa)
    g = geometry(edges, mhsa.cutoff, mhsa.heads[0].window, q.dtype)
    return Softmax.apply(q.contiguous(), k.contiguous(), g.transport, g.bias, g.inside, descriptors(mhsa, p, q.device),  # type: ignore[no-any-return]
                         g.row_ptr, g.source, p.heads, float(mhsa.heads[0]._score_scale), max(g.max_degree, 1))


def softmax_head(head: Any, q: Tensor, k: Tensor, edges: Any) -> Tensor:
    """One head's attention weights ``(E,)``."""
    p = plan_head(head)
    g = geometry(edges, head.cutoff, head.window, q.dtype)
    alpha = Softmax.apply(q.contiguous(), k.contiguous(), g.transport, g.bias, g.inside, descriptors(head, p, q.device),
                          g.row_ptr, g.source, 1, float(head._score_scale), max(g.max_degree, 1))
    return alpha.reshape(-1)  # type: ignore[no-any-return]
