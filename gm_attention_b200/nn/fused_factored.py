"""Host driver of the factored steerable kernel.

Mirror of the reference's ``gm_attention/nn/fused_factored.py`` for callers:
``MODE`` and the bounds, ``Block`` / ``Plan`` / ``plan`` / ``descriptors``,
``pack``, ``source_groups`` (with its bounded cache), ``enabled``, the
``Factored`` and ``FactoredAggregate`` autograd functions with the reference's
argument orders, ``inputs`` / ``groups_for`` / ``forward`` /
``forward_aggregated``.  Kernels (``SO2SteerableKernel``-like) and edge sets are
duck-typed.  ``extension()`` returns the ctypes-backed shim of ``libgmb200.so``;
``GM_FUSED_FACTORED=cpu`` is refused (no CPU path).

One bound is lifted: the reference declines when the packed width
``2 wc + wr`` exceeds 320 (``MAX_C``); here ``MAX_C`` is 409 for the largest
trunk (``k (2 wc + wr) <= 8192``), which admits the 392- and 400-wide value
kernels of the 128 x 256 and 256 x 512 configurations.
"""

from __future__ import annotations

import functools
import os
import weakref
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

MAX_K, MAX_OUT, MAX_BM, MAX_KC, DESC = 20, 128, 32, 8192, 8
MAX_C = MAX_KC // MAX_K
NARROW_BM, NARROW_C = 16, 256  # kept for callers that report the tier; the sm_100a kernels have a single tier
MODE = os.environ.get("GM_FUSED_FACTORED", "0")


@functools.cache
def extension(cuda: bool = False) -> Any:
    if not cuda:
        raise RuntimeError("gm_attention_b200 has no CPU driver: the fused ops run on CUDA tensors only")
    from gm_attention_b200 import _lib
    from gm_attention_b200.nn.ext import FactoredExtension

    _lib.lib()
    return FactoredExtension()


@dataclass(frozen=True)
class Block:
    """One coefficient block's descriptor row."""

    block: tuple[int, int, str]
    kind: int
    z_offset: int
    b_m: int
    angular: int
    transport: int
    power: int
    out_offset: int
    take_real: int

    def row(self) -> list[int]:
        return [self.kind, self.z_offset, self.b_m, self.angular, self.transport, self.power, self.out_offset, self.take_real]


@dataclass(frozen=True)
class Plan:
    blocks: tuple[Block, ...]
    wc: int
    wr: int
    d_out: int
    max_bm: int


def block_orders(n: int, m: int, role: str) -> tuple[int, int]:
    """(angular order, transport order) of a block n -> m (reference ``fused_factored.py:127-136``):
    0 -> m: (m, 0); n -> 0: (n, -n); linear: (m - n, n); antilinear: (m + n, -n)."""
    if n == 0:
        return m, 0
    if m == 0:
        return n, -n
    return (m - n, n) if role == "linear" else (m + n, -n)


def plan_blocks(blocks: list[tuple[int, int, str]], field_type_out: Any, powers: dict[tuple[int, int, str], int]) -> Plan:
    """Descriptor rows for ``blocks`` (readout order), stably sorted by output offset; complex
    blocks' mixes are packed side by side in that order."""
    starts = {m: s.start for m, s in field_type_out.slices().items()}
    rows: list[Block] = []
    wc = wr = 0
    for n, m, role in sorted(blocks, key=lambda b: starts[b[1]]):
        b_m = field_type_out.multiplicity(m)
        if role == "real":
            rows.append(Block((n, m, role), 0, 0, b_m, 0, 0, 0, starts[0], 0))
            wr = b_m
            continue
        angular, transport = block_orders(n, m, role)
        rows.append(Block((n, m, role), 1, wc, b_m, angular, transport, int(powers[(n, m, role)]), starts[m], int(m == 0)))
        wc += b_m
    return Plan(tuple(rows), wc, wr, field_type_out.dimension, max((b.b_m for b in rows), default=1))


def plan(kernel: Any) -> Plan:
    cached = kernel.__dict__.get("_fused_factored_plan")
    if cached is None:
        cached = plan_blocks(kernel._blocks(), kernel.field_type_out, kernel._pair_powers)
        kernel.__dict__["_fused_factored_plan"] = cached
    return cached  # type: ignore[no-any-return]


def descriptors(kernel: Any, device: torch.device) -> Tensor:
    cache = kernel.__dict__.setdefault("_fused_factored_descriptors", {})
    if str(device) not in cache:
        cache[str(device)] = torch.tensor([b.row() for b in plan(kernel).blocks], dtype=torch.int32, device=device).reshape(-1, DESC)
    return cache[str(device)]  # type: ignore[no-any-return]


PACKED = "_packed"


def pack(kernel: Any, products: dict) -> tuple[Tensor, Tensor]:
    """``node_products`` as ``zc (N, K, wc, 2)`` and ``zr (N, K, wr)``, remembered on the dict."""
    if products.get(PACKED) is None:
        with torch.profiler.record_function("gm::kernel/pack"):
            products[PACKED] = _pack(plan(kernel), products)
    return products[PACKED]  # type: ignore[no-any-return]


def _pack(p: Plan, products: dict) -> tuple[Tensor, Tensor]:
    any_block = next(v for key, v in products.items() if key != PACKED)
    n_nodes, k = any_block.shape[0], any_block.shape[1]
    real_dtype = torch.float64 if any_block.dtype in (torch.complex128, torch.float64) else torch.float32
    complex_blocks = [b.block for b in p.blocks if b.kind == 1]
    real_blocks = [b.block for b in p.blocks if b.kind == 0]
    if complex_blocks:
        zc = torch.view_as_real(torch.cat([products[b] for b in complex_blocks], dim=-1).contiguous()).contiguous()
    else:
        zc = torch.zeros(n_nodes, k, 0, 2, dtype=real_dtype, device=any_block.device)
    zr = products[real_blocks[0]].contiguous() if real_blocks else torch.zeros(n_nodes, k, 0, dtype=real_dtype, device=any_block.device)
    return zc, zr


_GROUPS: OrderedDict[tuple, tuple[Any, tuple[Tensor, Tensor, Tensor]]] = OrderedDict()
GROUP_CACHE_SIZE = 512


def source_groups(source_index: Tensor, key: tuple | None = None, owner: Tensor | None = None) -> tuple[Tensor, Tensor, Tensor]:
    """``(order, group_ptr, group_source)``: the edges stably sorted by source, each source's
    half-open run in that order, and the sources; cached under ``key`` (tied to ``owner`` while it lives)."""
    if key is not None and key in _GROUPS:
        held, groups = _GROUPS[key]
        alive = owner is None if held is None else (held() is not None and held() is owner)
        if alive and groups[0].device == source_index.device:
            _GROUPS.move_to_end(key)
            return groups
    order = torch.argsort(source_index, stable=True)
    group_source, counts = torch.unique_consecutive(source_index[order], return_counts=True)
    group_ptr = torch.zeros(group_source.shape[0] + 1, dtype=torch.long, device=source_index.device)
    group_ptr[1:] = torch.cumsum(counts, 0)
    groups = (order.contiguous(), group_ptr.contiguous(), group_source.contiguous())
    if key is not None:
        _GROUPS[key] = (None if owner is None else weakref.ref(owner), groups)
        while len(_GROUPS) > GROUP_CACHE_SIZE:
            _GROUPS.popitem(last=False)
    return groups


def group_key(parent: Any, first: int, last: int) -> tuple:
    return (id(parent), parent.edge_index.data_ptr(), int(parent.n_edges), int(first), int(last))


def enabled(kernel: Any, x: Any, edges: Any) -> bool:
    if MODE == "0":
        return False
    if MODE == "cpu":
        raise RuntimeError("GM_FUSED_FACTORED=cpu is not provided by gm_attention_b200 (no CPU path)")
    if x.device.type != "cuda" or x.dtype not in (torch.float32, torch.float64):
        return False
    p = plan(kernel)
    head = kernel.complex_head if kernel.complex_head is not None else kernel.real_head
    k = head.in_features + 1
    if k > MAX_K or p.d_out > MAX_OUT or p.max_bm > MAX_BM or k * (-(-(2 * p.wc + p.wr) // 4) * 4) > MAX_KC:  # packed width padded to whole 16-byte vectors
        return False
    return edges.n_edges > 0


class Factored(torch.autograd.Function):
    """Rows ``(E, d_out)`` of the factored kernel, differentiable in ``(h, zc, zr)``."""

    @staticmethod
    def forward(ctx: Any, h: Tensor, zc: Tensor, zr: Tensor, angular: Tensor, transport: Tensor, rho: Tensor, desc: Tensor, source: Tensor,
                order: Tensor, group_ptr: Tensor, group_source: Tensor, d_out: int, max_bm: int) -> Tensor:
        with torch.profiler.record_function("gm::kernel/pairs"):
            out = extension(True).forward(h, zc, zr, angular, transport, rho, desc, source, order, group_ptr, group_source, d_out, max_bm)
        ctx.save_for_backward(h, zc, zr, angular, transport, rho, desc, source, order, group_ptr, group_source)
        return out  # type: ignore[no-any-return]

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_out: Tensor) -> tuple:  # type: ignore[override]
        with torch.profiler.record_function("gm::kernel/pairs_backward"):
            dh, dzc, dzr = extension(True).backward(grad_out.contiguous(), *ctx.saved_tensors)
        return (dh, dzc, dzr) + (None,) * 10


class FactoredAggregate(torch.autograd.Function):
    """Each target's weighted sum of its rows, differentiable in ``(h, zc, zr, weights)``."""

    @staticmethod
    def forward(ctx: Any, h: Tensor, zc: Tensor, zr: Tensor, weights: Tensor, angular: Tensor, transport: Tensor, rho: Tensor, desc: Tensor,
                source: Tensor, target: Tensor, row_ptr: Tensor, order: Tensor, group_ptr: Tensor, group_source: Tensor, d_out: int,
                max_bm: int) -> Tensor:
        ext = extension(True)
        with torch.profiler.record_function("gm::kernel/pairs"):
            rows = ext.forward(h, zc, zr, angular, transport, rho, desc, source, order, group_ptr, group_source, d_out, max_bm)
        with torch.profiler.record_function("gm::kernel/aggregate"):
            out = ext.aggregate(rows, weights, row_ptr)
        ctx.save_for_backward(h, zc, zr, weights, rows, angular, transport, rho, desc, source, target, order, group_ptr, group_source)
        return out  # type: ignore[no-any-return]

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_out: Tensor) -> tuple:  # type: ignore[override]
        h, zc, zr, weights, rows, angular, transport, rho, desc, source, target, order, group_ptr, group_source = ctx.saved_tensors
        with torch.profiler.record_function("gm::kernel/pairs_backward"):
            dh, dzc, dzr, dweights = extension(True).backward_aggregated(grad_out.contiguous(), target, weights, rows, h, zc, zr, angular,
                                                                         transport, rho, desc, source, order, group_ptr, group_source)
        return (dh, dzc, dzr, dweights) + (None,) * 12


@dataclass(frozen=True)
class Inputs:
    h: Tensor
    zc: Tensor
    zr: Tensor
    angular: Tensor
    transport: Tensor
    rho: Tensor
    desc: Tensor
    source: Tensor
    plan: Plan


def inputs(kernel: Any, x: Any, edges: Any, products: dict | None) -> Inputs:
    """The op's inputs for ``kernel`` over ``edges`` on the node field ``x``."""
    if products is None:
        products = kernel.node_products(x)
    h = kernel._trunk_hidden(edges)
    zc, zr = pack(kernel, products)
    rho = (edges.distances / kernel.radial_basis.cutoff).to(h.dtype).contiguous()
    angular = torch.view_as_real(edges.angular_phases.contiguous()).contiguous().to(h.dtype)
    transport = torch.view_as_real(edges.transport_phases.contiguous()).contiguous().to(h.dtype)
    p = plan(kernel)
    needed = max((max(abs(b.angular), abs(b.transport)) for b in p.blocks), default=0)
    if needed >= angular.shape[1] or needed >= transport.shape[1]:
        raise ValueError(f"the geometry's phase tables ({angular.shape[1]} orders) are narrower than the kernel's blocks need (order {needed})")
    return Inputs(h.contiguous(), zc, zr, angular, transport, rho, descriptors(kernel, h.device), edges.source_index.contiguous(), p)


def groups_for(edges: Any, source: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    from gm_attention_b200.nn import fused_attention

    registered = fused_attention.chunk_of(edges)
    parent, first, last = registered if registered is not None else (edges, 0, int(edges.n_edges))
    return source_groups(source, group_key(parent, first, last), owner=parent.edge_index)


def _wrap_output(kernel: Any, flat: Tensor) -> Any:
    make = getattr(kernel, "output_field", None)  # kernels of the reference library wrap with SO2FeatureField.from_flat
    return make(flat) if make is not None else flat


def forward(kernel: Any, x: Any, edges: Any, products: dict | None = None, groups: tuple[Tensor, Tensor, Tensor] | None = None) -> Any:
    i = inputs(kernel, x, edges, products)
    order, group_ptr, group_source = groups_for(edges, i.source) if groups is None else groups
    flat = Factored.apply(i.h, i.zc, i.zr, i.angular, i.transport, i.rho, i.desc, i.source, order, group_ptr, group_source, i.plan.d_out,
                          i.plan.max_bm)
    return _wrap_output(kernel, flat)


def forward_aggregated(kernel: Any, x: Any, edges: Any, weights: Tensor, products: dict | None = None,
                       groups: tuple[Tensor, Tensor, Tensor] | None = None) -> Any:
    i = inputs(kernel, x, edges, products)
    order, group_ptr, group_source = groups_for(edges, i.source) if groups is None else groups
    flat = FactoredAggregate.apply(i.h, i.zc, i.zr, weights.to(i.h.dtype).contiguous(), i.angular, i.transport, i.rho, i.desc, i.source,
                                   edges.target_index.contiguous(), edges.row_ptr.contiguous(), order, group_ptr, group_source,
                                   i.plan.d_out, i.plan.max_bm)
    return _wrap_output(kernel, flat)
