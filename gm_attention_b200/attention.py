"""The fully fused gauge-attention layer as one differentiable op.

``out_i = sum_e softmax_e(scale <q_i, tau(e) k_j> + bias_e) tau(e) v_j`` per
head: the composition of the reference's ``Softmax`` op
(``nn/fused_attention.py:371-397``) with its eager value path (transport the
gathered values, weight by alpha, segment-sum per target;
``nn/kernels.py:156-189``, ``nn/_scatter.py:36-46``).  Neither alpha nor any
per-edge field is materialised; the backward recomputes the logits from the
saved per-(node, head) log-sum-exp.

The geometry describes one sample; ``q, k, v`` are ``(batch * n_nodes, D)`` and
every sample shares the tables.  Node fields may be float32, float64 or
bfloat16 (bf16 storage, fp32 arithmetic; the tables are then float32).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

from gm_attention_b200 import _lib


@dataclass(frozen=True)
class AttentionTables:
    """Resident per-edge constants of one edge set (device tensors) plus the
    head layout in host memory."""

    transport: Tensor  # (E, orders, 2) fp32 / fp64
    bias: Tensor  # (E,)
    inside: Tensor  # (E,) uint8
    row_ptr: Tensor  # (N + 1,) int64
    source: Tensor  # (E,) int64
    rows: tuple[tuple[int, int, int, int, int], ...]  # descriptor rows (n, a_n, offset, coeff offset, dim)
    heads: int
    scale: float

    @property
    def n_nodes(self) -> int:
        return self.row_ptr.shape[0] - 1

    @property
    def n_edges(self) -> int:
        return self.source.shape[0]

    def host_descriptor(self) -> Any:
        flat = [x for row in self.rows for x in row]
        return (ctypes.c_int64 * len(flat))(*flat)


def _table_dtype(dtype: torch.dtype) -> torch.dtype:
    return torch.float64 if dtype == torch.float64 else torch.float32


def _check(q: Tensor, k: Tensor, v: Tensor, t: AttentionTables) -> tuple[torch.device, int]:
    device = _lib.require_cuda(q, k, v, t.transport, t.bias, t.inside, t.row_ptr, t.source)
    if not (q.dim() == 2 and q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype):
        raise RuntimeError("q, k and v must be (batch * n_nodes, D) tensors of one dtype")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise RuntimeError("q, k and v must be contiguous")
    if t.n_nodes == 0 or q.shape[0] % t.n_nodes:
        raise RuntimeError(f"the node fields hold {q.shape[0]} rows, not a multiple of the geometry's {t.n_nodes} nodes")
    want = _table_dtype(q.dtype)
    if t.transport.dtype != want or t.bias.dtype != want:
        raise RuntimeError(f"tables must be {want} for {q.dtype} node fields")
    if t.inside.dtype != torch.uint8 or t.row_ptr.dtype != torch.int64 or t.source.dtype != torch.int64:
        raise RuntimeError("inside must be uint8; row_ptr and source int64")
    return device, q.shape[0] // t.n_nodes


def attention_forward(q: Tensor, k: Tensor, v: Tensor, t: AttentionTables) -> tuple[Tensor, Tensor]:
    """``(out, lse)``: the layer's output ``(batch * n_nodes, D)`` and each row's log-sum-exp ``(batch * n_nodes, H)``."""
    device, batch = _check(q, k, v, t)
    out = torch.empty_like(q)
    lse = torch.empty((q.shape[0], t.heads), dtype=_table_dtype(q.dtype), device=device)
    desc = t.host_descriptor()
    with torch.cuda.device(device):
        _lib.call("gm_attention_forward", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(t.transport), _lib.ptr(t.bias),
                  _lib.ptr(t.inside), ctypes.addressof(desc), _lib.ptr(t.row_ptr), _lib.ptr(t.source), t.n_nodes, t.n_edges, batch,
                  q.shape[1], len(t.rows), t.transport.shape[1], t.heads, float(t.scale), _lib.dtype_code(q.dtype), _lib.ptr(out),
                  _lib.ptr(lse), _lib.stream(device))
    return out, lse


def attention_backward(dout: Tensor, q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor,
                       t: AttentionTables) -> tuple[Tensor, Tensor, Tensor]:
    device, batch = _check(q, k, v, t)
    dout = dout.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    code = _lib.dtype_code(q.dtype)
    need = _lib.lib().gm_attention_backward_scratch_bytes(t.n_nodes, batch, q.shape[1], code)
    scratch = torch.empty(need, dtype=torch.uint8, device=device) if need else None
    desc = t.host_descriptor()
    with torch.cuda.device(device):
        _lib.call("gm_attention_backward", _lib.ptr(dout), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse),
                  _lib.ptr(t.transport), _lib.ptr(t.bias), _lib.ptr(t.inside), ctypes.addressof(desc), _lib.ptr(t.row_ptr),
                  _lib.ptr(t.source), t.n_nodes, t.n_edges, batch, q.shape[1], len(t.rows), t.transport.shape[1], t.heads,
                  float(t.scale), code, _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(scratch), _lib.stream(device))
    return dq, dk, dv


class GaugeAttention(torch.autograd.Function):
    """``GaugeAttention.apply(q, k, v, tables) -> out``."""

    @staticmethod
    def forward(ctx: Any, q: Tensor, k: Tensor, v: Tensor, tables: AttentionTables) -> Tensor:
        with torch.profiler.record_function("gm::attention/fused"):
            out, lse = attention_forward(q.contiguous(), k.contiguous(), v.contiguous(), tables)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.tables = tables
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_out: Tensor) -> tuple:  # type: ignore[override]
        q, k, v, out, lse = ctx.saved_tensors
        with torch.profiler.record_function("gm::attention/fused_backward"):
            dq, dk, dv = attention_backward(grad_out, q.contiguous(), k.contiguous(), v.contiguous(), out, lse, ctx.tables)
        return dq, dk, dv, None
