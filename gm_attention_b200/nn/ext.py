"""Extension-module level of the operator interface.

The reference loads three pybind modules whose functions take and return
``torch.Tensor`` (``attention_cpu.cpp:256-261``, ``factored_cpu.cpp:223-234``,
``pairs_cpu.cpp:140-148``).  The classes here expose the same function names
and positional signatures, so an instance can stand where the reference's
``extension(cuda=True)`` result stands; each function validates its inputs
the way the reference's ``TORCH_CHECK``s do (``RuntimeError`` with the same
wording), allocates the outputs with torch on the inputs' device, and hands
raw device pointers to ``libgmb200.so`` on the current CUDA stream.
"""

from __future__ import annotations

import torch
from torch import Tensor

from gm_attention_b200 import _lib

MAX_F, DESC = 8, 5


def _check(condition: bool, message: str) -> None:
    if not condition:
        raise RuntimeError(message)


class AttentionExtension:
    """``conv_forward``, ``conv_backward``, ``softmax_forward``, ``softmax_backward``."""

    with_cuda = True

    # -- depthwise convolution -------------------------------------------------
    @staticmethod
    def _check_conv(v: Tensor, rc: Tensor, cc: Tensor, transport: Tensor, angular: Tensor, rho: Tensor, weights: Tensor,
                    desc: Tensor, row_ptr: Tensor, source: Tensor, a0: int, w: int) -> None:
        _check(v.dim() == 2, "v must be (n_nodes, D)")
        n, e = v.size(0), source.size(0)
        for t in (v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source):
            _check(t.is_contiguous(), "every tensor must be contiguous")
            _check(t.device == v.device, "every tensor must live on v's device")
        for t in (rc, cc, transport, angular, rho, weights):
            _check(t.dtype == v.dtype, "v, the coefficients, the weights and the tables must share a dtype")
        _check(rc.numel() == e * a0, "rc must hold (1, n_edges, a_0) entries")
        _check(cc.numel() == e * w, "cc must hold (1, n_edges, W) entries")
        _check(transport.dim() == 3 and transport.size(0) == e and transport.size(2) == 2, "transport must be (n_edges, orders, 2)")
        _check(angular.shape == transport.shape, "angular must match transport's shape")
        _check(rho.dim() == 1 and rho.size(0) == e and weights.shape == rho.shape, "rho and weights must be (n_edges,)")
        _check(desc.dtype == torch.int64 and desc.dim() == 2 and desc.size(1) == DESC and desc.size(0) <= MAX_F,
               f"desc must be int64 (F <= {MAX_F}, {DESC})")
        _check(row_ptr.dtype == torch.int64 and row_ptr.dim() == 1 and row_ptr.size(0) == n + 1, "row_ptr must be int64 (n_nodes + 1,)")
        _check(source.dtype == torch.int64 and source.dim() == 1, "source must be int64 (n_edges,)")
        _check(v.size(1) >= 1, "D must be positive")

    def conv_forward(self, v: Tensor, rc: Tensor, cc: Tensor, transport: Tensor, angular: Tensor, rho: Tensor, weights: Tensor,
                     desc: Tensor, row_ptr: Tensor, source: Tensor, a0: int, w: int) -> Tensor:
        self._check_conv(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, a0, w)
        out = torch.empty_like(v)
        if v.size(0) == 0:
            return out
        device = _lib.require_cuda(v)
        with torch.cuda.device(device):
            _lib.call("gm_conv_forward", _lib.ptr(v), _lib.ptr(rc), _lib.ptr(cc), _lib.ptr(transport), _lib.ptr(angular),
                      _lib.ptr(rho), _lib.ptr(weights), _lib.ptr(desc), _lib.ptr(row_ptr), _lib.ptr(source), v.size(0),
                      source.size(0), v.size(1), desc.size(0), transport.size(1), int(a0), int(w), _lib.dtype_code(v.dtype),
                      _lib.ptr(out), _lib.stream(device))
        return out

    def conv_backward(self, g: Tensor, v: Tensor, rc: Tensor, cc: Tensor, transport: Tensor, angular: Tensor, rho: Tensor,
                      weights: Tensor, desc: Tensor, row_ptr: Tensor, source: Tensor, a0: int, w: int) -> list[Tensor]:
        self._check_conv(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, a0, w)
        _check(g.shape == v.shape and g.is_contiguous() and g.dtype == v.dtype, "g must be contiguous, shaped and typed as v")
        dv = torch.zeros_like(v)
        drc = torch.empty_like(rc)
        dcc = torch.empty_like(cc)
        if v.size(0) == 0:
            return [dv, drc, dcc]
        device = _lib.require_cuda(v, g)
        with torch.cuda.device(device):
            _lib.call("gm_conv_backward", _lib.ptr(g), _lib.ptr(v), _lib.ptr(rc), _lib.ptr(cc), _lib.ptr(transport),
                      _lib.ptr(angular), _lib.ptr(rho), _lib.ptr(weights), _lib.ptr(desc), _lib.ptr(row_ptr), _lib.ptr(source),
                      v.size(0), source.size(0), v.size(1), desc.size(0), transport.size(1), int(a0), int(w),
                      _lib.dtype_code(v.dtype), _lib.ptr(dv), _lib.ptr(drc), _lib.ptr(dcc), _lib.stream(device))
        return [dv, drc, dcc]

    # -- scores + softmax --------------------------------------------------------
    @staticmethod
    def _check_softmax(q: Tensor, k: Tensor, transport: Tensor, bias: Tensor, inside: Tensor, desc: Tensor, row_ptr: Tensor,
                       source: Tensor, heads: int) -> None:
        _check(q.dim() == 2, "q must be (n_nodes, D)")
        n, e = q.size(0), source.size(0)
        for t in (q, k, transport, bias, inside, desc, row_ptr, source):
            _check(t.is_contiguous(), "every tensor must be contiguous")
            _check(t.device == q.device, "every tensor must live on q's device")
        for t in (k, transport, bias):
            _check(t.dtype == q.dtype, "q, k and the tables must share a dtype")
        _check(k.shape == q.shape, "q and k must share a shape")
        _check(1 <= heads <= 8, "at most 8 heads")
        _check(transport.dim() == 3 and transport.size(0) == e and transport.size(2) == 2, "transport must be (n_edges, orders, 2)")
        _check(bias.dim() == 1 and bias.size(0) == e, "bias must be (n_edges,)")
        _check(inside.dtype == torch.uint8 and inside.shape == bias.shape, "inside must be uint8 (n_edges,)")
        _check(desc.dtype == torch.int64 and desc.dim() == 2 and desc.size(1) == DESC and desc.size(0) <= MAX_F,
               f"desc must be int64 (F <= {MAX_F}, {DESC})")
        _check(row_ptr.dtype == torch.int64 and row_ptr.dim() == 1 and row_ptr.size(0) == n + 1, "row_ptr must be int64 (n_nodes + 1,)")
        _check(source.dtype == torch.int64 and source.dim() == 1, "source must be int64 (n_edges,)")
        _check(q.size(1) >= 1, "D must be positive")

    def softmax_forward(self, q: Tensor, k: Tensor, transport: Tensor, bias: Tensor, inside: Tensor, desc: Tensor, row_ptr: Tensor,
                        source: Tensor, heads: int, scale: float, deg_max: int) -> Tensor:
        self._check_softmax(q, k, transport, bias, inside, desc, row_ptr, source, heads)
        alpha = torch.empty((source.size(0), heads), dtype=q.dtype, device=q.device)
        if q.size(0) == 0 or source.size(0) == 0:
            return alpha
        device = _lib.require_cuda(q)
        with torch.cuda.device(device):
            _lib.call("gm_softmax_forward", _lib.ptr(q), _lib.ptr(k), _lib.ptr(transport), _lib.ptr(bias), _lib.ptr(inside),
                      _lib.ptr(desc), _lib.ptr(row_ptr), _lib.ptr(source), q.size(0), source.size(0), q.size(1), desc.size(0),
                      transport.size(1), int(heads), float(scale), int(deg_max), _lib.dtype_code(q.dtype), _lib.ptr(alpha),
                      _lib.stream(device))
        return alpha

    def softmax_backward(self, dalpha: Tensor, q: Tensor, k: Tensor, transport: Tensor, bias: Tensor, inside: Tensor, desc: Tensor,
                         row_ptr: Tensor, source: Tensor, alpha: Tensor, heads: int, scale: float, deg_max: int) -> list[Tensor]:
        self._check_softmax(q, k, transport, bias, inside, desc, row_ptr, source, heads)
        for t in (alpha, dalpha):
            _check(t.is_contiguous() and t.dim() == 2 and t.size(0) == source.size(0) and t.size(1) == heads and t.dtype == q.dtype,
                   "alpha and dalpha must be contiguous (n_edges, H) in q's dtype")
        dq = torch.empty_like(q)
        dk = torch.zeros_like(q)
        if q.size(0) == 0:
            return [dq, dk]
        device = _lib.require_cuda(q, alpha, dalpha)
        with torch.cuda.device(device):
            _lib.call("gm_softmax_backward", _lib.ptr(dalpha), _lib.ptr(q), _lib.ptr(k), _lib.ptr(transport), _lib.ptr(bias),
                      _lib.ptr(inside), _lib.ptr(desc), _lib.ptr(row_ptr), _lib.ptr(source), _lib.ptr(alpha), q.size(0),
                      source.size(0), q.size(1), desc.size(0), transport.size(1), int(heads), float(scale), int(deg_max),
                      _lib.dtype_code(q.dtype), _lib.ptr(dq), _lib.ptr(dk), _lib.stream(device))
        return [dq, dk]
