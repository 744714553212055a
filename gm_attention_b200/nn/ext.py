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

    def __init__(self) -> None:
        #: largest multiplicity of a descriptor tensor, read back from the device once per tensor
        self._max_mult: dict[tuple[int, int], tuple[object, int]] = {}

    def _largest_multiplicity(self, desc: Tensor) -> int:
        key = (desc.data_ptr(), desc.size(0))
        hit = self._max_mult.get(key)
        if hit is not None and hit[0]() is desc:
            return hit[1]
        import weakref

        value = int(desc[:, 1].max()) if desc.size(0) else 0
        if len(self._max_mult) > 256:
            self._max_mult.clear()
        self._max_mult[key] = (weakref.ref(desc), value)
        return value

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
                      transport.size(1), int(heads), float(scale), int(deg_max), self._largest_multiplicity(desc),
                      _lib.dtype_code(q.dtype), _lib.ptr(alpha), _lib.stream(device))
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


MAX_K, MAX_OUT, MAX_BM, FDESC = 20, 128, 32, 8
#: the reference bounds the packed width 2 wc + wr by 320; here only k * (2 wc + wr) is bounded
MAX_KC = 8192


def _fcheck(condition: bool, message: str) -> None:
    if not condition:
        raise RuntimeError("gm_factored: " + message)


class FactoredExtension:
    """``forward``, ``aggregate``, ``backward``, ``backward_aggregated``."""

    with_cuda = True

    @staticmethod
    def _check_common(h: Tensor, zc: Tensor, zr: Tensor, angular: Tensor, transport: Tensor, rho: Tensor, desc: Tensor, source: Tensor,
                      d_out: int) -> None:
        _fcheck(h.dim() == 2 and h.is_contiguous(), "h must be a contiguous (n_edges, k - 1) tensor")
        _fcheck(zc.dim() == 4 and zc.size(3) == 2 and zc.is_contiguous(), "zc must be a contiguous (n_nodes, k, wc, 2) tensor")
        _fcheck(zr.dim() == 3 and zr.is_contiguous(), "zr must be a contiguous (n_nodes, k, wr) tensor")
        _fcheck(zc.size(1) == h.size(1) + 1 and zr.size(1) == h.size(1) + 1, "zc and zr must have k = h's width + 1 (the constant feature)")
        _fcheck(zc.size(0) == zr.size(0), "zc and zr must have the same node count")
        _fcheck(angular.dim() == 3 and angular.size(2) == 2 and angular.is_contiguous() and angular.size(0) == h.size(0),
                "angular must be a contiguous (n_edges, n_f, 2) tensor")
        _fcheck(transport.shape == angular.shape and transport.is_contiguous(), "transport must match angular")
        _fcheck(rho.dim() == 1 and rho.is_contiguous() and rho.size(0) == h.size(0), "rho must be a contiguous (n_edges,) tensor")
        _fcheck(desc.dim() == 2 and desc.size(1) == FDESC and desc.dtype == torch.int32 and desc.is_contiguous(),
                "desc must be a contiguous int32 (n_blocks, 8) tensor")
        _fcheck(source.dim() == 1 and source.size(0) == h.size(0) and source.dtype == torch.int64 and source.is_contiguous(),
                "source must be a contiguous int64 (n_edges,) tensor")
        _fcheck(h.size(1) + 1 <= MAX_K, "k exceeds MAX_K")
        _fcheck(1 <= d_out <= MAX_OUT, "d_out must be in [1, MAX_OUT]")
        _fcheck((h.size(1) + 1) * (2 * zc.size(2) + zr.size(2)) <= MAX_KC, "k (2 wc + wr) exceeds the kernels' bound")
        for t in (zc, zr, angular, transport, rho):
            _fcheck(t.dtype == h.dtype, "every floating tensor must share h's dtype")
            _fcheck(t.device == h.device, "every tensor must be on h's device")
        _fcheck(desc.device == h.device and source.device == h.device, "desc and source must be on h's device")

    @staticmethod
    def _sizes(h: Tensor, zc: Tensor, zr: Tensor, angular: Tensor, desc: Tensor, group_source: Tensor) -> tuple:
        return (h.size(0), group_source.size(0), h.size(1) + 1, zc.size(2), zr.size(2), angular.size(1), desc.size(0))

    def forward(self, h: Tensor, zc: Tensor, zr: Tensor, angular: Tensor, transport: Tensor, rho: Tensor, desc: Tensor, source: Tensor,
                order: Tensor, group_ptr: Tensor, group_source: Tensor, d_out: int, max_bm: int) -> Tensor:
        self._check_common(h, zc, zr, angular, transport, rho, desc, source, d_out)
        out = torch.empty((h.size(0), d_out), dtype=h.dtype, device=h.device)
        _fcheck(1 <= max_bm <= MAX_BM, "max_bm must be in [1, MAX_BM]")
        if h.size(0) == 0:
            return out
        device = _lib.require_cuda(h, order, group_ptr, group_source)
        with torch.cuda.device(device):
            _lib.call("gm_factored_forward", _lib.ptr(h), _lib.ptr(zc), _lib.ptr(zr), _lib.ptr(angular), _lib.ptr(transport), _lib.ptr(rho),
                      _lib.ptr(desc), _lib.ptr(source), _lib.ptr(order.contiguous()), _lib.ptr(group_ptr.contiguous()),
                      _lib.ptr(group_source.contiguous()), *self._sizes(h, zc, zr, angular, desc, group_source), int(d_out),
                      _lib.dtype_code(h.dtype), _lib.ptr(out), _lib.stream(device))
        return out

    def aggregate(self, rows: Tensor, weights: Tensor, row_ptr: Tensor) -> Tensor:
        _fcheck(rows.dim() == 2 and rows.is_contiguous() and 1 <= rows.size(1) <= MAX_OUT,
                "rows must be a contiguous (n_edges, d_out <= MAX_OUT) tensor")
        _fcheck(weights.dim() == 1 and weights.is_contiguous() and weights.size(0) == rows.size(0) and weights.dtype == rows.dtype,
                "weights must be a contiguous (n_edges,) tensor in the rows' dtype")
        _fcheck(row_ptr.dim() == 1 and row_ptr.is_contiguous() and row_ptr.size(0) >= 1 and row_ptr.dtype == torch.int64,
                "row_ptr must be a contiguous int64 (n_targets + 1,) tensor")
        _fcheck(weights.device == rows.device and row_ptr.device == rows.device, "every tensor must be on the rows' device")
        n_targets = row_ptr.size(0) - 1
        out = torch.empty((n_targets, rows.size(1)), dtype=rows.dtype, device=rows.device)
        if n_targets == 0:
            return out
        device = _lib.require_cuda(rows)
        with torch.cuda.device(device):
            _lib.call("gm_factored_aggregate", _lib.ptr(rows), _lib.ptr(weights), _lib.ptr(row_ptr), n_targets, rows.size(0), rows.size(1),
                      _lib.dtype_code(rows.dtype), _lib.ptr(out), _lib.stream(device))
        return out

    def _backward(self, g: Tensor, target: Tensor | None, weights: Tensor | None, rows: Tensor | None, h: Tensor, zc: Tensor, zr: Tensor,
                  angular: Tensor, transport: Tensor, rho: Tensor, desc: Tensor, source: Tensor, order: Tensor, group_ptr: Tensor,
                  group_source: Tensor) -> list[Tensor]:
        _fcheck(g.dim() == 2 and g.is_contiguous() and g.dtype == h.dtype and g.device == h.device,
                "g must be a contiguous (rows, d_out) tensor in h's dtype")
        self._check_common(h, zc, zr, angular, transport, rho, desc, source, g.size(1))
        aggregated = target is not None and target.numel() > 0
        if aggregated:
            _fcheck(target.dim() == 1 and target.size(0) == h.size(0) and target.dtype == torch.int64 and target.is_contiguous()
                    and target.device == h.device, "target must be a contiguous int64 (n_edges,) tensor")
            _fcheck(weights.dim() == 1 and weights.size(0) == h.size(0) and weights.is_contiguous() and weights.dtype == h.dtype
                    and weights.device == h.device, "weights must be a contiguous (n_edges,) tensor in h's dtype")
            _fcheck(rows.dim() == 2 and rows.size(0) == h.size(0) and rows.size(1) == g.size(1) and rows.is_contiguous()
                    and rows.dtype == h.dtype and rows.device == h.device, "rows must be a contiguous (n_edges, d_out) tensor in h's dtype")
        else:
            _fcheck(g.size(0) == h.size(0), "g must have one row per edge")
        dh = torch.empty_like(h)
        dzc = torch.zeros_like(zc)
        dzr = torch.zeros_like(zr)
        dweights = torch.empty_like(weights) if aggregated else None
        if h.size(0) == 0:
            return [dh, dzc, dzr, dweights]
        device = _lib.require_cuda(h, g, order, group_ptr, group_source)
        with torch.cuda.device(device):
            _lib.call("gm_factored_backward", _lib.ptr(g), _lib.ptr(target) if aggregated else None, _lib.ptr(weights) if aggregated else None,
                      _lib.ptr(rows) if aggregated else None, _lib.ptr(h), _lib.ptr(zc), _lib.ptr(zr), _lib.ptr(angular), _lib.ptr(transport),
                      _lib.ptr(rho), _lib.ptr(desc), _lib.ptr(source), _lib.ptr(order.contiguous()), _lib.ptr(group_ptr.contiguous()),
                      _lib.ptr(group_source.contiguous()), *self._sizes(h, zc, zr, angular, desc, group_source), g.size(1),
                      _lib.dtype_code(h.dtype), _lib.ptr(dh), _lib.ptr(dzc), _lib.ptr(dzr), _lib.ptr(dweights), _lib.stream(device))
        return [dh, dzc, dzr, dweights]

    def backward(self, g: Tensor, h: Tensor, zc: Tensor, zr: Tensor, angular: Tensor, transport: Tensor, rho: Tensor, desc: Tensor,
                 source: Tensor, order: Tensor, group_ptr: Tensor, group_source: Tensor) -> list[Tensor]:
        return self._backward(g, None, None, None, h, zc, zr, angular, transport, rho, desc, source, order, group_ptr, group_source)[:3]

    def backward_aggregated(self, g: Tensor, target: Tensor, weights: Tensor, rows: Tensor, h: Tensor, zc: Tensor, zr: Tensor,
                            angular: Tensor, transport: Tensor, rho: Tensor, desc: Tensor, source: Tensor, order: Tensor,
                            group_ptr: Tensor, group_source: Tensor) -> list[Tensor]:
        if h.size(0) == 0:
            return [torch.empty_like(h), torch.zeros_like(zc), torch.zeros_like(zr), torch.empty_like(weights)]
        _fcheck(target.numel() == h.size(0), "target must list every edge")
        return self._backward(g, target, weights, rows, h, zc, zr, angular, transport, rho, desc, source, order, group_ptr, group_source)


MATRIX_COMPLEX, U_REAL, CONJ_U, OUT_REAL = 1, 2, 4, 8


def _pcheck(condition: bool, message: str) -> None:
    if not condition:
        raise RuntimeError("gm_pairs: " + message)


def _as_real(t: Tensor) -> Tensor:
    return torch.view_as_real(t) if t.is_complex() else t


class PairsExtension:
    """``forward`` (accumulates into ``out``) and ``backward`` (accumulates ``grad_u``,
    ``grad_hidden``; writes ``grad_k``).  Absent ``bias`` / ``pre`` / ``post`` / ``scale`` are empty tensors."""

    with_cuda = True

    @staticmethod
    def _check(hidden: Tensor, weight: Tensor, u: Tensor, out: Tensor, a: int, b: int, flags: int) -> None:
        trunk = hidden.size(1)
        _pcheck(1 <= a <= 16 and 1 <= b <= 16, "block dimensions must be in 1..16")
        _pcheck(1 <= trunk <= 16, "trunk width must be in 1..16")
        _pcheck(hidden.is_contiguous() and weight.is_contiguous() and u.is_contiguous() and out.is_contiguous(),
                "hidden, weight, u and out must be contiguous")
        width = (2 if flags & MATRIX_COMPLEX else 1) * a * b
        _pcheck(weight.size(0) == width and weight.size(1) == trunk, "weight must be (width, trunk)")
        _pcheck(u.size(1) == a and out.size(1) == b, "u must be (n_edges, a) and out (n_edges, b)")
        _pcheck(u.size(0) == hidden.size(0) and out.size(0) == hidden.size(0), "n_edges mismatch")
        _pcheck(bool(flags & U_REAL) == (not u.is_complex()), "u must be real iff U_REAL")
        _pcheck(bool(flags & OUT_REAL) == (not out.is_complex()), "out must be real iff OUT_REAL")

    def forward(self, hidden: Tensor, weight: Tensor, bias: Tensor, u: Tensor, pre: Tensor, post: Tensor, scale: Tensor, out: Tensor,
                a: int, b: int, flags: int) -> None:
        self._check(hidden, weight, u, out, a, b, flags)
        if hidden.size(0) == 0:
            return
        device = _lib.require_cuda(hidden, weight, u, out)
        with torch.cuda.device(device):
            _lib.call("gm_pairs_forward", _lib.ptr(hidden), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(_as_real(u)), _lib.ptr(_as_real(pre)),
                      _lib.ptr(_as_real(post)), _lib.ptr(scale), _lib.ptr(_as_real(out)), hidden.size(0), int(a), int(b), hidden.size(1),
                      int(flags), _lib.dtype_code(hidden.dtype), _lib.stream(device))

    def backward(self, hidden: Tensor, weight: Tensor, bias: Tensor, u: Tensor, pre: Tensor, post: Tensor, scale: Tensor, grad_out: Tensor,
                 grad_u: Tensor, grad_hidden: Tensor, grad_k: Tensor, a: int, b: int, flags: int) -> None:
        self._check(hidden, weight, u, grad_out, a, b, flags)
        _pcheck(grad_u.is_contiguous() and grad_hidden.is_contiguous(), "grad_u and grad_hidden must be contiguous")
        width = (2 if flags & MATRIX_COMPLEX else 1) * a * b
        _pcheck(grad_k.is_contiguous() and grad_k.size(1) == hidden.size(0) and grad_k.size(0) == width,
                "grad_k must be (width, n_edges), contiguous")
        if hidden.size(0) == 0:
            return
        device = _lib.require_cuda(hidden, weight, u, grad_out, grad_u, grad_hidden, grad_k)
        with torch.cuda.device(device):
            _lib.call("gm_pairs_backward", _lib.ptr(hidden), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(_as_real(u)), _lib.ptr(_as_real(pre)),
                      _lib.ptr(_as_real(post)), _lib.ptr(scale), _lib.ptr(_as_real(grad_out)), _lib.ptr(_as_real(grad_u)),
                      _lib.ptr(grad_hidden), _lib.ptr(grad_k), hidden.size(0), int(a), int(b), hidden.size(1), int(flags),
                      _lib.dtype_code(hidden.dtype), _lib.stream(device))
