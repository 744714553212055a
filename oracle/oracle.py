"""ctypes front end of the C oracle (``gm_oracle.c``) on numpy arrays.

TEST INFRASTRUCTURE ONLY (see ``gm_oracle.c``).  ``build()`` compiles the
library with gcc next to the source; every function takes C-contiguous numpy
arrays in float32 or float64 and returns numpy arrays.
"""

from __future__ import annotations

import ctypes
import functools
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIBRARY = HERE / "libgm_oracle.so"
SOURCES = [HERE / "gm_oracle.c", HERE / "gm_oracle_impl.h"]


def build(force: bool = False) -> Path:
    stamp = max(s.stat().st_mtime for s in SOURCES)
    if force or not LIBRARY.exists() or LIBRARY.stat().st_mtime < stamp:
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-ffp-contract=off", "-o", str(LIBRARY), str(SOURCES[0]), "-lm"], check=True)
    return LIBRARY


@functools.cache
def _lib() -> ctypes.CDLL:
    return ctypes.CDLL(str(build()))


def _suffix(dtype: np.dtype) -> str:
    return {np.dtype(np.float32): "_f32", np.dtype(np.float64): "_f64"}[np.dtype(dtype)]


def _p(a: np.ndarray | None) -> ctypes.c_void_p:
    if a is None or a.size == 0:
        return ctypes.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def _call(name: str, dtype: np.dtype, *args) -> None:
    fn = getattr(_lib(), name + _suffix(dtype))
    fn.restype = None
    real = ctypes.c_float if np.dtype(dtype) == np.float32 else ctypes.c_double
    converted = []
    for a in args:
        if isinstance(a, np.ndarray) or a is None:
            converted.append(_p(a))
        elif isinstance(a, float):
            converted.append(real(a))
        elif isinstance(a, tuple):  # ("i64", value)
            converted.append(ctypes.c_int64(a[1]))
        else:
            converted.append(ctypes.c_int(a))
    fn(*converted)


def _c(a, dtype=None) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def softmax_forward(q, k, transport, bias, inside, desc, row_ptr, source, heads, scale):
    dt = q.dtype
    q, k, transport, bias = _c(q), _c(k), _c(transport), _c(bias)
    inside, desc, row_ptr, source = _c(inside, np.uint8), _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    alpha = np.zeros((source.shape[0], heads), dt)
    _call("oracle_softmax_forward", dt, q, k, transport, bias, inside, desc, row_ptr, source, ("i64", q.shape[0]), q.shape[1],
          desc.shape[0], transport.shape[1], heads, float(scale), alpha)
    return alpha


def softmax_backward(dalpha, q, k, transport, desc, row_ptr, source, alpha, heads, scale):
    dt = q.dtype
    dalpha, q, k, transport, alpha = _c(dalpha), _c(q), _c(k), _c(transport), _c(alpha)
    desc, row_ptr, source = _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    dq, dk = np.zeros_like(q), np.zeros_like(q)
    _call("oracle_softmax_backward", dt, dalpha, q, k, transport, desc, row_ptr, source, alpha, ("i64", q.shape[0]), q.shape[1],
          desc.shape[0], transport.shape[1], heads, float(scale), dq, dk)
    return dq, dk


def conv_forward(v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, a0, w):
    dt = v.dtype
    v, rc, cc, transport, angular, rho, weights = map(_c, (v, rc, cc, transport, angular, rho, weights))
    desc, row_ptr, source = _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    out = np.zeros_like(v)
    _call("oracle_conv_forward", dt, v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, ("i64", v.shape[0]),
          v.shape[1], desc.shape[0], transport.shape[1], a0, w, out)
    return out


def conv_backward(g, v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, a0, w):
    dt = v.dtype
    g, v, rc, cc, transport, angular, rho, weights = map(_c, (g, v, rc, cc, transport, angular, rho, weights))
    desc, row_ptr, source = _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    dv, drc, dcc = np.zeros_like(v), np.zeros_like(rc), np.zeros_like(cc)
    _call("oracle_conv_backward", dt, g, v, rc, cc, transport, angular, rho, weights, desc, row_ptr, source, ("i64", v.shape[0]),
          v.shape[1], desc.shape[0], transport.shape[1], a0, w, dv, drc, dcc)
    return dv, drc, dcc


def attention_forward(q, k, v, transport, bias, inside, desc, row_ptr, source, heads, scale, batch=1):
    dt = q.dtype
    q, k, v, transport, bias = map(_c, (q, k, v, transport, bias))
    inside, desc, row_ptr, source = _c(inside, np.uint8), _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    n = row_ptr.shape[0] - 1
    assert q.shape[0] == n * batch
    alpha = np.zeros((source.shape[0], heads), dt)
    out = np.zeros_like(q)
    _call("oracle_attention_forward", dt, q, k, v, transport, bias, inside, desc, row_ptr, source, ("i64", n), ("i64", batch),
          q.shape[1], desc.shape[0], transport.shape[1], heads, float(scale), alpha, out)
    return out


def attention_backward(dout, q, k, v, transport, bias, inside, desc, row_ptr, source, heads, scale, batch=1):
    dt = q.dtype
    dout, q, k, v, transport, bias = map(_c, (dout, q, k, v, transport, bias))
    inside, desc, row_ptr, source = _c(inside, np.uint8), _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    n = row_ptr.shape[0] - 1
    alpha = np.zeros((source.shape[0], heads), dt)
    dalpha = np.zeros_like(alpha)
    dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(q)
    _call("oracle_attention_backward", dt, dout, q, k, v, transport, bias, inside, desc, row_ptr, source, ("i64", n),
          ("i64", batch), q.shape[1], desc.shape[0], transport.shape[1], heads, float(scale), alpha, dalpha, dq, dk, dv)
    return dq, dk, dv


def value_forward(alpha, v, transport, desc, row_ptr, source, heads):
    dt = v.dtype
    alpha, v, transport = _c(alpha), _c(v), _c(transport)
    desc, row_ptr, source = _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    out = np.zeros_like(v)
    _call("oracle_value_forward", dt, alpha, v, transport, desc, row_ptr, source, ("i64", v.shape[0]), v.shape[1], desc.shape[0],
          transport.shape[1], heads, out)
    return out


def value_backward(dout, alpha, v, transport, desc, row_ptr, source, heads):
    dt = v.dtype
    dout, alpha, v, transport = _c(dout), _c(alpha), _c(v), _c(transport)
    desc, row_ptr, source = _c(desc, np.int64), _c(row_ptr, np.int64), _c(source, np.int64)
    dalpha, dv = np.zeros_like(alpha), np.zeros_like(v)
    _call("oracle_value_backward", dt, dout, alpha, v, transport, desc, row_ptr, source, ("i64", v.shape[0]), v.shape[1],
          desc.shape[0], transport.shape[1], heads, dalpha, dv)
    return dalpha, dv
