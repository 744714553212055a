"""numpy restatement of the reference's pair-term and factored-kernel arithmetic (TEST INFRASTRUCTURE, not product).

Only ``tests/`` import this module.  Every function states the reference lines it follows
(paths inside masonfaldet/gm-attention); the restatement is pinned against the reference's own
compiled CPU drivers (``oracle/_ref``) by ``tests/test_oracle_cpu.py``.

Conventions: complex tensors are numpy complex arrays; ``flags`` are the reference's
(``src/gm_attention/nn/fused/pairs.h:83-86``): MATRIX_COMPLEX = 1, U_REAL = 2, CONJ_U = 4, OUT_REAL = 8.
"""

from __future__ import annotations

import numpy as np

MATRIX_COMPLEX, U_REAL, CONJ_U, OUT_REAL = 1, 2, 4, 8


def _pair_matrix(hidden: np.ndarray, weight: np.ndarray, bias: np.ndarray | None, a: int, b: int, flags: int) -> np.ndarray:
    """M(e) = W h(e) + b as (E, b, a), complex or real (``pairs.h:201-238``: rows 2 idx / 2 idx + 1 are the real /
    imaginary parts of entry idx = bi * a + x of a complex matrix; row idx of a real one)."""
    rows = hidden @ weight.T  # (E, width)
    if bias is not None:
        rows = rows + bias
    if flags & MATRIX_COMPLEX:
        m = rows[:, 0::2] + 1j * rows[:, 1::2]
    else:
        m = rows
    return m.reshape(hidden.shape[0], b, a)


def _transported_input(u: np.ndarray, pre: np.ndarray | None, flags: int) -> np.ndarray:
    """uu = pre * u~ with u~ = u, or conj(u) under CONJ_U; a real u stays real-valued in u~ (``pairs.h:240-262``)."""
    ut = u.astype(np.complex128 if u.dtype in (np.float64, np.complex128) else np.complex64)
    if (flags & CONJ_U) and not (flags & U_REAL):
        ut = np.conj(ut)
    if pre is not None:
        ut = pre[:, None] * ut
    return ut


def pairs_forward(hidden, weight, bias, u, pre, post, scale, out, a: int, b: int, flags: int) -> np.ndarray:
    """out(e) += post(e) * f(M(e) (pre(e) u~(e))), f = identity or real part; the real per-edge scale rides on post
    (``pairs.h:301-330``, driver ``pairs_cpu.cpp:88-106``).  Returns the updated ``out`` (a copy)."""
    m = _pair_matrix(hidden, weight, bias, a, b, flags)
    uu = _transported_input(u, pre, flags)
    acc = np.einsum("eba,ea->eb", m, uu)
    s = np.ones(hidden.shape[0], hidden.dtype) if scale is None else scale
    if flags & OUT_REAL:
        return out + acc.real * s[:, None]
    q = s if post is None else post * s
    return out + q[:, None] * acc


def pairs_backward(hidden, weight, bias, u, pre, post, scale, grad_out, grad_u, grad_hidden, a: int, b: int, flags: int):
    """Backward of :func:`pairs_forward` (``pairs.h:332-365``, driver ``pairs_cpu.cpp:108-136``): returns
    ``(grad_u + d u, grad_hidden + d hidden, grad_k)`` with ``grad_k`` the coefficient gradient ``(width, E)``."""
    e = hidden.shape[0]
    m = _pair_matrix(hidden, weight, bias, a, b, flags)
    uu = _transported_input(u, pre, flags)
    s = np.ones(e, hidden.dtype) if scale is None else scale
    if flags & OUT_REAL:
        gq = (grad_out * s[:, None]).astype(uu.dtype)
    else:
        q = s if post is None else post * s
        gq = np.conj(q)[:, None] * grad_out  # dL/d(M uu)
    gm = gq[:, :, None] * np.conj(uu)[:, None, :]  # (E, b, a): gradient of the matrix entries
    guu = np.einsum("eba,eb->ea", np.conj(m), gq)
    gm_flat = gm.reshape(e, a * b)
    if flags & MATRIX_COMPLEX:
        rows = np.empty((e, 2 * a * b), hidden.dtype)
        rows[:, 0::2], rows[:, 1::2] = gm_flat.real, gm_flat.imag
    else:
        rows = np.ascontiguousarray(gm_flat.real).astype(hidden.dtype)
    grad_k = rows.T.copy()
    d_hidden = rows @ weight
    gu = guu if pre is None else np.conj(pre)[:, None] * guu
    if flags & U_REAL:
        d_u = gu.real.astype(u.dtype)
    else:
        d_u = (np.conj(gu) if flags & CONJ_U else gu).astype(u.dtype)
    return grad_u + d_u, grad_hidden + d_hidden.astype(hidden.dtype), grad_k


# ----------------------------------------------------------------------------- factored steerable kernel

def _block_factor(angular: np.ndarray, transport: np.ndarray, rho: np.ndarray, ang: int, trn: int, power: int) -> np.ndarray:
    """F_b(e) = e^{i ang phi} e^{i trn gamma} (r / c)^power per edge; negative orders are conjugates, the power is a
    repeated product starting from 1 (``src/gm_attention/nn/fused/factored.h:118-144``)."""
    f = np.ones(rho.shape[0], np.complex128 if rho.dtype == np.float64 else np.complex64)
    for table, order in ((angular, ang), (transport, trn)):
        if order != 0:
            p = table[:, abs(order), 0] + 1j * table[:, abs(order), 1]
            f = f * (np.conj(p) if order < 0 else p)
    s = np.ones_like(rho)
    for _ in range(power):
        s = s * rho
    return f * s


def factored_forward(h, zc, zr, angular, transport, rho, desc, source, d_out: int) -> np.ndarray:
    """rows (E, d_out): row_e = sum over blocks of F_b(e) * sum_t h~_t(e) Z_{t,b}(source_e), h~ = (1, h); blocks that
    share an output offset add up, rows n -> 0 keep the real part (``factored.h:158-250``, driver
    ``factored_cpu.cpp:77-109``).  ``desc`` rows: (kind, z_off, b_m, ang, trn, power, out_off, take_real)."""
    e = source.shape[0]
    ht = np.concatenate([np.ones((e, 1), h.dtype), h], axis=1)  # (E, K)
    rows = np.zeros((e, d_out), h.dtype)
    for kind, zoff, bm, ang, trn, power, ooff, take_real in desc.tolist():
        if kind == 0:
            rows[:, ooff:ooff + bm] += np.einsum("et,etc->ec", ht, zr[source][:, :, zoff:zoff + bm])
            continue
        z = zc[source][:, :, zoff:zoff + bm]
        u = np.einsum("et,etc->ec", ht, z[..., 0] + 1j * z[..., 1])
        v = _block_factor(angular, transport, rho, ang, trn, power)[:, None] * u
        if take_real:
            rows[:, ooff:ooff + bm] += v.real
        else:
            rows[:, ooff:ooff + 2 * bm:2] += v.real
            rows[:, ooff + 1:ooff + 2 * bm:2] += v.imag
    return rows


def factored_aggregate(rows, weights, row_ptr) -> np.ndarray:
    """out_i = sum over the edges of target i of w_e row_e (``factored.h:337-347``, ``factored_cpu.cpp:113-138``)."""
    out = np.zeros((row_ptr.shape[0] - 1, rows.shape[1]), rows.dtype)
    weighted = rows * weights[:, None]
    for i in range(out.shape[0]):
        out[i] = weighted[row_ptr[i]:row_ptr[i + 1]].sum(0)
    return out


def factored_backward(g, h, zc, zr, angular, transport, rho, desc, source, target=None, weights=None, rows=None):
    """(dh, dzc, dzr[, dweights]).  Per edge the packed row W(e) = scale * G conj(F_b); dh_t(e) = <W(e), Z_t(j)> for
    t >= 1 and dZ_t(j) = sum over the edges leaving j of h~_t(e) W(e) (``factored.h:254-334``,
    ``factored_cpu.cpp:140-219``).  Plain form: G = g[e].  Aggregated form (``target`` given): G = w_e g[target_e] and
    dweights_e = <g[target_e], row_e>."""
    e = source.shape[0]
    ht = np.concatenate([np.ones((e, 1), h.dtype), h], axis=1)
    ge = g if target is None else g[target] * weights[:, None]
    wc_pack = np.zeros((e, zc.shape[2]), np.complex128 if h.dtype == np.float64 else np.complex64)
    wr_pack = np.zeros((e, zr.shape[2]), h.dtype)
    for kind, zoff, bm, ang, trn, power, ooff, take_real in desc.tolist():
        if kind == 0:
            wr_pack[:, zoff:zoff + bm] += ge[:, ooff:ooff + bm]
            continue
        gc = ge[:, ooff:ooff + bm].astype(wc_pack.dtype) if take_real else ge[:, ooff:ooff + 2 * bm:2] + 1j * ge[:, ooff + 1:ooff + 2 * bm:2]
        wc_pack[:, zoff:zoff + bm] += gc * np.conj(_block_factor(angular, transport, rho, ang, trn, power))[:, None]
    zcs = zc[source]
    zcs = zcs[..., 0] + 1j * zcs[..., 1]  # (E, K, wc)
    dh_all = np.einsum("ec,etc->et", wc_pack.real, zcs.real) + np.einsum("ec,etc->et", wc_pack.imag, zcs.imag) + np.einsum("ec,etc->et", wr_pack, zr[source])
    dh = dh_all[:, 1:].astype(h.dtype)
    dzc = np.zeros_like(zc)
    dzr = np.zeros_like(zr)
    contrib_c = ht[:, :, None] * wc_pack[:, None, :]
    np.add.at(dzc[..., 0], source, contrib_c.real)
    np.add.at(dzc[..., 1], source, contrib_c.imag)
    np.add.at(dzr, source, ht[:, :, None] * wr_pack[:, None, :])
    if target is None:
        return dh, dzc, dzr
    return dh, dzc, dzr, (g[target] * rows).sum(1)
