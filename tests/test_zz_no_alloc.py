"""The allocation-free backward entry point, gm_attention_backward_static.

It exists for embedders that cannot allocate device memory at call time (all
of HBM committed to their own arena at start-up; loops that must stay off the
driver's allocator): the fp32 accumulation buffer of the bf16 backward lives in
a fixed array inside the library instead of being passed in.  The test drives
both entry points through the C ABI on the same inputs and requires the same
gradients, twice in a row (the shared array keeps the first call's sums, so the
second call proves it is cleared), and checks that an oversized problem is
refused with a message rather than run.

Collected last on purpose: a failure here cannot hide any other test's result
from a run that stops at the first failure.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import pytest
import torch

from tests.helpers import cuda, make_case, seeded

pytestmark = pytest.mark.gpu


def _backward(entry: str, tensors, tables, case, batch, scratch=None):
    from gm_attention_b200 import _lib

    dout, q, k, v, out, lse = tensors
    dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
    flat = [int(x) for row in case.desc for x in row]
    desc = (ctypes.c_int64 * len(flat))(*flat)
    transport, bias, inside, row_ptr, source = tables
    args = [_lib.ptr(dout), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(transport), _lib.ptr(bias),
            _lib.ptr(inside), ctypes.addressof(desc), _lib.ptr(row_ptr), _lib.ptr(source), case.n_nodes, source.shape[0], batch,
            q.shape[1], len(case.desc), transport.shape[1], case.heads, float(case.scale), _lib.dtype_code(q.dtype), _lib.ptr(dq),
            _lib.ptr(dk), _lib.ptr(dv)]
    if entry == "gm_attention_backward":
        args.append(_lib.ptr(scratch))
    args.append(_lib.stream(q.device))
    _lib.call(entry, *args)
    torch.cuda.synchronize()
    return dq, dk, dv


def test_static_backward_equals_the_allocating_entry_point_twice():
    from gm_attention_b200 import _lib
    from gm_attention_b200.attention import AttentionTables, attention_forward

    batch = 2
    case = make_case(12, 24, 3 * math.pi / 12, {0: 16, 1: 16, 2: 16}, 4, dtype=np.float32)
    tables = tuple(cuda(x) for x in (case.transport, case.bias, case.inside, case.row_ptr, case.source))
    t = AttentionTables(*tables, tuple(tuple(int(x) for x in row) for row in case.desc), case.heads, case.scale)
    for seed in (7, 8):  # two calls in a row on different data
        q, k, v, g = (torch.from_numpy(x).bfloat16().cuda() for x in seeded((batch * case.n_nodes, case.width), seed, np.float32, 4))
        out, lse = attention_forward(q, k, v, t)
        need = _lib.lib().gm_attention_backward_scratch_bytes(case.n_nodes, batch, case.width, _lib.GM_BF16)
        assert 0 < need <= _lib.lib().gm_attention_backward_static_capacity()
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        want = _backward("gm_attention_backward", (g, q, k, v, out, lse), tables, case, batch, scratch)
        _backward("gm_attention_backward_static", (g, q, k, v, out, lse), tables, case, batch)  # first call on the device: image loaded, address resolved
        free_before, _ = torch.cuda.mem_get_info()
        got = _backward("gm_attention_backward_static", (g, q, k, v, out, lse), tables, case, batch)
        free_after, _ = torch.cuda.mem_get_info()
        # the outputs of _backward come from torch's caching allocator (blocks it already holds after the call above);
        # the entry point itself must not have taken anything from the driver
        assert free_after == free_before, "the allocation-free entry point changed the device's free memory"
        for name, a, b in zip(("dq", "dk", "dv"), got, want):
            a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
            assert np.isfinite(a).all(), name
            # same kernels, same inputs: only the order of the atomic sums differs (2e-2 relative is the bf16 bar)
            assert np.abs(a - b).max() <= 2e-2 * max(1.0, np.abs(b).max()), name


def test_static_backward_refuses_problems_beyond_its_buffer():
    from gm_attention_b200 import _lib

    handle = _lib.lib()
    capacity = handle.gm_attention_backward_static_capacity()
    d, n = 320, capacity // (2 * 4 * 320) + 1  # one node too many
    status = handle.gm_attention_backward_static(*([None] * 12), n, 0, 1, d, 1, 1, 4, 1.0, _lib.GM_BF16, None, None, None, None)
    assert status == -4
    message = handle.gm_last_error().decode()
    assert "built-in buffer" in message and "gm_attention_backward" in message
