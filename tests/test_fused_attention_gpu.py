"""Parity of the fully fused gauge-attention layer (forward + backward) with
the oracle "reference fused Softmax (CPU) + reference eager transport /
segment-sum", on seeded inputs and on the golden fixtures the reference's
Python produced.

Tolerances: float64 1e-10; float32 1e-5 relative / 1e-6 absolute (absolute
part scaled by the tensor's magnitude for gradients); bf16 storage with fp32
accumulation 2e-2 relative to the tensor's magnitude, against the oracle run
in float32 on the bf16-rounded inputs."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import oracle as O

from tests.helpers import assert_close, cuda, make_case, rel_err, seeded

pytestmark = pytest.mark.gpu

CASES = [
    (8, 16, 2 * math.pi / 8, {0: 3, 1: 2, 2: 1}, 2, "hard", 2),
    (8, 16, 2.5 * math.pi / 8, {0: 2, 1: 2}, 4, "quartic", 1),
    (6, 12, 2 * math.pi / 6, {1: 3, 3: 2}, 1, "hard", 3),
    (16, 32, 2 * math.pi / 16, {0: 4, 1: 4, 2: 4}, 2, "hard", 2),
    (12, 24, 3 * math.pi / 12, {0: 16, 1: 16, 2: 16}, 4, "hard", 1),  # the headline head type 16 x (m = 0, 1, 2), H = 4
    (8, 16, 2 * math.pi / 8, {0: 1, 1: 9}, 8, "quartic", 1),
]


def tables_for(c, dtype):
    from gm_attention_b200.attention import AttentionTables

    tdt = np.float64 if dtype == np.float64 else np.float32
    return AttentionTables(cuda(c.transport.astype(tdt)), cuda(c.bias.astype(tdt)), cuda(c.inside), cuda(c.row_ptr), cuda(c.source),
                           tuple(tuple(int(x) for x in row) for row in c.desc), c.heads, c.scale)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", CASES)
def test_fused_attention_matches_oracle(case, dtype):
    from gm_attention_b200.attention import attention_backward, attention_forward

    batch = case[6]
    c = make_case(*case[:5], dtype=dtype, window=case[5])
    q, k, v, g = seeded((batch * c.n_nodes, c.width), 31, dtype, 4)
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    dq_w, dk_w, dv_w = O.attention_backward(g, q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    t = tables_for(c, dtype)
    Q, K, V, G = cuda(q), cuda(k), cuda(v), cuda(g)
    out, lse = attention_forward(Q, K, V, t)
    rtol, atol = (1e-10, 1e-11) if dtype == np.float64 else (1e-5, 1e-6)
    assert_close(out.cpu().numpy(), want, rtol, atol * max(1.0, np.abs(want).max()), "out")
    dq, dk, dv = attention_backward(G, Q, K, V, out, lse, t)
    for name, got, ref in (("dq", dq, dq_w), ("dk", dk, dk_w), ("dv", dv, dv_w)):
        assert_close(got.cpu().numpy(), ref, rtol, 10 * atol * max(1.0, np.abs(ref).max()), name)


@pytest.mark.parametrize("case", CASES[:5])
def test_fused_attention_bf16_storage(case):
    from gm_attention_b200.attention import attention_backward, attention_forward

    batch = case[6]
    c = make_case(*case[:5], dtype=np.float32, window=case[5])
    rounded = [torch.from_numpy(x).bfloat16() for x in seeded((batch * c.n_nodes, c.width), 41, np.float32, 4)]
    q, k, v, g = (x.float().numpy() for x in rounded)
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    grads = O.attention_backward(g, q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    t = tables_for(c, np.float32)
    Q, K, V, G = (x.cuda() for x in rounded)
    out, lse = attention_forward(Q, K, V, t)
    assert rel_err(out.float().cpu().numpy(), want) < 2e-2
    got = attention_backward(G, Q, K, V, out, lse, t)
    for name, a, b in zip(("dq", "dk", "dv"), got, grads):
        assert rel_err(a.float().cpu().numpy(), b) < 2e-2, name


@pytest.mark.parametrize("name,rtol,atol", [("f64_hard", 1e-10, 1e-11), ("f32_quartic", 1e-5, 2e-6)])
def test_fused_attention_matches_reference_golden(golden_dir, name, rtol, atol):
    """Inputs and outputs produced by the reference's own Python (fused Softmax + eager value path + autograd)."""
    from gm_attention_b200.attention import AttentionTables, GaugeAttention

    g = np.load(golden_dir / f"attention_{name}.npz")
    t = AttentionTables(cuda(g["transport"]), cuda(g["bias"]), cuda(g["inside"]), cuda(g["row_ptr"]), cuda(g["source"]),
                        tuple(tuple(int(x) for x in row) for row in g["desc"]), int(g["heads"]), float(g["scale"]))
    q, k, v = (cuda(g[x]).requires_grad_(True) for x in ("q", "k", "v"))
    out = GaugeAttention.apply(q, k, v, t)
    assert_close(out.detach().cpu().numpy(), g["out"], rtol, atol, "out")
    (out * cuda(g["dout"])).sum().backward()
    for x, grad in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
        assert_close(grad.cpu().numpy(), g[x], rtol, 10 * atol * max(1.0, np.abs(g[x]).max()), x)


def test_unsupported_head_count_is_a_clear_error():
    from gm_attention_b200.attention import attention_forward

    c = make_case(6, 12, 2 * math.pi / 6, {0: 2}, 3, dtype=np.float32)
    q, = seeded((c.n_nodes, c.width), 1, np.float32)
    with pytest.raises(RuntimeError, match="heads must be 1, 2, 4 or 8"):
        attention_forward(cuda(q), cuda(q), cuda(q), tables_for(c, np.float32))


def test_one_infinite_value_reaches_its_neighbours_only():
    """The reference's edge loop (plain float arithmetic, ``nn/fused/attention.h:295-316`` + the eager value path) lets
    a non-finite value of a node reach exactly the targets that see the node, in that column.  The general (CSR)
    kernels do the same; the oracle on the same field is the witness.  (The lattice kernels, FMA and tensor-core, do
    not: owners that share staged neighbour rows multiply them by zero weights outside their own windows.)"""
    from gm_attention_b200.attention import attention_forward

    c = make_case(12, 24, 3 * math.pi / 12, {0: 4, 1: 4, 2: 4}, 2, dtype=np.float32)
    q, k, v = seeded((c.n_nodes, c.width), 77, np.float32, 3)
    node, column = 5 * c.nlon + 23, 6  # a scalar channel of the second head
    v[node, column] = np.inf
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, 1)
    seen_by = np.unique(c.target[c.source == node])
    assert np.array_equal(np.flatnonzero(~np.isfinite(want).all(1)), seen_by) and np.isfinite(np.delete(want, column, 1)).all()
    out, _ = attention_forward(cuda(q), cuda(k), cuda(v), tables_for(c, np.float32))
    out = out.cpu().numpy()
    assert np.array_equal(np.isfinite(out), np.isfinite(want))
    finite = np.isfinite(want)
    assert_close(out[finite], want[finite], 1e-5, 1e-6 * max(1.0, np.abs(want[finite]).max()), "finite entries")
