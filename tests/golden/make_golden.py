"""Generate the golden fixtures under ``tests/golden/`` by running the reference.

Run where a checkout of masonfaldet/gm-attention is mounted (``$GM_REFERENCE_ROOT``,
default: a directory ``reference`` next to this repository) and ``oracle/_ref``
has been built (``python oracle/build_ref.py``)::

    python tests/golden/make_golden.py

The reference's Python (``gm_attention.discretization.edge_geometry``,
``gm_attention.nn.fused_attention``, ``gm_attention.nn.kernels``,
``gm_attention.nn._scatter``, ``gm_attention.representations``) is imported
from the checkout; its extension loader is pointed at the modules compiled
from the reference's own C++ sources by ``oracle/build_ref.py`` (same sources,
no JIT).  Outputs are small ``.npz`` files:

* ``geometry_<nlat>x<nlon>.npz``  -- CSR + per-edge tables of
  ``compute_edge_geometry`` on the midpoint lattice with (east, north) frames;
* ``geometry_counts.npz``         -- edge counts, per-row degrees and a CSR
  checksum for the larger benchmark lattices;
* ``attention_<case>.npz``        -- seeded inputs, ``Softmax`` alpha, the fused
  layer's output (reference fused Softmax + eager transport / segment sum) and
  the gradients autograd returns for ``q, k, v``;
* ``plans.npz``                   -- descriptor rows of the reference planner;
* ``depthwise_<case>.npz``        -- a depthwise ``SO2Convolution`` (radial network included) on a small lattice through
  the reference's eager path: its parameters, the per-edge coefficients of ``stacked_coefficients``, a seeded field and
  output gradient, the output, and autograd's gradients for the field and every parameter.
"""

from __future__ import annotations

import math
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REFERENCE = Path(os.environ.get("GM_REFERENCE_ROOT", str(REPO.parent / "reference")))
sys.path.insert(0, str(REFERENCE / "src"))
sys.path.insert(0, str(REPO))

from gm_attention.discretization.edge_geometry import compute_edge_geometry  # noqa: E402
from gm_attention.nn import fused_attention as ref_fa  # noqa: E402
from gm_attention.nn._scatter import gather_to_edges, scatter_add_to_nodes  # noqa: E402
from gm_attention.nn.convolution import SO2Convolution  # noqa: E402
from gm_attention.nn.depthwise import stacked_coefficients  # noqa: E402
from gm_attention.nn.kernels import transport_field  # noqa: E402
from gm_attention.representations.field_type import SO2FeatureField, SO2FieldType  # noqa: E402

from oracle import build_ref  # noqa: E402
from oracle import geometry_np as G  # noqa: E402

ref_fa.extension = lambda cuda=False: build_ref.load("gm_fused_attention_cpu")
ref_fa.MODE = "cpu"


def reference_edges(nlat: int, nlon: int, radius: float, dtype: torch.dtype, max_frequency: int = 4):
    lat = G.midpoint_lattice(nlat, nlon)
    grid = SimpleNamespace(nodes=torch.from_numpy(lat.nodes).to(dtype), quadrature_weights=torch.from_numpy(lat.weights).to(dtype),
                           exact_nodes=torch.from_numpy(lat.nodes))
    return compute_edge_geometry(grid, torch.from_numpy(lat.frames).to(dtype), radius, max_frequency=max_frequency)


from tests.golden.make_golden_checksum import csr_checksum  # noqa: E402


def dump_geometry() -> None:
    for nlat, nlon, radius, dtype in [(8, 16, 2 * math.pi / 8, torch.float64), (12, 24, 3 * math.pi / 12, torch.float32)]:
        e = reference_edges(nlat, nlon, radius, dtype)
        np.savez_compressed(
            HERE / f"geometry_{nlat}x{nlon}.npz", radius=radius, edge_index=e.edge_index.numpy(), row_ptr=e.row_ptr.numpy(),
            distances=e.distances.numpy(), polar_angles=e.polar_angles.numpy(), transport_angles=e.transport_angles.numpy(),
            tangent_quadrature_weights=e.tangent_quadrature_weights.numpy(), log_coordinates=e.log_coordinates.numpy(),
            angular_phases=e.angular_phases.numpy(), transport_phases=e.transport_phases.numpy())
    names, counts, sums, degrees = [], [], [], []
    for nlat, nlon, mult in [(32, 64, 2), (32, 64, 3), (64, 128, 3), (128, 256, 3), (256, 512, 3), (256, 512, 4)]:
        e = reference_edges(nlat, nlon, mult * math.pi / nlat, torch.float32, max_frequency=2)
        deg = (e.row_ptr[1:] - e.row_ptr[:-1]).reshape(nlat, nlon)
        assert bool((deg == deg[:, :1]).all())
        names.append(f"{nlat}x{nlon}_r{mult}")
        counts.append(e.n_edges)
        sums.append(csr_checksum(e.row_ptr.numpy(), e.edge_index[1].numpy()))
        degrees.append(np.pad(deg[:, 0].numpy(), (0, 256 - nlat)))
    np.savez_compressed(HERE / "geometry_counts.npz", names=np.array(names), counts=np.array(counts, np.int64),
                        checksums=np.array(sums, np.uint64), degrees=np.stack(degrees))


def attention_case(name: str, nlat: int, nlon: int, radius: float, head_type: dict[int, int], heads: int, batch: int,
                   dtype: torch.dtype, window: str, seed: int) -> None:
    e = reference_edges(nlat, nlon, radius, dtype)
    attn = SO2FieldType(head_type)
    full = attn.scaled(heads)
    owner = SimpleNamespace()
    plan = ref_fa._plan(owner, attn, full, heads)
    desc = ref_fa.descriptors(owner, plan, torch.device("cpu"))
    geo = ref_fa.geometry(e, radius, window, dtype)
    n = nlat * nlon
    gen = torch.Generator().manual_seed(seed)
    q, k, v, dout = (torch.randn(batch * n, full.dimension, generator=gen, dtype=torch.float32).to(dtype) for _ in range(4))
    scale = 1.0 / math.sqrt(attn.dimension)
    head_of_column = torch.empty(full.dimension, dtype=torch.long)
    for nfreq, a_n in attn.items():
        dim = 1 if nfreq == 0 else 2
        start = full.slices()[nfreq].start
        for h in range(heads):
            head_of_column[start + h * a_n * dim: start + (h + 1) * a_n * dim] = h
    outs, alphas, grads = [], [], []
    for b in range(batch):
        qb, kb, vb = (t[b * n:(b + 1) * n].clone().requires_grad_(True) for t in (q, k, v))
        alpha = ref_fa.Softmax.apply(qb, kb, geo.transport, geo.bias, geo.inside, desc, geo.row_ptr, geo.source, heads, scale,
                                     max(geo.max_degree, 1))
        field = SO2FeatureField.from_flat(full, vb)
        transported = transport_field(gather_to_edges(field, e.source_index), e).to_flat()
        out = scatter_add_to_nodes(transported * alpha[:, head_of_column], e.row_ptr)
        (out * dout[b * n:(b + 1) * n]).sum().backward()
        outs.append(out.detach())
        alphas.append(alpha.detach())
        grads.append((qb.grad, kb.grad, vb.grad))
    np.savez_compressed(
        HERE / f"attention_{name}.npz", nlat=nlat, nlon=nlon, radius=radius, heads=heads, batch=batch, window=window, scale=scale,
        head_type=np.array(sorted(head_type.items()), np.int64), desc=desc.numpy(),
        q=q.numpy(), k=k.numpy(), v=v.numpy(), dout=dout.numpy(), alpha=torch.stack(alphas).numpy(),
        out=torch.cat(outs).numpy(), dq=torch.cat([g[0] for g in grads]).numpy(), dk=torch.cat([g[1] for g in grads]).numpy(),
        dv=torch.cat([g[2] for g in grads]).numpy(), transport=geo.transport.numpy(), bias=geo.bias.numpy(),
        inside=geo.inside.numpy(), row_ptr=geo.row_ptr.numpy(), source=geo.source.numpy())


def dump_plans() -> None:
    # the known-answer layout of tests/nn/test_fused_attention.py:91-95 of the reference
    attn = SO2FieldType({0: 3, 1: 2, 2: 1})
    owner = SimpleNamespace()
    plan = ref_fa._plan(owner, attn, attn.scaled(2), 2)
    np.savez_compressed(HERE / "plans.npz", rows=np.array(plan.rows, np.int64),
                        summary=np.array([plan.heads, plan.width, plan.a_0, plan.complex_width, plan.max_order], np.int64))


def depthwise_case(name: str, nlat: int, nlon: int, radius: float, types: dict[int, int], normalize: bool, seed: int) -> None:
    """nn/convolution.py:297-356 with depthwise=True through the eager path (GM_FUSED_ATTENTION off)."""
    dtype = torch.float64
    edges = reference_edges(nlat, nlon, radius, dtype)
    field_type = SO2FieldType(types)
    torch.manual_seed(seed)
    conv = SO2Convolution(field_type, field_type, cutoff=radius, window="hard", depthwise=True, normalize=normalize, n_radial_basis=4,
                          radial_hidden_features=(16,), dtype=dtype)
    gen = torch.Generator().manual_seed(seed + 100)
    n = nlat * nlon
    flat = torch.randn(n, field_type.dimension, generator=gen, dtype=dtype).requires_grad_(True)
    dout = torch.randn(n, field_type.dimension, generator=gen, dtype=dtype)
    mode, ref_fa.MODE = ref_fa.MODE, "0"
    try:
        out = conv(SO2FeatureField.from_flat(field_type, flat), edges).to_flat()
        out.backward(dout)
        rc, cc = stacked_coefficients([conv.kernel], edges)
    finally:
        ref_fa.MODE = mode
    params = {k.replace(".", "__"): v.detach().numpy() for k, v in conv.kernel.named_parameters()}
    grads = {"grad__" + k.replace(".", "__"): v.grad.numpy() for k, v in conv.kernel.named_parameters()}
    np.savez_compressed(HERE / f"depthwise_{name}.npz", nlat=nlat, nlon=nlon, radius=radius, normalize=int(normalize),
                        types=np.array(sorted(types.items()), np.int64), v=flat.detach().numpy(), dout=dout.numpy(), out=out.detach().numpy(),
                        dv=flat.grad.numpy(), rc=rc[0].detach().numpy(), cc=cc[0].detach().numpy(), distances=edges.distances.numpy(),
                        **params, **grads)


if __name__ == "__main__":
    build_ref.build()
    dump_geometry()
    dump_plans()
    attention_case("f64_hard", 8, 16, 2 * math.pi / 8, {0: 3, 1: 2, 2: 1}, 2, 2, torch.float64, "hard", 0)
    attention_case("f32_quartic", 8, 16, 2.5 * math.pi / 8, {0: 2, 1: 2}, 4, 1, torch.float32, "quartic", 1)
    depthwise_case("plain", 8, 16, 2 * math.pi / 8, {0: 4, 1: 3, 2: 2}, False, 3)
    depthwise_case("normalized", 8, 16, 2.5 * math.pi / 8, {0: 2, 1: 2, 2: 2}, True, 4)
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
