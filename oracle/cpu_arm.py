"""The reference's CPU path of the fused gauge-attention layer, timed on the host cores.

TEST INFRASTRUCTURE / CPU BASELINE ONLY: executed by ``bench.py`` (``--impl reference`` and the
``cpu_baseline`` leg); the shipped package never imports it.

What runs, per sample of the batch (the reference's batch is a disjoint-union graph, so samples are independent):

1. scores + softmax forward: the REFERENCE's compiled C++ driver ``softmax_forward``
   (``nn/fused/attention_cpu.cpp:197-219``, built from the reference's sources into ``oracle/_ref``);
2. value path forward and backward: a C PORT (``gm_oracle.c``) of the reference's eager
   ``transport_field`` + ``scatter_add_to_nodes`` (``nn/kernels.py:156-189``, ``nn/_scatter.py:36-46``) and of its
   adjoint -- the reference has no compiled driver for this half, and its Python package is not present on the
   benchmark host;
3. scores + softmax backward: the reference's ``softmax_backward`` (``attention_cpu.cpp:222-252``).

When ``oracle/_ref`` was never built the C port stands in for 1 and 3 too (``kind: "port"``).

The reference's drivers are single-threaded loops over the target nodes (``attention_cpu.cpp:216, 249``).  To use
every host core on the benchmark's own lattice, the TARGET ROWS of a sample are dealt to one worker process per
core (largest rows first, each to the least loaded worker): a worker calls the drivers on a CSR in which only its
rows have edges, which is what a user of the reference would do to parallelise it; every edge of the sample is
processed exactly once, by some worker.  Workers are forked after the tables are built, so they share them.
"""

from __future__ import annotations

import math
import multiprocessing as mp
import os
import time

import numpy as np

_STATE: dict = {}


def _deal_rows(edges_per_row: np.ndarray, parts: int) -> list[np.ndarray]:
    load = [0] * parts
    rows: list[list[int]] = [[] for _ in range(parts)]
    for r in np.argsort(-edges_per_row, kind="stable"):
        p = min(range(parts), key=load.__getitem__)
        rows[p].append(int(r))
        load[p] += int(edges_per_row[r])
    return [np.array(sorted(x), np.int64) for x in rows]


def prepare(nlat: int, nlon: int, radius: float, head_type: dict[int, int], heads: int, workers: int) -> dict:
    """Build the lattice's CSR and per-edge constants once (numpy oracle geometry), cut them into one sub-CSR per
    worker, and load the reference's driver in this process (workers inherit all of it through fork)."""
    from gm_attention_b200.fields import FieldType
    from oracle import build_ref
    from oracle import geometry_np as G
    from oracle import oracle as O
    from tests.helpers import descriptor_rows

    attn = FieldType(head_type)
    lat = G.midpoint_lattice(nlat, nlon)
    e = G.lattice_edges_by_symmetry(lat, radius, max(head_type), np.float32)
    tiny = np.finfo(np.float32).tiny
    win = (e.distances <= radius + 1e-5).astype(np.float32)
    bias = (np.log(np.maximum(win, tiny)) + np.log(np.maximum(e.tangent_quadrature_weights, tiny))).astype(np.float32)
    inside = (win > 0).astype(np.uint8)
    transport = np.ascontiguousarray(np.stack([e.transport_phases.real, e.transport_phases.imag], -1).astype(np.float32))
    source = np.ascontiguousarray(e.source_index)
    degree = np.diff(e.row_ptr)
    per_row = degree.reshape(nlat, nlon).sum(1)
    parts = []
    for rows in _deal_rows(per_row, workers):
        keep_node = np.zeros(nlat * nlon, bool)
        keep_node.reshape(nlat, nlon)[rows] = True
        keep_edge = np.repeat(keep_node, degree)
        row_ptr = np.zeros(nlat * nlon + 1, np.int64)
        np.cumsum(np.where(keep_node, degree, 0), out=row_ptr[1:])
        parts.append(dict(row_ptr=row_ptr, source=source[keep_edge], transport=np.ascontiguousarray(transport[keep_edge]),
                          bias=bias[keep_edge], inside=inside[keep_edge], edges=int(keep_edge.sum())))
    ref = None
    if (build_ref.OUT / "gm_fused_attention_cpu.so").exists():
        ref = build_ref.load("gm_fused_attention_cpu")
    O.build()
    _STATE.update(parts=parts, desc=descriptor_rows(attn, heads), heads=heads, scale=1.0 / math.sqrt(attn.dimension),
                  width=attn.scaled(heads).dimension, n_nodes=nlat * nlon, max_degree=int(degree.max()), ref=ref)
    return {"edges_per_sample": int(e.n_edges), "workers": workers, "kind": "reference+port" if ref is not None else "port",
            "worker_edges": [p["edges"] for p in parts]}


def _worker(job: tuple[int, list[int]]) -> float:
    """Forward + backward of this worker's target rows for the given samples; returns the seconds spent in the
    layer itself (input generation excluded: the device arm is likewise timed with its inputs resident)."""
    part_index, samples = job
    import torch

    from oracle import oracle as O

    torch.set_num_threads(1)
    s = _STATE
    p = s["parts"][part_index]
    t = torch.from_numpy
    tables = (t(p["transport"]), t(p["bias"]), t(p["inside"]), t(s["desc"]), t(p["row_ptr"]), t(p["source"]))
    spent = 0.0
    for b in samples:
        gen = torch.Generator().manual_seed(4321 + b)
        q, k, v, g = (torch.randn(s["n_nodes"], s["width"], generator=gen) for _ in range(4))
        t0 = time.perf_counter()
        if s["ref"] is not None:
            alpha = s["ref"].softmax_forward(q, k, *tables, s["heads"], s["scale"], s["max_degree"])
            O.value_forward(alpha.numpy(), v.numpy(), p["transport"], s["desc"], p["row_ptr"], p["source"], s["heads"])
            dalpha, _ = O.value_backward(g.numpy(), alpha.numpy(), v.numpy(), p["transport"], s["desc"], p["row_ptr"], p["source"], s["heads"])
            s["ref"].softmax_backward(t(dalpha), q, k, *tables, alpha, s["heads"], s["scale"], s["max_degree"])
        else:
            args = (p["transport"], p["bias"], p["inside"], s["desc"], p["row_ptr"], p["source"], s["heads"], s["scale"], 1)
            O.attention_forward(q.numpy(), k.numpy(), v.numpy(), *args)
            O.attention_backward(g.numpy(), q.numpy(), k.numpy(), v.numpy(), *args)
        spent += time.perf_counter() - t0
    return spent


class Pool:
    """One forked worker per core, kept across steps."""

    def __init__(self, info: dict) -> None:
        self.info = info
        self.pool = mp.get_context("fork").Pool(info["workers"])

    def step(self, samples: list[int]) -> dict:
        """All target rows of the given samples; ``seconds`` = the slowest worker's time inside the layer."""
        t0 = time.perf_counter()
        spent = self.pool.map(_worker, [(i, samples) for i in range(self.info["workers"])], chunksize=1)
        wall = time.perf_counter() - t0
        edges = self.info["edges_per_sample"] * len(samples)
        return {"seconds": max(spent), "seconds_wall": wall, "edges": edges, "value": edges / max(spent)}

    def close(self) -> None:
        self.pool.close()
        self.pool.join()


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1
