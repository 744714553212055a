"""Benchmark of the fused gauge-attention layer (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16|f32] [--impl ours|reference]

Metric: neighbour-edges per second of one fused gauge-attention layer, forward +
backward, where one edge is one (target <- source) CSR entry of one sample;
``value = batch * E1 / t(fwd + bwd)``.  Workload: the 256 x 512 midpoint
equiangular lattice, radius 3 pi / 256 (E1 = 13 527 040), batch 8, 4 heads of
16 x (m = 0, 1, 2) (D = 320); inputs ~ N(0, 1) from a fixed seed (synthetic
stand-ins for the shallow-water fields the reference trains on).

One JSON line is printed by rank 0.  ``value`` is timed with the inputs
resident in HBM; ``e2e`` is the same step driven from pinned HOST buffers with
the host->device and device->host copies inside the timed region.  With N > 1
the sphere is cut into edge-balanced latitude bands (one per rank), the key /
value halos are exchanged before the forward and the gradient halos after the
backward, all inside the timed region.

Before anything is timed the step's results are compared with the CPU oracle on
sampled targets and sources of the workload's own lattice (``"parity"`` in the
line); a failed check prints no number and exits non-zero.

``--impl reference`` times the reference's own CPU implementation of the same
layer, on the same lattice and batch, on the host cores: its compiled
scores+softmax driver (oracle/_ref, built from the reference's sources) plus a C
port of its eager value path, the target rows dealt to one worker process per
core (``oracle/cpu_arm.py``).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HEADLINE = dict(nlat=256, nlon=512, radius_rows=3, batch=8, heads=4, head_type={0: 16, 1: 16, 2: 16})
SMALL = dict(nlat=64, nlon=128, radius_rows=3, batch=2, heads=4, head_type={0: 16, 1: 16, 2: 16})
MID = dict(nlat=128, nlon=256, radius_rows=3, batch=4, heads=4, head_type={0: 16, 1: 16, 2: 16})  # profiling size: > L2, < 1 GB
L2_BYTES = 126 * 1024 * 1024


def parse() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--dtype", choices=["bf16", "f32"], default="bf16")
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--workload", choices=["headline", "mid", "small", "ops", "conv", "conv-mid"], default="headline",
                   help="headline (default): 256 x 512, batch 8; mid / small: 128 x 256 x 4 and 64 x 128 x 2 (profiling and smoke sizes); "
                        "ops: times every op-level entry point (scores+softmax, depthwise conv, factored kernel, pair term) "
                        "against its own interface bytes and prints one JSON object; conv: the depthwise convolution with its radial "
                        "network on the 256 x 512 lattice, radius 4 pi / 256, batch 4, 64 x (m = 0, 1, 2), forward + backward (conv-mid: "
                        "128 x 256, for profiler captures)")
    p.add_argument("--kernel", choices=["lattice", "csr"], default="lattice",
                   help="lattice: compact-table fast path (default); csr: general per-edge-table kernels")
    p.add_argument("--radius-rows", type=float, default=None,
                   help="neighbourhood radius in lattice row spacings (default: the workload's own, 3); other values are for profiling")
    p.add_argument("--overlap", action="store_true",
                   help="N > 1: run the layer around the halo exchange (interior rows while the halos travel) instead of exchanging "
                        "before / after it; bit-identical results; with the peer-memory exchange measured 0.6 %% faster at N = 4 and 2 %% slower "
                        "at N = 8 (the split launches cost more than the exchange they hide), so off by default")
    p.add_argument("--halo", choices=["auto", "peer", "native", "native-slabs", "torch"], default="auto",
                   help="N > 1: peer = the library's own copy kernels storing into the neighbour's mapped buffer (needs GPUs that can map each "
                        "other's memory); native = the library's NCCL groups issued from C, one packed message per neighbour and direction "
                        "(native-slabs: one message per field and sample); torch = torch.distributed point-to-point with staging buffers; "
                        "auto (default) = peer where it can be set up and its waits stay within their bounds during the warm-up, else native")
    p.add_argument("--per-rank", action="store_true",
                   help="every rank prints its own per-step timings (halo exchange in, forward, backward, halo sums out) to stderr")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-extra", action="store_true", help="skip the op-level and depthwise measurements the default run appends under \"extra\"")
    p.add_argument("--no-parity", action="store_true", help="skip the oracle check of the step's results (for profiler captures)")
    return p.parse_args()


# ----------------------------------------------------------------------------- CPU legs (oracle = checker / baseline only)

def cpu_pool(cfg: dict):
    """Worker pool over the workload's own lattice (built once: geometry, per-worker sub-tables, the reference's driver)."""
    from oracle import cpu_arm

    workers = cpu_arm.host_cores()
    info = cpu_arm.prepare(cfg["nlat"], cfg["nlon"], cfg["radius_rows"] * math.pi / cfg["nlat"], cfg["head_type"], cfg["heads"], workers)
    return cpu_arm.Pool(info)


def cpu_sample_text(cfg: dict, info: dict, samples: int) -> str:
    part = ("scores+softmax fwd/bwd = the reference's compiled C++ driver (single-threaded by construction), value path fwd/bwd = C port of "
            "the reference's eager transport + segment sum" if info["kind"] == "reference+port" else "C port of the reference's drivers and eager value path")
    return (f"{samples} of the batch's {cfg['batch']} samples on the workload's own {cfg['nlat']}x{cfg['nlon']} lattice ({info['edges_per_sample']} edges each), fp32, "
            f"target rows dealt to {info['workers']} worker processes (one per host core); {part}; seconds = the slowest worker's time inside the layer")


def run_reference(args: argparse.Namespace, cfg: dict) -> None:
    """The reference's CPU path on the workload's own lattice and batch.  One step = the whole batch; a step is
    tens of seconds of all host cores, so at most two steps are timed and none is spent on warm-up."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pool = cpu_pool(cfg)
    steps = max(1, min(args.steps, 2))
    results = [pool.step(list(range(cfg["batch"]))) for _ in range(steps)]
    pool.close()
    sec = statistics.median(r["seconds"] for r in results)
    value = results[0]["edges"] / sec
    info = pool.info
    line = {
        "impl": "reference", "metric": "gauge-attn fwd+bwd neighbour-edges/sec", "value": value, "unit": "edges/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": 0, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args, 1),
        "cpu_baseline": {"value": value, "unit": "edges/s", "cores": info["workers"], "kind": info["kind"],
                         "sample": cpu_sample_text(cfg, info, cfg["batch"]),
                         "seconds_wall_per_step": statistics.median(r["seconds_wall"] for r in results),
                         "pure_pytorch_path": "unavailable on this box: the reference's Python package is not present on the benchmark host"},
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(cfg: dict, args: argparse.Namespace, world: int) -> dict:
    return {"workload": f"fused gauge attention fwd+bwd, {cfg['nlat']}x{cfg['nlon']} midpoint equiangular lattice, radius "
                        f"{cfg['radius_rows']}pi/{cfg['nlat']}, batch {cfg['batch']}, {cfg['heads']} heads of 16x(m=0,1,2), D=320",
            "kernel_path": args.kernel, "global_batch": cfg["batch"], "parallelism": f"latitude-bands x{world}" if world > 1 else "single GPU",
            "l2": "inputs larger than L2 (no flush needed)"}


# ----------------------------------------------------------------------------- GPU arm

class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU while a timed region runs (read-only NVML queries from a
    thread, every few milliseconds; ``nvidia-smi -lms`` as the fallback when NVML cannot be loaded)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int, uuid: str | None = None) -> None:
        self.index, self.uuid, self.proc, self.thread = index, uuid, None, None
        self.samples: list[tuple[float, int]] = []  # (SM MHz, reason mask)
        self.sm_max = None
        self.source = None

    def _nvml_loop(self, nv, handle) -> None:
        while not self._stop.is_set():
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)), int(nv.nvmlDeviceGetCurrentClocksEventReasons(handle))))
            except Exception:  # noqa: BLE001  (a failed query is a missing sample)
                pass
            self._stop.wait(0.004)

    def __enter__(self):
        try:
            import threading

            import pynvml as nv

            nv.nvmlInit()
            handle = None
            if self.uuid:
                try:
                    handle = nv.nvmlDeviceGetHandleByUUID(self.uuid.encode() if hasattr(self.uuid, "encode") else self.uuid)
                except Exception:  # noqa: BLE001
                    handle = None
            if handle is None:
                handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self._masks = [nv.nvmlClocksEventReasonHwSlowdown, nv.nvmlClocksEventReasonHwThermalSlowdown,
                           nv.nvmlClocksEventReasonSwThermalSlowdown, nv.nvmlClocksEventReasonSwPowerCap]
            self._stop = threading.Event()
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            self.source = "nvml"
            return self
        except Exception:  # noqa: BLE001  (no NVML binding: fall back to the command-line tool)
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.rows = []
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            return
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def summary(self) -> dict:
        if self.thread is not None and self.samples:
            sm = sorted(s[0] for s in self.samples)
            reasons = [n for n, m in zip(self.NAMES, self._masks) if any(s[1] & m for s in self.samples)]
            busy = sm[len(sm) // 2:] or sm  # upper half = samples under load
            return {"sm_mhz": statistics.median(busy), "sm_max_mhz": self.sm_max, "reasons": reasons, "samples": len(sm), "source": "nvml"}
        rows = getattr(self, "rows", [])
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[5 + i].lower().startswith("active") for r in rows)]
        busy = sorted(sm)[len(sm) // 2:] or sm  # upper half = samples under load
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": float(rows[0][2]), "reasons": reasons,
                "samples": len(rows), "source": "nvidia-smi"}


def bind_to_gpu_cpus(uuid: str | None, index: int) -> None:
    """Pin this process to the CPU cores NVML reports as local to its GPU, so that the pinned host buffers of the
    end-to-end measurement are allocated on the GPU's own NUMA node (one process per GPU on a multi-socket host)."""
    try:
        import pynvml as nv

        nv.nvmlInit()
        handle = nv.nvmlDeviceGetHandleByUUID(uuid.encode()) if uuid else nv.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:  # noqa: BLE001  (no NVML, no affinity information: stay where the launcher put us)
        pass


def run_ours(args: argparse.Namespace, cfg: dict) -> None:
    import numpy as np
    import torch

    Tensor4 = torch.Tensor  # (4, batch, nlon, D): q, k, v, dO of one lattice row
    import torch.distributed as dist

    from gm_attention_b200 import _lib
    from gm_attention_b200.attention import (AttentionTables, attention_backward, attention_forward, build_lattice_tables,
                                             lattice_attention_backward, lattice_attention_forward)
    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa
    from gm_attention_b200.parallel import (BandPlan, HaloExchanger, NativeHaloExchanger, PeerHaloExchanger, band_geometry, overlap_tables, row_degrees,
                                            row_pair_counts, tensor_core_row_cost)

    _lib.lib()
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        peak, peak_kind = float(json.loads(peaks_path.read_text())["hbm_gbs"]), "measured"
    else:
        peak, peak_kind = 6650.0, "fallback"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        gpu_uuid0 = getattr(torch.cuda.get_device_properties(local), "uuid", None)
        bind_to_gpu_cpus(f"GPU-{gpu_uuid0}" if gpu_uuid0 is not None else None, local)
        # the halo messages are a few tens of MB between NVLink neighbours: give NCCL's point-to-point path more channels
        # than its default for small peer counts (a user's own setting wins)
        os.environ.setdefault("NCCL_MIN_P2P_NCHANNELS", "8")
        dist.init_process_group("nccl", device_id=device)
    nlat, nlon, batch, heads = cfg["nlat"], cfg["nlon"], cfg["batch"], cfg["heads"]
    radius = cfg["radius_rows"] * math.pi / nlat
    attn = FieldType(cfg["head_type"])
    full = attn.scaled(heads)
    D = full.dimension
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    elem = 2 if args.dtype == "bf16" else 4

    # ---- resident geometry (built once, on the device; not timed)
    lattice = midpoint_lattice(nlat, nlon, device)
    w = lattice.band(radius)
    if world > 1:
        if args.kernel == "lattice" and args.dtype == "bf16":  # balance the kernels' cost model, not the raw edge count
            row_cost = tensor_core_row_cost(row_pair_counts(lattice, radius))
        else:
            row_cost = row_degrees(lattice, radius)
        plan = BandPlan.balanced(nlat, nlon, w, row_cost, world)
    else:
        plan = BandPlan(nlat, nlon, w, (0, nlat))
    lo, hi = plan.owned(rank)
    elo, ehi = plan.extended(rank)
    rows_ext = ehi - elo
    edges = band_geometry(lattice, plan, rank, radius, max_frequency=2, dtype=torch.float32)
    geo = fa.geometry(edges, radius, "hard", torch.float32)
    owner = type("Layer", (), {})()
    p = fa._plan(owner, attn, full, heads)
    tables = AttentionTables(geo.transport, geo.bias, geo.inside, geo.row_ptr, geo.source, p.rows, heads, 1.0 / math.sqrt(attn.dimension))
    if args.kernel == "lattice":
        tables = build_lattice_tables(tables, rows_ext, nlon, p.rows, heads, tables.scale)
        attention_forward, attention_backward = lattice_attention_forward, lattice_attention_backward
        top_kernel, launches = "lattice_kernel<MODE_BWD_S> (timed: the whole backward call)", 4
    else:
        top_kernel, launches = "fused_backward_kernel (timed: the whole backward call)", 2 + (2 if args.dtype == "bf16" else 0)
    local_edges = edges.n_edges * batch
    n_ext = rows_ext * nlon

    # ---- inputs: seeded N(0, 1), generated on the host, resident on the device for `value`.  A lattice row's values
    # depend on its GLOBAL row index only, so every rank holds the same sphere whatever the cut, and the parity check
    # below can regenerate any row it needs.
    def row_fields(row: int) -> Tensor4:
        gen = torch.Generator().manual_seed(1234 + 7919 * row)
        return torch.randn((4, batch, nlon, D), generator=gen, dtype=torch.float32).to(dtype)

    shape = (batch, rows_ext, nlon, D)
    host = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(4)]
    for r in range(elo, ehi):
        block = row_fields(r)
        for f in range(4):
            host[f][:, r - elo] = block[f]
    q, k, v, g = (h.to(device, non_blocking=True) for h in host)
    flat = lambda t: t.view(batch * n_ext, D)
    # the library's own NCCL groups (sends / receives in place, nothing on the host); --halo torch: torch.distributed with staging
    halo_kind = args.halo

    def make_halo(band_plan, probe):
        """The exchanger --halo names; "auto" and "peer" try the peer-memory path on `probe` (two fields of the shape the
        exchanger will serve: set-up is collective and happens at the first exchange) and fall back to NCCL together."""
        nonlocal halo_kind
        if halo_kind in ("auto", "peer"):
            candidate = PeerHaloExchanger(band_plan, rank, device)
            try:
                candidate.fill_halos(*probe)
                halo_kind = "peer"
                return candidate
            except RuntimeError as exc:
                if args.halo == "peer":
                    raise
                if rank == 0:
                    print(json.dumps({"note": f"peer-memory halo exchange unavailable, using NCCL: {exc}"}), file=sys.stderr, flush=True)
                halo_kind = "native"
        if halo_kind == "torch":
            return HaloExchanger(band_plan, rank)
        return NativeHaloExchanger(band_plan, rank, device, packed=halo_kind != "native-slabs")

    halo = make_halo(plan, (k, v)) if world > 1 else None
    reduce_kw = {"zero_halo": False} if halo_kind != "torch" else {}  # the halo rows of dk / dv are not part of the rank's result
    fwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    bwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]

    mark_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]  # step start, step end

    # With latitude bands on the tensor-core path the layer runs AROUND the halo exchange: the forward of the rows that
    # need no halo while the K / V halos travel, the source-major backward of the rank's own rows while the dK / dV halo
    # sums travel (the halo rows' sums are formed first).
    split = overlap_tables(tables, plan, rank) if (world > 1 and args.kernel == "lattice" and args.dtype == "bf16" and args.overlap) else None

    def step(index: int | None = None):
        if index is not None:
            mark_ev[index][0].record()
        if split is not None:
            pending = halo.start_fill(k, v)
            if index is not None:
                fwd_ev[index][0].record()
            out, lse = attention_forward(flat(q), flat(k), flat(v), split.interior)
            halo.finish_fill(pending)
            attention_forward(flat(q), flat(k), flat(v), split.boundary, out=out, lse=lse)
            if index is not None:
                fwd_ev[index][1].record()
                bwd_ev[index][0].record()
            # every row the rank owns is written by one of the passes below; the halo rows of dq are not part of its result
            ws = (torch.empty_like(flat(q)), torch.empty_like(flat(q)), torch.empty_like(flat(q)),
                  torch.empty((batch * n_ext, heads), dtype=torch.float32, device=device))
            attention_backward(flat(g), flat(q), flat(k), flat(v), out, lse, split.full, passes=3, workspace=ws)
            attention_backward(flat(g), flat(q), flat(k), flat(v), out, lse, split.halo_sources, passes=4, workspace=ws)
            dq, dk, dv = ws[:3]
            pending = halo.start_reduce(dk.view(shape), dv.view(shape))
            attention_backward(flat(g), flat(q), flat(k), flat(v), out, lse, split.owned_sources, passes=4, workspace=ws)
            if index is not None:
                bwd_ev[index][1].record()
            halo.finish_reduce(pending, **reduce_kw)
            if index is not None:
                mark_ev[index][1].record()
            return out, dq, dk, dv
        if halo is not None:
            halo.fill_halos(k, v)
        if index is not None:
            fwd_ev[index][0].record()
        out, lse = attention_forward(flat(q), flat(k), flat(v), tables)
        if index is not None:
            fwd_ev[index][1].record()
            bwd_ev[index][0].record()
        dq, dk, dv = attention_backward(flat(g), flat(q), flat(k), flat(v), out, lse, tables)
        if index is not None:
            bwd_ev[index][1].record()
        if halo is not None:
            halo.reduce_halos(dk.view(shape), dv.view(shape), **reduce_kw)
        if index is not None:
            mark_ev[index][1].record()
        return out, dq, dk, dv

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if isinstance(halo, PeerHaloExchanger):
        # a bounded wait of the peer-memory exchange that ran out during the warm-up: every rank falls back to NCCL together
        code = torch.tensor([halo.error()], device=device, dtype=torch.int32)
        dist.all_reduce(code, op=dist.ReduceOp.MAX)
        if int(code.item()):
            if args.halo == "peer":
                print(json.dumps({"error": "a bounded wait of the peer-memory halo exchange ran out", "rank": rank, "code": int(code.item())}), file=sys.stderr, flush=True)
                sys.exit(5)
            halo, halo_kind = NativeHaloExchanger(plan, rank, device), "native"
            for _ in range(3):
                step()
            barrier()

    # ---- parity self-check at the workload's own size: one more step, compared with the CPU oracle on sampled targets
    # (out, dq) and sources (dk, dv) of this rank's rows -- complete CSR rows cut out of the GLOBAL lattice, so with
    # latitude bands the sums that cross a cut (halo exchange and reduction) are checked too.  Nothing is timed here.
    parity = None
    if not args.no_parity:
        from oracle import geometry_np as GN
        from oracle import sampled as SP

        result = step()
        torch.cuda.synchronize()
        near_pole = args.workload != "headline"  # a source next to the pole is ~1.5 M edges of oracle work at 256 x 512
        t_nodes, s_nodes = SP.default_sample_nodes(nlat, nlon, lo, hi, polar_source_row=2 if near_pole else None)
        sample = SP.sample_problem(GN.midpoint_lattice(nlat, nlon), radius, t_nodes, s_nodes, max(cfg["head_type"]), np.float32)
        b_chk = batch - 1
        cache: dict[int, torch.Tensor] = {}

        def gather(nodes):
            rows_needed = sorted(set((nodes // nlon).tolist()))
            for r in rows_needed:
                if r not in cache:
                    cache[r] = row_fields(r)[:, b_chk].float()  # (4, nlon, D)
            out4 = [np.empty((nodes.shape[0], D), np.float32) for _ in range(4)]
            for r in rows_needed:
                sel = np.flatnonzero(nodes // nlon == r)
                cols = torch.from_numpy(nodes[sel] % nlon)
                for f in range(4):
                    out4[f][sel] = cache[r][f][cols].numpy()
            return tuple(out4)

        want = SP.run(sample, gather, np.array(p.rows, np.int64), heads, tables.scale)

        def local_rows(x, nodes):
            idx = torch.from_numpy(nodes)
            return x.view(shape)[b_chk, (idx // nlon - elo).to(device), (idx % nlon).to(device)].float().cpu().numpy()

        got = {"out": local_rows(result[0], sample.targets), "dq": local_rows(result[1], sample.targets),
               "dk": local_rows(result[2], sample.sources), "dv": local_rows(result[3], sample.sources)}
        errs = [float(np.abs(got[n] - want[n]).max() / max(float(np.abs(want[n]).max()), 1e-30)) for n in ("out", "dq", "dk", "dv")]
        if world > 1:
            t = torch.tensor(errs, device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            errs = t.tolist()
            cnt = torch.tensor([sample.targets.shape[0], sample.sources.shape[0], sample.n_edges], device=device, dtype=torch.int64)
            dist.all_reduce(cnt)
            n_t, n_s, n_e = cnt.tolist()
        else:
            n_t, n_s, n_e = sample.targets.shape[0], sample.sources.shape[0], sample.n_edges
        tolerance = 2e-2 if args.dtype == "bf16" else 2e-5
        parity = {"max_rel": max(errs), "per_tensor": dict(zip(("out", "dq", "dk", "dv"), errs)), "tolerance": tolerance,
                  "targets": n_t, "sources": n_s, "oracle_edges": n_e, "sample_of_batch": b_chk,
                  "against": "CPU oracle (reference Softmax op + eager value path restated in C) in fp32 on the same "
                             + ("bf16-rounded " if args.dtype == "bf16" else "") + "inputs; error = max |a - b| / max |b| per tensor"}
        del result, cache
        if not max(errs) <= tolerance:
            if rank == 0:
                print(json.dumps({"error": "parity check failed: no number is reported", "parity": parity}), file=sys.stderr, flush=True)
            if world > 1:
                dist.destroy_process_group()
            sys.exit(3)

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu_uuid = getattr(torch.cuda.get_device_properties(local), "uuid", None)
    with ClockSampler(local, f"GPU-{gpu_uuid}" if gpu_uuid is not None else None) as clocks:
        barrier()  # the samplers start at different times on different ranks: line the ranks up again before the clock starts
        calls_before = dict(_lib.CALLS)
        start.record()
        for s in range(args.steps):
            step(s)
        stop.record()
        barrier()
    # this rank's own halo kernels inside the timed region (pack / unpack / add, or the peer-memory send / landing)
    halo_launches = sum(_lib.CALLS[n] - calls_before.get(n, 0) for n in ("gm_halo_move", "gm_halo_accumulate", "gm_peer_send", "gm_peer_land", "gm_peer_send_many", "gm_peer_land_many"))
    ms_total = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms_total], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t)
        tot = torch.tensor([local_edges], device=device, dtype=torch.int64)
        dist.all_reduce(tot)
        total_edges = int(tot)
    else:
        total_edges = local_edges
    ms_step = ms_total / args.steps
    if args.per_rank:
        detail = [{"halo_in": round(m[0].elapsed_time(f[0]), 3), "fwd": round(f[0].elapsed_time(f[1]), 3), "bwd": round(b[0].elapsed_time(b[1]), 3),
                   "halo_out": round(b[1].elapsed_time(m[1]), 3)} for m, f, b in zip(mark_ev, fwd_ev, bwd_ev)]
        print(json.dumps({"rank": rank, "rows": [plan.owned(rank)[0], plan.owned(rank)[1]] if world > 1 else [0, nlat], "steps_ms": detail}), file=sys.stderr, flush=True)
    fwd_ms = statistics.mean(a.elapsed_time(b) for a, b in fwd_ev)
    bwd_ms = statistics.mean(a.elapsed_time(b) for a, b in bwd_ev)

    # ---- the dominant kernel alone (CUDA events on the launching stream): the source-major backward pass of the
    # tensor-core lattice path; other paths report the whole backward call
    top_ms, top_bytes, top_traffic = bwd_ms, None, None
    n_rows_local = batch * n_ext
    if args.kernel == "lattice" and args.dtype == "bf16":
        out0, lse0 = attention_forward(flat(q), flat(k), flat(v), tables)
        ws = [torch.empty_like(flat(q)) for _ in range(3)] + [torch.empty((n_rows_local, heads), dtype=torch.float32, device=device)]
        attention_backward(flat(g), flat(q), flat(k), flat(v), out0, lse0, tables, passes=7, workspace=tuple(ws))
        per_pass = {}
        # forward, target-major pass (forms Delta = <dO, O> itself), source-major pass; around a halo exchange the forward and
        # the source-major pass are two launches each
        launches = 5 if split is not None else 3
        for name, mask in (("pass_t", 3), ("pass_s", 4)):  # mask 3: Delta + dq in one kernel
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(5)]
            for a_ev, b_ev in ev:
                a_ev.record()
                attention_backward(flat(g), flat(q), flat(k), flat(v), out0, lse0, tables, passes=mask, workspace=tuple(ws))
                b_ev.record()
            torch.cuda.synchronize()
            per_pass[name] = statistics.mean(x.elapsed_time(y) for x, y in ev[1:])
        top_kernel = "lattice_tn_kernel<1,2,2,TC_BWD_S,4> (source-major backward pass: dk, dv)"
        top_ms = per_pass["pass_s"]
        top_bytes = 6 * n_rows_local * D * elem + 2 * n_rows_local * heads * 4
        # DRAM read + write of this kernel per node, from the ncu capture on the 128x256x4 workload (profiles/), scaled by nodes
        top_traffic = int(4926 * n_rows_local)
        del out0, lse0, ws
    else:
        per_pass = None

    # ---- the same layer with fp32 node fields (FMA lattice kernels), for the record: 3 timed steps, N = 1 only
    f32_line = None
    if world == 1 and args.dtype == "bf16" and args.kernel == "lattice" and not args.no_e2e:
        q32, k32, v32, g32 = (flat(x).float() for x in (q, k, v, g))
        for _ in range(2):
            o32, l32 = attention_forward(q32, k32, v32, tables)
            attention_backward(g32, q32, k32, v32, o32, l32, tables)
        torch.cuda.synchronize()
        ev32 = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev32[0].record()
        for _ in range(3):
            o32, l32 = attention_forward(q32, k32, v32, tables)
        ev32[1].record()
        for _ in range(3):
            attention_backward(g32, q32, k32, v32, o32, l32, tables)
        ev32[2].record()
        torch.cuda.synchronize()
        f_ms, b_ms = ev32[0].elapsed_time(ev32[1]) / 3, ev32[1].elapsed_time(ev32[2]) / 3
        f32_line = {"dtype": "f32", "fwd_ms": f_ms, "bwd_ms": b_ms, "value": total_edges / ((f_ms + b_ms) * 1e-3), "unit": "edges/s",
                    "hbm_frac": (12 * n_rows_local * D * 4 + 2 * n_rows_local * heads * 4) / ((f_ms + b_ms) * 1e-3) / 1e9 / peak}
        del q32, k32, v32, g32, o32, l32

    # ---- end to end from pinned host buffers (copies inside the timed region)
    e2e = None
    if not args.no_e2e:
        outs_host = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(4)]
        e2e_rows, e2e_cuts, pipeline = rows_ext, None, None
        if args.kernel == "lattice":
            # host-resident fields through the public host API: sample chunks pipelined over three streams
            # (with latitude bands, every chunk's halos are exchanged inside the pipeline)
            from gm_attention_b200.attention import HostPipeline
            e_tables, e_halo, e_host = tables, halo, host
            if world > 1:
                # End to end a rank is bound by its copies, not its kernels: cut the sphere so that the slowest rank's
                # (copy time + compute time) is smallest, instead of compute alone.  Copies: one lattice row of the four
                # fields each way at the ~25 GB/s per direction a GPU gets when all GPUs of the host copy at once.
                copy_ms_row = 4 * batch * nlon * D * elem / 25e9 * 1e3
                unit = world * (fwd_ms + bwd_ms) / max(sum(row_cost), 1e-30)  # ms of kernel time per unit of the cost model
                plan2 = BandPlan.balanced(nlat, nlon, w, [copy_ms_row + unit * c for c in row_cost], world)
                e2e_cuts = list(plan2.cuts)
                lo2, hi2 = plan2.extended(rank)
                e2e_rows = hi2 - lo2
                edges2 = band_geometry(lattice, plan2, rank, radius, max_frequency=2, dtype=torch.float32)
                geo2 = fa.geometry(edges2, radius, "hard", torch.float32)
                gen2 = AttentionTables(geo2.transport, geo2.bias, geo2.inside, geo2.row_ptr, geo2.source, p.rows, heads, 1.0 / math.sqrt(attn.dimension))
                e_tables = build_lattice_tables(gen2, e2e_rows, nlon, p.rows, heads, gen2.scale)
                shape2 = (batch, e2e_rows, nlon, D)
                probe2 = [torch.zeros((1, e2e_rows, nlon, D), dtype=dtype, device=device) for _ in range(2)]  # the pipeline exchanges per one-sample chunk
                e_halo = make_halo(plan2, probe2)
                e_host = [torch.empty(shape2, dtype=dtype).pin_memory() for _ in range(4)]
                for r in range(lo2, hi2):
                    block = row_fields(r)
                    for f in range(4):
                        e_host[f][:, r - lo2] = block[f]
                outs_host = [torch.empty(shape2, dtype=dtype).pin_memory() for _ in range(4)]
            pipeline = HostPipeline(e_tables, batch, D, dtype, device, chunk=1, halo=e_halo)
            pipeline.profile = True
            host_flat = [x.view(batch * e2e_rows * nlon, D) for x in e_host]
            outs_flat = [x.view(batch * e2e_rows * nlon, D) for x in outs_host]
            def e2e_step():  # enqueue only: consecutive steps overlap their first / last copies; joined before the clock stops
                pipeline.run(*host_flat, *outs_flat, wait=False)
            e2e_join = pipeline.join
        else:
            e2e_join = lambda: None
            def e2e_step():
                dev = [x.to(device, non_blocking=True) for x in host]
                qq, kk, vv, gg = dev
                if halo is not None:
                    halo.fill_halos(kk, vv)
                out, lse = attention_forward(flat(qq), flat(kk), flat(vv), tables)
                dq, dk, dv = attention_backward(flat(gg), flat(qq), flat(kk), flat(vv), out, lse, tables)
                if halo is not None:
                    halo.reduce_halos(dk.view(shape), dv.view(shape))
                for dst, src in zip(outs_host, (out, dq, dk, dv)):
                    dst.copy_(src.view(shape), non_blocking=True)
        barrier()  # pinning hundreds of MB takes the ranks different times: the bounded waits of the exchange assume aligned starts
        for _ in range(2):
            e2e_step()
        e2e_join()
        barrier()
        n_e2e = max(3, min(args.steps, 5))
        start.record()
        for _ in range(n_e2e):
            e2e_step()
        e2e_join()
        stop.record()
        barrier()
        ms = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        nbytes = 4 * batch * e2e_rows * D * nlon * elem
        phases = pipeline.phase_ms() if pipeline is not None else None
        if world > 1:
            # bytes: the largest share of a rank (what bounds the step) and the whole job's; phases: the slowest rank's
            every = [None] * world
            dist.all_gather_object(every, {"bytes": nbytes, "phases": phases})
            slowest = max(every, key=lambda x: max(x["phases"].values()) if x["phases"] else 0.0)
            nbytes, total_bytes, phases = max(x["bytes"] for x in every), sum(x["bytes"] for x in every), slowest["phases"]
        else:
            total_bytes = nbytes
        e2e = {"value": total_edges / (ms / n_e2e * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
               "ms_per_step": ms / n_e2e, "steps": n_e2e, "bytes_counted": "the largest share of a rank" if world > 1 else "the whole job's",
               "job_bytes_per_direction": total_bytes, "band_cuts": e2e_cuts,
               "last_step_phases_ms_slowest_rank": phases}

    # a wait on a TMA completion barrier that ran out is recorded by the kernels instead of hanging: results would be invalid
    import ctypes
    expired = ctypes.c_int(0)
    _lib.call("gm_lattice_attention_tc_wait_expired", ctypes.byref(expired))
    if expired.value:
        print(json.dumps({"error": "a wait on a copy barrier ran out inside the tensor-core lattice kernels: no number is reported", "rank": rank}),
              file=sys.stderr, flush=True)
        sys.exit(4)
    if isinstance(halo, PeerHaloExchanger) and halo.error():
        print(json.dumps({"error": "a bounded wait of the peer-memory halo exchange ran out: no number is reported", "rank": rank, "code": halo.error()}),
              file=sys.stderr, flush=True)
        sys.exit(5)
    if rank == 0:
        n_rows = batch * n_ext
        bwd_bytes = top_bytes if top_bytes is not None else 8 * n_rows * D * elem + n_rows * heads * 4
        layer_bytes = 12 * n_rows * D * elem + 2 * n_rows * heads * 4
        achieved = bwd_bytes / (top_ms * 1e-3) / 1e9
        line = {
            "metric": "gauge-attn fwd+bwd neighbour-edges/sec", "value": total_edges / (ms_step * 1e-3), "unit": "edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "config": workload_config(cfg, args, world),
            "roofline": {"bound": "hbm", "kernel": top_kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": top_traffic, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": bwd_bytes, "launch_ms": top_ms, "passes_ms": per_pass},
            "layer": {"fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "algorithmic_bytes": layer_bytes,
                      "hbm_frac": layer_bytes / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak, "edges": total_edges},
            "gpu_launches": args.steps * launches + halo_launches,
            "clocks": clocks.summary(),
            "e2e": e2e,
            "tma_wait_expired": expired.value,
            "halo_exchange": None if world == 1 else {"kind": halo_kind, "own_kernel_launches_rank0": halo_launches, "overlapped_with_layer": split is not None},
            "other_dtypes": f32_line,
        }
        line["parity"] = parity
        if not args.no_cpu_baseline and world == 1:
            # one sample of the batch on the workload's own lattice, all host cores (tens of core-seconds)
            pool = cpu_pool(cfg)
            res = pool.step([0])
            pool.close()
            line["cpu_baseline"] = {"value": res["value"], "unit": "edges/s", "cores": pool.info["workers"], "kind": pool.info["kind"],
                                    "sample": cpu_sample_text(cfg, pool.info, 1), "seconds": res["seconds"],
                                    "pure_pytorch_path": "unavailable on this box: the reference's Python package is not present on the benchmark host"}
        if world == 1 and args.workload == "headline" and not args.no_extra:
            # the other entry points of the library, measured in the same run: every op-level drop-in (128 x 256, fp32) and the
            # depthwise convolution with its radial network (256 x 512, radius 4 pi / 256, batch 4); a failure there is recorded,
            # it does not take the line away
            torch.cuda.empty_cache()
            extra = {}
            for name, fn in (("ops", run_ops), ("conv", run_conv)):
                sub = argparse.Namespace(**{**vars(args), "workload": name, "no_e2e": True, "no_cpu_baseline": True, "steps": 5})
                try:
                    res = fn(sub, emit=False)
                    extra[name] = res if name == "ops" else {key: res[key] for key in ("metric", "value", "unit", "ms_per_step", "dtype", "config", "roofline", "parity")}
                except (Exception, SystemExit) as exc:  # noqa: BLE001
                    extra[name] = {"error": repr(exc)}
            line["extra"] = extra
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_ops(args: argparse.Namespace, emit: bool = True) -> dict:
    """Per-op timings of the drop-in entry points on a 128 x 256 lattice (radius 3 pi / 128, ~3.0 M edges), fp32:
    achieved GB/s of each op's own interface bytes (inputs + outputs, each byte once), CUDA events, 3 warm-up + 10 timed."""
    import numpy as np
    import torch

    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa
    from gm_attention_b200.nn import fused_factored as ff
    from gm_attention_b200.nn import fused_pairs as fp

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    nlat, nlon = 128, 256
    radius = 3 * math.pi / nlat
    lattice = midpoint_lattice(nlat, nlon, dev)
    edges = compute_edge_geometry(lattice, lattice.frames, radius, max_frequency=4, dtype=torch.float32)
    geo = fa.geometry(edges, radius, "hard", torch.float32)
    n, e = nlat * nlon, edges.n_edges
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32)
    peak = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"] if (ROOT / "MEASURED_PEAKS.json").exists() else 6650.0
    results = {}

    def timed(name: str, fn, nbytes: int) -> None:
        for _ in range(3):
            fn()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
        for a, b in ev:
            a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ms = statistics.mean(a.elapsed_time(b) for a, b in ev)
        results[name] = {"ms": ms, "interface_bytes": nbytes, "GB/s": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peak,
                         "edges_per_s": e / (ms * 1e-3)}

    # scores + softmax: 4 heads of 8 x (m = 0..3), D = 224 (the 128 x 256 configuration's head layout)
    heads, attn = 4, FieldType({0: 8, 1: 8, 2: 8, 3: 8})
    owner = type("Layer", (), {})()
    p = fa._plan(owner, attn, attn.scaled(heads), heads)
    desc = fa.descriptors(owner, p, dev)
    D = p.width
    q, k = rnd(n, D), rnd(n, D)
    ext = fa.extension(True)
    sm = (geo.transport, geo.bias, geo.inside, desc, geo.row_ptr, geo.source, heads, 1.0 / math.sqrt(attn.dimension), geo.max_degree)
    alpha = ext.softmax_forward(q, k, *sm[:6], *sm[6:])
    dalpha = rnd(e, heads)
    tab = e * (geo.transport.shape[1] * 2 * 4 + 4 + 1 + 8) + (n + 1) * 8
    timed("softmax_forward", lambda: ext.softmax_forward(q, k, *sm), 2 * n * D * 4 + tab + e * heads * 4)
    timed("softmax_backward", lambda: ext.softmax_backward(dalpha, q, k, *sm[:6], alpha, *sm[6:]), 4 * n * D * 4 + tab + 2 * e * heads * 4)
    del q, k, alpha, dalpha
    # depthwise conv: 16 x (m = 0, 1, 2): D = 80, a0 = 16, W = 128
    conv_type = FieldType({0: 16, 1: 16, 2: 16})
    owner2 = type("Layer", (), {})()
    p2 = fa._plan(owner2, conv_type, conv_type, 1)
    desc2 = fa.descriptors(owner2, p2, dev)
    v, g = rnd(n, p2.width), rnd(n, p2.width)
    rc, cc = rnd(e, p2.a_0), rnd(e, p2.complex_width)
    cv = (rc, cc, geo.transport, geo.angular, geo.rho, geo.weights, desc2, geo.row_ptr, geo.source, p2.a_0, p2.complex_width)
    coeff = e * (p2.a_0 + p2.complex_width) * 4
    tab2 = e * (2 * geo.transport.shape[1] * 2 * 4 + 8 + 8) + (n + 1) * 8
    timed("conv_forward", lambda: ext.conv_forward(v, *cv), 2 * n * p2.width * 4 + coeff + tab2)
    timed("conv_backward", lambda: ext.conv_backward(g, v, *cv), 3 * n * p2.width * 4 + 2 * coeff + tab2)
    del rc, cc, v, g
    # factored value kernel {8, 8, 8} -> {4, 4, 4}, trunk 16 (value kernel of the 32 x 64 configuration: 13 blocks, wc 48, wr 4)
    tin, tout, kk = {0: 8, 1: 8, 2: 8}, {0: 4, 1: 4, 2: 4}, 17
    blocks, powers = [(0, 0, "real")], {}
    for a_n in sorted(tin):
        for m in sorted(tout):
            if a_n == 0 and m == 0:
                continue
            blocks.append((a_n, m, "linear")); powers[(a_n, m, "linear")] = abs(m - a_n)
            if a_n and m:
                blocks.append((a_n, m, "antilinear")); powers[(a_n, m, "antilinear")] = m + a_n
    fplan = ff.plan_blocks(blocks, FieldType(tout), powers)
    fdesc = torch.tensor([b.row() for b in fplan.blocks], dtype=torch.int32, device=dev)
    h, zc, zr = rnd(e, kk - 1), rnd(n, kk, fplan.wc, 2), rnd(n, kk, fplan.wr)
    order, gptr, gsrc = ff.source_groups(geo.source)
    fext = ff.extension(True)
    fa_args = (h, zc, zr, geo.angular, geo.transport, geo.rho, fdesc, geo.source, order, gptr, gsrc)
    rows = fext.forward(*fa_args, fplan.d_out, fplan.max_bm)
    grow = rnd(e, fplan.d_out)
    zbytes = n * kk * (2 * fplan.wc + fplan.wr) * 4
    ftab = e * (2 * geo.transport.shape[1] * 2 * 4 + 4 + 8 + 8)
    timed("factored_forward", lambda: fext.forward(*fa_args, fplan.d_out, fplan.max_bm), e * (kk - 1) * 4 + zbytes + ftab + e * fplan.d_out * 4)
    timed("factored_aggregate", lambda: fext.aggregate(rows, geo.weights, geo.row_ptr), e * (fplan.d_out + 1) * 4 + n * fplan.d_out * 4)
    timed("factored_backward", lambda: fext.backward(grow, *fa_args), 2 * e * (kk - 1) * 4 + 2 * zbytes + ftab + e * fplan.d_out * 4)
    del h, zc, zr, rows, grow
    # pair term 8 -> 8 linear block, trunk 16, complex matrix
    a_, b_, t_ = 8, 8, 16
    pext = fp.extension()
    hidden, weight, bias = rnd(e, t_), rnd(2 * a_ * b_, t_), rnd(2 * a_ * b_)
    u = torch.view_as_complex(rnd(e, a_, 2))
    pre, post = geo.angular[:, 1].contiguous(), geo.angular[:, 2].contiguous()
    pre_c, post_c = torch.view_as_complex(pre), torch.view_as_complex(post)
    out = torch.view_as_complex(torch.zeros(e, b_, 2, device=dev))
    timed("pairs_forward", lambda: pext.forward(hidden, weight, bias, u, pre_c, post_c, geo.rho, out, a_, b_, 1),
          e * (t_ + 2 * a_ + 4 + 1 + 4 * b_) * 4)
    gu, gh, gk = torch.zeros_like(u), torch.zeros_like(hidden), torch.empty(2 * a_ * b_, e, device=dev)
    gout = torch.view_as_complex(rnd(e, b_, 2))
    timed("pairs_backward", lambda: pext.backward(hidden, weight, bias, u, pre_c, post_c, geo.rho, gout, gu, gh, gk, a_, b_, 1),
          e * (3 * t_ + 6 * a_ + 4 + 1 + 2 * b_ + 2 * a_ * b_) * 4)
    line = {"workload": f"op-level entry points, {nlat}x{nlon} lattice, radius 3pi/{nlat}, {e} edges, fp32", "hbm_peak_GB/s": peak, "ops": results}
    if emit:
        print(json.dumps(line))
    return line


def run_conv(args: argparse.Namespace, emit: bool = True) -> dict:
    """Depthwise steerable convolution, forward + backward, with its radial network: 256 x 512 lattice, radius 4 pi / 256,
    batch 4, field type 64 x (m = 0, 1, 2) (D = 320, a_0 = 64, W = 512; 22 999 040 edges per sample), radial network of 4
    Gaussians -> 16 -> (64 | 512).  One step = radial network on the table entries, fold, apply, and the backward of all
    three (field gradient, table gradient, network gradients).  Single GPU."""
    import numpy as np
    import torch

    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa
    from gm_attention_b200.nn.lattice_depthwise import RadialCoefficients, _apply, _table_gradient, conv_tables, fold, lattice_depthwise

    nlat, nlon, batch, copies = (256, 512, 4, 64) if args.workload == "conv" else (128, 256, 4, 64)
    radius = 4 * math.pi / nlat
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    elem = 2 if args.dtype == "bf16" else 4
    head = FieldType({0: copies, 1: copies, 2: copies})
    D, a0, w = head.dimension, copies, 8 * copies
    lattice = midpoint_lattice(nlat, nlon, device)
    edges = compute_edge_geometry(lattice, lattice.frames, radius, max_frequency=4, dtype=torch.float32)
    geo = fa.geometry(edges, radius, "hard", torch.float32)
    owner = type("Layer", (), {})()
    plan = fa._plan(owner, head, head, 1)
    tables = conv_tables(geo, edges.distances.float(), geo.weights, plan.rows, nlat, nlon)
    e1, n1 = edges.n_edges, nlat * nlon
    del edges, geo
    torch.manual_seed(0)
    net = RadialCoefficients(a0, w, radius, n_radial_basis=4, radial_hidden_features=(16,), device=device)
    gen = torch.Generator().manual_seed(0)
    host = [torch.randn(batch * n1, D, generator=gen).to(dtype).pin_memory() for _ in range(2)]
    v, g = (h.to(device) for h in host)
    v.requires_grad_(True)
    peak, peak_kind = 6650.0, "fallback"
    try:
        peak, peak_kind = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        pass

    def step():
        v.grad = None
        net.zero_grad(set_to_none=True)
        rc, cc = net(tables.distances)
        y = lattice_depthwise(v, rc, cc, tables)
        y.backward(g)
        return y.detach(), v.grad

    for _ in range(max(args.warmup, 3)):
        y, dv = step()
    torch.cuda.synchronize()

    # ---- parity: sampled targets / sources of the last sample against the CPU oracle of the reference's depthwise op,
    # fed with this step's own coefficients expanded to the sampled edges
    parity = None
    if not args.no_parity:
        from oracle import geometry_np as GN
        from oracle import sampled as SP

        with torch.no_grad():
            rc_t, cc_t = net(tables.distances)
        lat = tables.lattice
        t_rows = [0, 1, 4, 9, nlat // 2, nlat - 1]
        targets = np.array([r * nlon + c for r in t_rows for c in (0, nlon - 1, nlon // 2 + 1)], np.int64)
        sources = np.array([9 * nlon, (nlat // 2) * nlon + nlon - 1], np.int64)
        sample = SP.sample_problem(GN.midpoint_lattice(nlat, nlon), radius, targets, sources, 4, np.float32)
        span = 2 * lat.halo + 1
        cnt, lo, off = (x.cpu().numpy().reshape(-1) for x in (lat.win_cnt, lat.win_lo, lat.win_off))
        tgt, src = np.repeat(sample.nodes, np.diff(sample.row_ptr)), sample.nodes[sample.source_index]
        win = (tgt // nlon) * span + (src // nlon - tgt // nlon + lat.halo)
        entry = torch.from_numpy(off[win] + (src % nlon - tgt % nlon - lo[win]) % nlon).to(device)
        b = batch - 1
        pick = lambda x, nodes: x[torch.from_numpy(b * n1 + nodes).to(device)].float().cpu().numpy()
        want = SP.run_conv(sample, pick(v.detach(), sample.nodes), pick(g, sample.nodes), rc_t[entry].float().cpu().numpy(),
                           cc_t[entry].float().cpu().numpy(), np.array(plan.rows, np.int64), radius, a0, w)
        got = {"out": pick(y, sample.targets), "dv": pick(dv, sample.sources)}
        errs = {n: float(np.abs(got[n] - want[n]).max() / max(float(np.abs(want[n]).max()), 1e-30)) for n in got}
        tolerance = 2e-2 if args.dtype == "bf16" else 2e-5
        parity = {"max_rel": max(errs.values()), "per_tensor": errs, "tolerance": tolerance, "targets": int(targets.shape[0]),
                  "sources": int(sources.shape[0]), "oracle_edges": sample.n_edges,
                  "against": "CPU oracle of the reference's depthwise op (C restatement pinned to its compiled driver), float32, on the same "
                             "rounded inputs, per-edge coefficients = this step's table entries"}
        if not parity["max_rel"] < tolerance:
            print(json.dumps({"error": "parity check failed", "parity": parity}), file=sys.stderr)
            sys.exit(3)

    clocks = ClockSampler(0)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with clocks:
        torch.cuda.synchronize()
        for a_ev, b_ev in ev:
            a_ev.record()
            step()
            b_ev.record()
        torch.cuda.synchronize()
    ms_step = statistics.mean(a.elapsed_time(b) for a, b in ev)

    # ---- the three kernels alone
    with torch.no_grad():
        table = fold(*net(tables.distances), tables)
        t_table = table.index_select(0, tables.lattice.t_entry)
        kernels = {"apply (forward)": lambda: _apply(v.detach(), table, tables, False),
                   "apply, transposed (field gradient)": lambda: _apply(g, t_table, tables, True),
                   "table_grad": lambda: _table_gradient(g, v.detach(), tables)}
        kernel_ms = {}
        for name, fn in kernels.items():
            fn()
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(5)]
            for a_ev, b_ev in pairs:
                a_ev.record(); fn(); b_ev.record()
            torch.cuda.synchronize()
            kernel_ms[name] = statistics.mean(a.elapsed_time(b) for a, b in pairs)
    top = max(kernel_ms, key=kernel_ms.get)
    n_nodes, total_edges = batch * n1, batch * e1
    table_bytes = table.numel() * 4
    bytes_of = {"apply (forward)": 2 * n_nodes * D * elem + table_bytes, "apply, transposed (field gradient)": 2 * n_nodes * D * elem + table_bytes,
                "table_grad": 2 * n_nodes * D * elem + table_bytes}
    flops_pass = 2.0 * (a0 + 4 * 2 * copies) * total_edges
    achieved = bytes_of[top] / (kernel_ms[top] * 1e-3) / 1e9

    # ---- end to end from pinned host buffers: v and g in, y and dv out, every step
    e2e = None
    if not args.no_e2e:
        outs = [torch.empty_like(host[0]).pin_memory() for _ in range(2)]
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(max(3, args.steps // 2))]
        for a_ev, b_ev in pairs:
            a_ev.record()
            with torch.no_grad():
                v.copy_(host[0], non_blocking=True)
                g.copy_(host[1], non_blocking=True)
            y, dv = step()
            outs[0].copy_(y, non_blocking=True)
            outs[1].copy_(dv, non_blocking=True)
            b_ev.record()
        torch.cuda.synchronize()
        e_ms = statistics.mean(a.elapsed_time(b) for a, b in pairs[1:])
        e2e = {"value": total_edges / (e_ms * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": 2 * n_nodes * D * elem,
               "d2h_bytes_per_step": 2 * n_nodes * D * elem, "ms_per_step": e_ms, "steps": len(pairs) - 1}

    cpu = None
    if not args.no_cpu_baseline:
        from oracle import geometry_np as GN
        from oracle import sampled as SP

        row = nlat // 4
        whole = SP.sample_problem(GN.midpoint_lattice(nlat, nlon), radius, row * nlon + np.arange(nlon, dtype=np.int64), np.zeros(0, np.int64), 4, np.float32)
        rng = np.random.default_rng(0)
        cv, cg = (rng.standard_normal((whole.nodes.shape[0], D)).astype(np.float32) for _ in range(2))
        crc, ccc = rng.standard_normal((whole.n_edges, a0)).astype(np.float32), rng.standard_normal((whole.n_edges, w)).astype(np.float32)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            SP.run_conv(whole, cv, cg, crc, ccc, np.array(plan.rows, np.int64), radius, a0, w)
            reps += 1
        seconds = time.perf_counter() - t0
        cpu = {"value": reps * whole.n_edges / seconds, "unit": "edges/s", "cores": 1, "kind": "port",
               "sample": f"all {nlon} targets of lattice row {row} of one sample ({whole.n_edges} edges), float32, forward + backward of the depthwise op "
                         f"with per-edge coefficients given (the reference's radial network per edge is NOT timed), {reps} repetitions", "seconds": seconds}

    line = {
        "metric": "depthwise-conv fwd+bwd neighbour-edges/sec", "value": total_edges / (ms_step * 1e-3), "unit": "edges/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"depthwise steerable convolution fwd+bwd with its radial network, {nlat}x{nlon} midpoint equiangular lattice, radius "
                               f"4pi/{nlat}, batch {batch}, {copies}x(m=0,1,2), D={D}, a0={a0}, W={w}, {e1} edges per sample, {tables.n_entries} table entries",
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (no flush needed)"},
        "roofline": {"bound": "hbm", "kernel": f"conv kernel: {top}", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "algorithmic_bytes_per_launch": bytes_of[top], "launch_ms": kernel_ms[top],
                     "kernels_ms": kernel_ms, "fp32_fma_tflops_per_kernel": {k: flops_pass / (ms * 1e-3) / 1e12 for k, ms in kernel_ms.items()},
                     "note": "FMA-bound by construction: 4 multiply-adds per complex copy, edge and sample against ~0.01 B of compulsory traffic"},
        "gpu_launches": args.steps * 3, "clocks": clocks.summary(), "e2e": e2e, "parity": parity, "cpu_baseline": cpu}
    if emit:
        print(json.dumps(line))
    return line


def main() -> None:
    args = parse()
    if args.workload in ("conv", "conv-mid"):
        if args.impl == "reference" or args.gpus > 1:
            print(json.dumps({"impl": args.impl, "unavailable": "the depthwise workload is measured on one GPU, its CPU figure is the cpu_baseline of that line"}))
            return
        run_conv(args)
        return
    if args.workload == "ops":
        run_ops(args)
        return
    cfg = dict({"headline": HEADLINE, "mid": MID, "small": SMALL}[args.workload])
    if args.radius_rows is not None:
        cfg["radius_rows"] = args.radius_rows
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
