#!/usr/bin/env python
"""Benchmark of the SpMM / SDDMM hot path at feat_len 64 on the power-law graph.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One STEP = one CSR SpMM (Y = A.X) followed by one COO SDDMM
(out[e] = dot(X[row[e]], Y2[col[e]])) on the same synthetic 232 965-vertex / ~114.6 M-edge
power-law graph, fp32, feat_len 64.  The line printed by rank 0 carries the whole-job
GFLOP/s (`value`), the same thing measured end to end from pinned host buffers (`e2e`), the
roofline of the dominant kernel and a CPU baseline (the oracle port on the host cores).

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the SAME graph is
split across the ranks -- SpMM by nnz-balanced row blocks, SDDMM by edge ranges -- and the
outputs are all-gathered over NCCL inside the timed region (strong scaling).

--impl reference times the CPU restatement of the reference's x86 kernels (oracle/) on the
host cores instead; TVM, which the reference needs to generate its kernels, is not
installable, so that port is the only runnable form of the reference here.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from featgraph_b200 import _lib, graphs  # noqa: E402

FEAT = 64
METRIC = "spmm_plus_sddmm_fp32_feat64_gflops"
UNIT = "GFLOP/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the default workload on one GPU.
# STATIC figures from one ncu capture (they do not follow later kernel changes until the
# capture is repeated); other sizes and world sizes report null.
NCU_TRAFFIC_BYTES = {"spmm": 1494.9e6 + 55.6e6, "sddmm": 1417.8e6 + 449.7e6}
NCU_TRAFFIC_SOURCE = ("static: one ncu capture (dram__bytes_read.sum + dram__bytes_write.sum, 1 pass) "
                      "of the full-size 1-GPU workload, summarised in "
                      "profiles/bench_full_size_launch_list_and_dram.md; it does not follow later "
                      "kernel changes until that capture is repeated")
FALLBACK_HBM_GBS = 6650.0


def spmm_alg_bytes(n_rows, nnz, f):
    """indptr + indices + values + every gathered X row + Y."""
    return 4 * (n_rows + 1) + 8 * nnz + 4 * nnz * f + 4 * n_rows * f


def sddmm_alg_bytes(nnz, f, heads=1):
    """row + col + both gathered rows of every edge + out."""
    return 8 * nnz + 8 * nnz * f + 4 * nnz * heads


def spmm_l2_bytes(n_rows, nnz, f):
    """Bytes that have to cross the L2 -> SM path: structure, one gathered X row per nonzero,
    and Y once."""
    return 8 * nnz + 4 * nnz * f + 4 * n_rows * f


def sddmm_l2_bytes(n_rows, nnz, f, heads=1):
    """The same for SDDMM on a row-sorted edge list: the src row of every edge, but the dst
    row only once per run of equal rows (bounded below by once per row), and the output."""
    return 8 * nnz + 4 * nnz * f + 4 * n_rows * f + 4 * nnz * heads


def host_threads():
    """Threads the CPU legs use: the cores this process may run on, NOT the inherited
    OMP_NUM_THREADS (torch.distributed.run exports OMP_NUM_THREADS=1 to every rank)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def config_block(n_rows, nnz, degree):
    """`config` of the JSON line: identical in the GPU arm and the reference arm."""
    return {"workload": ("powerlaw_chung_lu_zipf2.1 N=%d nnz=%d feat_len=%d fp32: CSR SpMM + "
                         "COO SDDMM (synthetic stand-in for the Reddit graph)"
                         % (n_rows, nnz, FEAT)),
            "graph_seed": graphs.GRAPH_SEED, "degree": degree,
            "l2": "inputs larger than L2: each kernel streams 0.9 GB of adjacency (7 x L2) "
                  "between uses of anything; no explicit flush"}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------ clocks --

class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML while the timed
    region runs (read-only queries)."""

    REASONS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20),
               ("hw_thermal_slowdown", 0x40), ("hw_power_brake", 0x80),
               ("applications_clocks", 0x2), ("sync_boost", 0x10), ("display_clocks", 0x100))

    def __init__(self, device_index, period=0.01):
        super().__init__(daemon=True)
        self.period = period
        self.samples = []       # (t, sm_mhz, reasons bitmask, power W)
        self.sm_max = None
        self._halt = threading.Event()
        self.handle = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception as exc:      # no NVML: the line then says so
            self.error = repr(exc)

    def run(self):
        if self.handle is None:
            return
        nv = self.nv
        while not self._halt.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                watts = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.samples.append((time.perf_counter(), mhz, mask, watts))
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)

    def summary(self, t0, t1):
        if self.handle is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [],
                    "note": "NVML unavailable: " + getattr(self, "error", "?")}
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-3:]
        mask = 0
        for s in inside:
            mask |= s[2]
        return {"sm_mhz": statistics.median(s[1] for s in inside) if inside else None,
                "sm_max_mhz": self.sm_max, "samples": len(inside),
                "power_w_max": round(max((s[3] for s in inside), default=0.0), 1),
                "reasons": [name for name, bit in self.REASONS if mask & bit]}


# --------------------------------------------------------------------------- CPU oracle --

def cpu_oracle_rates(csr_host, rows_host, x_host, y2_host, budget_s):
    """Times the oracle port (all host threads) on a bounded sample of the workload.

    SpMM: a contiguous block of rows; SDDMM: a contiguous range of edges; both sized from a
    short probe so that each measurement takes about budget_s / 2.  Returns per-kernel and
    combined GFLOP/s plus a description of the sample."""
    from oracle import fg_oracle
    fg_oracle.build()
    threads = host_threads()
    fg_oracle.set_threads(threads)
    indptr, indices, vals = csr_host
    n_rows, nnz, f = indptr.shape[0] - 1, indices.shape[0], x_host.shape[1]

    def spmm_block(rows):
        sub_ptr = (indptr[:rows + 1] - indptr[0]).astype(np.int32)
        e1 = int(indptr[rows])
        work = np.empty((rows + x_host.shape[0]) * f, np.float32)
        out = np.empty((rows, f), np.float32)
        t = time.perf_counter()
        fg_oracle.spmm_csr_f32(sub_ptr, indices[:e1], vals[:e1], x_host, out=out, work=work)
        return time.perf_counter() - t, e1

    def sddmm_range(edges, parallel):
        out = np.empty((edges, 1), np.float32)
        t = time.perf_counter()
        # reference operand order: SrcFeat is indexed by col, DstFeat by row
        fg_oracle.sddmm_coo_f32(rows_host[:edges], indices[:edges], y2_host, x_host,
                                parallel=parallel, out=out)
        return time.perf_counter() - t

    probe_rows = max(1, n_rows // 64)
    t_probe, e_probe = spmm_block(probe_rows)
    rate = e_probe / max(t_probe, 1e-6)
    want_edges = min(nnz, max(e_probe, int(rate * budget_s / 2)))
    rows = int(np.searchsorted(indptr, want_edges, side="right") - 1)
    rows = min(max(rows, probe_rows), n_rows)
    t_spmm, e_spmm = spmm_block(rows)

    probe_edges = max(1, nnz // 256)
    t_probe = sddmm_range(probe_edges, True)
    edges = int(min(nnz, max(probe_edges, probe_edges / max(t_probe, 1e-6) * budget_s / 2)))
    t_sddmm = sddmm_range(edges, True)
    serial_edges = max(1, min(edges, nnz // 64))
    t_serial = sddmm_range(serial_edges, False)

    spmm_gflops = 2.0 * e_spmm * f / t_spmm / 1e9
    sddmm_gflops = 2.0 * edges * f / t_sddmm / 1e9
    # one step = one SpMM + one SDDMM over all nnz edges; extrapolate the sample rates
    step_s = (2.0 * nnz * f / 1e9) / spmm_gflops + (2.0 * nnz * f / 1e9) / sddmm_gflops
    return {
        "value": round(2 * 2.0 * nnz * f / 1e9 / step_s, 3), "unit": UNIT, "cores": threads,
        "kind": "port",
        "sample": "SpMM: first %d rows (%d nnz, %.2f s); SDDMM: first %d edges (%.2f s); "
                  "rates extrapolated to the full step" % (rows, e_spmm, t_spmm, edges, t_sddmm),
        "spmm_gflops": round(spmm_gflops, 3), "sddmm_gflops_all_threads": round(sddmm_gflops, 3),
        "sddmm_gflops_one_thread_as_reference_schedule":
            round(2.0 * serial_edges * f / t_serial / 1e9, 3),
        "est_step_ms": round(step_s * 1e3, 1),
    }


# ----------------------------------------------------------------------------- helpers --

def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def make_inputs(args, device):
    g = graphs.powerlaw_graph(n=args.vertices, nnz_target=args.edges, seed=graphs.GRAPH_SEED,
                              device=device)
    x = graphs.normal_features(g.n_cols, FEAT, graphs.FEAT_SEED, device)
    y2 = graphs.normal_features(g.n_cols, FEAT, graphs.FEAT2_SEED, device)
    return g, x, y2


def workload_name(g):
    return ("powerlaw_chung_lu_zipf2.1 N=%d nnz=%d feat_len=%d fp32: CSR SpMM + COO SDDMM "
            "(synthetic stand-in for the Reddit graph)" % (g.n_rows, g.nnz, FEAT))


# ------------------------------------------------------------------------------ parity --

def parity_check(adj, rows_dev, x, y2, spmm, sddmm, world, rank):
    """Bit-for-bit comparison of sampled parts of the FULL outputs held by this rank --
    its own block and the blocks written by its peers -- with the CPU oracle.

    SpMM: the 24 longest rows, 3 000 random rows and the rows on both sides of every shard
    boundary.  SDDMM: windows of 50 000 edges, one at the start of every rank's range (so
    every writer is covered), one straddling every range boundary, and four random ones.
    Returns (rows checked, edges checked, mismatching values)."""
    from oracle import fg_oracle
    fg_oracle.build()
    fg_oracle.set_threads(max(1, host_threads() // world))
    x_h, y2_h = x.cpu().numpy(), y2.cpu().numpy()
    indptr = adj.indptr
    deg = np.diff(indptr)
    n_rows, nnz = adj.shape[0], int(adj.nnz)
    rng = np.random.default_rng(1234)          # the same picks on every rank
    near = np.concatenate([[b - 1, b] for b in spmm.bounds[1:-1]]) if world > 1 else []
    picks = np.unique(np.concatenate([np.argsort(deg)[-24:], rng.integers(0, n_rows, 3000),
                                      np.asarray(near, dtype=np.int64)]))
    picks = picks[(picks >= 0) & (picks < n_rows)].astype(np.int64)
    sub_ptr = np.concatenate(([0], np.cumsum(deg[picks]))).astype(np.int32)
    sel = np.concatenate([np.arange(indptr[r], indptr[r + 1]) for r in picks])
    want = fg_oracle.spmm_csr_f32(sub_ptr, adj.indices[sel], adj.data[sel], x_h,
                                  n_cols=adj.shape[1])
    got = spmm.out[torch.from_numpy(picks).to(spmm.out.device)].cpu().numpy()
    bad = int((want.view(np.int32) != got.view(np.int32)).sum())

    win = 50000
    starts = [int(b) for b in sddmm.bounds[:-1]]
    starts += [max(0, int(b) - win // 2) for b in sddmm.bounds[1:-1]]
    starts += [int(v) for v in rng.integers(0, max(1, nnz - win), 4)]
    rows_h = None
    edges = 0
    for s0 in sorted(set(starts)):
        s1 = min(nnz, s0 + win)
        if s1 <= s0:
            continue
        rows_h = rows_dev[s0:s1].cpu().numpy()
        want = fg_oracle.sddmm_coo_f32(rows_h, adj.indices[s0:s1], y2_h, x_h, parallel=True)
        got = sddmm.out[s0:s1].cpu().numpy()
        bad += int((want.view(np.int32) != got.view(np.int32)).sum())
        edges += s1 - s0
    return int(picks.shape[0]), int(edges), bad


# ---------------------------------------------------------------------- L2 gather peak --

def l2_gather_peak(device, n_rows):
    """GB/s at which the L2 -> SM path delivers gathered rows of a table that fits L2 (the
    size of X at feat_len 64): the library's gather-only probe kernel, 256-byte and 128-byte
    rows at pseudo-random indices, 16-byte loads, eight in flight per lane; CUDA events,
    best of 5 after warm-up."""
    import ctypes
    from featgraph_b200 import _lib
    lib = _lib.load()
    table = torch.randn(n_rows, 64, device=device)
    sink = torch.zeros(1, device=device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    stream = torch.cuda.current_stream(device)
    out = {}
    for row_floats in (64, 32):
        groups_per_block = 256 // (row_floats // 4)
        n_blocks, rows_per_group = sms * 8, 2048
        rows_tbl = n_rows * 64 // row_floats

        def launch():
            _lib.check(lib.fg_gather_probe(
                ctypes.c_void_p(table.data_ptr()), rows_tbl, row_floats, rows_per_group, n_blocks,
                ctypes.c_void_p(sink.data_ptr()), device.index or 0,
                ctypes.c_void_p(stream.cuda_stream)))
        for _ in range(3):
            launch()
        best = None
        for _ in range(5):
            a = _mark(stream)
            launch()
            b = _mark(stream)
            b.synchronize()
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
        total = n_blocks * groups_per_block * rows_per_group * row_floats * 4
        out[row_floats] = total / (best * 1e-3) / 1e9
    return out


# ------------------------------------------------------------------------- our GPU arm --

def run_gpu(args):
    import torch.distributed as dist
    from featgraph_b200.distributed import OverlappedPair, ShardedSDDMM, ShardedSpMM

    rank, world, local = dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torch.distributed.run with %d ranks"
                             % (args.gpus, args.gpus))
        args.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path "
                         "(--impl reference times the CPU oracle)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        # At NCCL_DEBUG=VERSION NCCL prints its version banner on stdout, and the contract of
        # this script is one JSON line there; that level carries nothing else, so it alone is
        # lowered.  Any other setting (INFO, ...) is the caller's and stays.
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)

    g, x, y2 = make_inputs(args, device)
    adj = g.to_scipy()
    rows_dev = g.coo_rows()
    n, nnz = g.n_rows, g.nnz

    fused = not args.nccl_gather
    spmm = ShardedSpMM(adj, FEAT, device, fused_gather=fused, peer_mode=args.peer_mode)
    sddmm = ShardedSDDMM(rows_dev, g.indices, n, g.n_cols, FEAT, device, fused_gather=fused,
                         peer_mode=args.peer_mode)
    pair = OverlappedPair(spmm, sddmm, order="split" if args.schedule == "split" else "chain")
    overlap = args.schedule in ("overlap", "split") or (args.schedule == "auto" and world > 1)
    stream = torch.cuda.current_stream(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def serial_step(events=None):
        """SpMM, then SDDMM, on one stream; five marks (SpMM kernels | its exchange | SDDMM
        kernel | its exchange)."""
        marks = []
        if events is not None:
            marks.append(_mark(stream))
        spmm.compute_local(x)
        if events is not None:
            marks.append(_mark(stream))
        spmm.gather()
        if events is not None:
            marks.append(_mark(stream))
        sddmm.compute_local(y2, x)          # SrcFeat (by col) = y2, DstFeat (by row) = x
        if events is not None:
            marks.append(_mark(stream))
        sddmm.gather()
        if events is not None:
            marks.append(_mark(stream))
            events.append(marks)

    def step(events=None):
        """One SpMM and one SDDMM.  'serial': as serial_step.  'overlap': one chain of
        programmatic launches with one barrier pair around both (OverlappedPair); only the
        step's own start and end are marked -- an event between the kernels would wait for
        the first one to complete and undo the overlap."""
        if not overlap:
            return serial_step(events)
        begin = _mark(stream) if events is not None else None
        pair.run(x, y2, x)                  # SrcFeat (by col) = y2, DstFeat (by row) = x
        if events is not None:
            events.append([begin, _mark(stream)])

    # Warm-up runs the very code of the timed loop (event records included), so that no
    # first-use cost (lazy module loading, event pools) lands inside the timed region.
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step([])
    barrier()

    events = []
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(events)
    barrier()
    t1 = time.perf_counter()
    spmm.device_status()                      # raises if a bounded device-side wait gave up
    sddmm.device_status()
    total_ms = events[0][0].elapsed_time(events[-1][-1])
    clocks = sampler.summary(t0, t1)
    if overlap:
        # the kernels' own durations: a second, serial pass over the same resident inputs
        # (not part of `value`; the overlapped step cannot be marked between its kernels)
        serial_events = []
        for _ in range(3):
            serial_step([])
        barrier()
        for _ in range(max(5, args.steps // 2)):
            serial_step(serial_events)
        barrier()
        phases = np.array([[m[i].elapsed_time(m[i + 1]) for i in range(4)]
                           for m in serial_events])
        pair.run(x, y2, x)                  # the outputs the parity check reads: the timed path's
        barrier()
    else:
        phases = np.array([[m[i].elapsed_time(m[i + 1]) for i in range(4)] for m in events])

    # ---- parity of what was just timed: sampled rows / edge windows of the full outputs ----
    par_rows, par_edges, par_bad = parity_check(adj, rows_dev, x, y2, spmm, sddmm, world, rank)

    # ---- end to end from pinned host buffers, through run_host ----------------------------
    x_host = torch.empty((g.n_cols, FEAT), dtype=torch.float32, pin_memory=True).copy_(x)
    y2_host = torch.empty((g.n_cols, FEAT), dtype=torch.float32, pin_memory=True).copy_(y2)
    y_host = torch.empty((n, FEAT), dtype=torch.float32, pin_memory=True)
    o_host = torch.empty((nnz,), dtype=torch.float32, pin_memory=True)
    e2e_steps = max(3, min(args.steps, 10))
    if world == 1:
        # one GPU: the two host-buffer calls side by side on two streams (HostPair), so that
        # one call's transfers overlap the other's kernels and the link runs both ways
        from featgraph_b200.pipeline import HostPair
        host_pair = HostPair(spmm.module, sddmm.module)

        def e2e_step():
            host_pair.run(x_host, y_host, y2_host, x_host, o_host)
    else:
        def e2e_step():
            spmm.run_host(x_host, y_host)
            sddmm.run_host(y2_host, x_host, o_host)
    for _ in range(2):
        e2e_step()
    barrier()
    a = _mark(stream)
    for _ in range(e2e_steps):
        e2e_step()
    b = _mark(stream)
    barrier()
    e2e_ms = a.elapsed_time(b)
    sampler.stop()
    # what came back to the host is the same result (this rank's blocks)
    e2e_bad = int((y_host[spmm.row_lo:spmm.row_hi].view(torch.int32)
                   != spmm.out[spmm.row_lo:spmm.row_hi].cpu().view(torch.int32)).sum())
    e2e_bad += int((o_host[sddmm.edge_lo:sddmm.edge_hi].view(torch.int32)
                    != sddmm.out[sddmm.edge_lo:sddmm.edge_hi].cpu().view(torch.int32)).sum())

    probe = None
    if rank == 0 and not args.no_l2_probe:
        probe = l2_gather_peak(device, n)

    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = float(t[0]), float(t[1])
        ph = torch.tensor(phases.mean(axis=0), device=device, dtype=torch.float64)
        dist.all_reduce(ph, op=dist.ReduceOp.MAX)
        phase_ms = ph.cpu().numpy()
        pb = torch.tensor([par_bad, e2e_bad, par_rows, par_edges], device=device,
                          dtype=torch.int64)
        dist.all_reduce(pb, op=dist.ReduceOp.SUM)
        par_bad, e2e_bad, par_rows, par_edges = (int(v) for v in pb)
    else:
        phase_ms = phases.mean(axis=0)

    flops_step = 2 * 2.0 * nnz * FEAT
    ms_per_step = total_ms / args.steps
    value = flops_step / (ms_per_step * 1e-3) / 1e9
    e2e_value = flops_step / (e2e_ms / e2e_steps * 1e-3) / 1e9

    if rank == 0:
        peak, peak_kind = measured_peak()
        local_rows, local_edges = spmm.row_hi - spmm.row_lo, sddmm.edge_hi - sddmm.edge_lo
        local_spmm_bytes = spmm_alg_bytes(local_rows, spmm.local_nnz, FEAT)
        local_sddmm_bytes = sddmm_alg_bytes(local_edges, FEAT)
        spmm_ms, sddmm_ms = float(phase_ms[0]), float(phase_ms[2])

        default_size = (world == 1 and n == graphs.REDDIT_NUM_VERTICES
                        and abs(nnz - graphs.REDDIT_NUM_EDGES) < 0.01 * graphs.REDDIT_NUM_EDGES)

        def traffic(kernel):
            return int(NCU_TRAFFIC_BYTES[kernel]) if default_size else None

        def roof(alg_bytes, ms, traffic, l2_bytes):
            ach = alg_bytes / (ms * 1e-3) / 1e9
            r = {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s",
                 "frac": round(ach / peak, 4), "peak_kind": peak_kind,
                 "frac_of_nominal_8TBs": round(ach / NOMINAL_HBM_GBS, 4),
                 "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": round(ms, 4),
                 "traffic": traffic,
                 "traffic_source": NCU_TRAFFIC_SOURCE if traffic is not None else None}
            if probe:
                l2_ach = l2_bytes / (ms * 1e-3) / 1e9
                r["roofline_l2"] = {
                    "bound": "l2_gather", "bytes_per_launch": l2_bytes,
                    "achieved": round(l2_ach, 1), "peak": round(probe[64], 1), "unit": "GB/s",
                    "frac_l2": round(l2_ach / probe[64], 4),
                    "peak_kind": "measured in this run: gather-only probe kernel, 256-byte rows "
                                 "at random indices of a table the size of X (fits L2)",
                    "peak_128_byte_rows": round(probe[32], 1)}
            return r

        kernels = {
            "spmm": dict(roof(local_spmm_bytes, spmm_ms, traffic("spmm"),
                              spmm_l2_bytes(local_rows, spmm.local_nnz, FEAT)),
                         kernels="spmm_chain_kernel (giant rows) + spmm_heavy_kernel + spmm_light_kernel "
                                 "(one stream, chained by programmatic dependent launches)",
                         gflops=round(2.0 * spmm.local_nnz * FEAT / (spmm_ms * 1e-3) / 1e9, 1),
                         gather_ms=round(float(phase_ms[1]), 4)),
            "sddmm": dict(roof(local_sddmm_bytes, sddmm_ms, traffic("sddmm"),
                               sddmm_l2_bytes(n, local_edges, FEAT)),
                          kernels=("sddmm_rowreg_kernel (dst operand in registers)"
                                   if getattr(getattr(sddmm, "module", None), "default_launch_flags", 0)
                                   & _lib.SDDMM_ROW_REGISTERS else "sddmm_tile_kernel"),
                          gflops=round(2.0 * local_edges * FEAT / (sddmm_ms * 1e-3) / 1e9, 1),
                          gather_ms=round(float(phase_ms[3]), 4)),
        }
        dominant = "sddmm" if sddmm_ms >= spmm_ms else "spmm"
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_block(n, nnz, g.degree_stats()),
            "parallelism": "spmm: nnz-balanced row blocks; sddmm: edge ranges; x%d; outputs "
                           "assembled by %s (spmm) / %s (sddmm); schedule: %s"
                           % (world, spmm.gather_mode, sddmm.gather_mode,
                              ("one chain of programmatic launches (%s) with one barrier pair per "
                               "step; the per-kernel times come from a separate serial pass"
                               % ("the SpMM's giant and heavy rows, the SDDMM, the SpMM's light rows"
                                  if pair.order == "split" else
                                  "SpMM, then the SDDMM dispatched under the tail of its giant rows"))
                              if overlap else
                              "SpMM, then SDDMM, on one stream"),
            "e2e": {"value": round(e2e_value, 1), "unit": UNIT,
                    "h2d_bytes_per_step": int(3 * g.n_cols * FEAT * 4),
                    "d2h_bytes_per_step": int(n * FEAT * 4 + nnz * 4),
                    "ms_per_step": round(e2e_ms / e2e_steps, 3), "steps": e2e_steps,
                    "note": "whole job: every replicated input crosses PCIe once (1/%d per rank, "
                            "exchanged over NVLink), every rank downloads its own block" % world
                            if world > 1 else "fg_*_host entry points on pinned host buffers, the "
                            "SpMM call and the SDDMM call issued side by side on two streams "
                            "(featgraph_b200.pipeline.HostPair)"},
            "gpu_launches": int(args.steps * (spmm.num_launches() + sddmm.num_launches()
                                              + (0 if world == 1 or not fused else
                                                 (2 if overlap else 4)))),
            "kernel_times": "a serial pass after the timed loop" if overlap else
                            "CUDA events inside the timed loop",
            "clocks": clocks,
            "parity": {"spmm_rows": par_rows, "sddmm_edges": par_edges, "mismatches": par_bad,
                       "e2e_mismatches": e2e_bad,
                       "how": "bit-for-bit against the CPU oracle on every rank's copy of the "
                              "full outputs, after the timed loop (sums over ranks)"},
            "roofline": dict(kernels[dominant], kernel=kernels[dominant]["kernels"]),
            "kernels": kernels,
            "cpu_baseline": None,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_oracle_rates(
                (adj.indptr, adj.indices, adj.data), rows_dev.cpu().numpy(), x.cpu().numpy(),
                y2.cpu().numpy(), args.cpu_budget)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if par_bad or e2e_bad:
        raise SystemExit("bench.py: %d sampled values differ from the oracle, %d host-side"
                         % (par_bad, e2e_bad))


def _mark(stream):
    ev = torch.cuda.Event(enable_timing=True)
    ev.record(stream)
    return ev


# ---------------------------------------------------------------------- reference arm --

def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    device = "cuda" if torch.cuda.is_available() else "cpu"   # generation only
    g, x, y2 = make_inputs(args, device)
    indptr, indices = g.indptr.cpu().numpy(), g.indices.cpu().numpy()
    vals, rows = g.vals.cpu().numpy(), g.coo_rows().cpu().numpy()
    x_h, y2_h = x.cpu().numpy(), y2.cpu().numpy()
    nnz = g.nnz
    degree = g.degree_stats()
    del g
    from oracle import fg_oracle
    fg_oracle.build()
    threads = host_threads()
    fg_oracle.set_threads(threads)

    # size the per-step sample from a probe so that warmup + steps fit the budget
    n_rows = indptr.shape[0] - 1
    probe_rows = max(1, n_rows // 64)
    e_probe = int(indptr[probe_rows])
    work = np.empty((n_rows + x_h.shape[0]) * FEAT, np.float32)
    t = time.perf_counter()
    fg_oracle.spmm_csr_f32((indptr[:probe_rows + 1]).astype(np.int32), indices[:e_probe],
                           vals[:e_probe], x_h, work=work)
    fg_oracle.sddmm_coo_f32(rows[:e_probe], indices[:e_probe], y2_h, x_h, parallel=True)
    rate = e_probe / max(time.perf_counter() - t, 1e-6)      # edges/s through both kernels
    total_steps = max(args.warmup, 3) + args.steps
    edges = int(min(nnz, max(e_probe, rate * args.reference_budget / total_steps)))
    rows_n = int(min(max(np.searchsorted(indptr, edges, side="right") - 1, 1), n_rows))
    edges = int(indptr[rows_n])
    sub_ptr = indptr[:rows_n + 1].astype(np.int32)
    y = np.empty((rows_n, FEAT), np.float32)
    out = np.empty((edges, 1), np.float32)

    def step():
        fg_oracle.spmm_csr_f32(sub_ptr, indices[:edges], vals[:edges], x_h, out=y, work=work)
        fg_oracle.sddmm_coo_f32(rows[:edges], indices[:edges], y2_h, x_h, parallel=True, out=out)

    for _ in range(max(args.warmup, 3)):
        step()
    t = time.perf_counter()
    for _ in range(args.steps):
        step()
    ms = (time.perf_counter() - t) * 1e3 / args.steps
    value = 2 * 2.0 * edges * FEAT / (ms * 1e-3) / 1e9
    sample = ("each step: oracle SpMM on the first %d rows + oracle SDDMM (edges split over "
              "threads) on the same %d of %d edges; %d threads" % (rows_n, edges, nnz, threads))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_block(n_rows, nnz, degree),
        "note": "CPU port of the reference's x86 kernels (TVM v0.7 cannot be installed); "
                "throughput on a bounded sample of the workload, %d host threads" % threads,
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads,
                         "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--vertices", type=int, default=graphs.REDDIT_NUM_VERTICES)
    ap.add_argument("--edges", type=int, default=graphs.REDDIT_NUM_EDGES)
    ap.add_argument("--cpu-budget", type=float, default=16.0,
                    help="seconds of CPU work for the cpu_baseline leg")
    ap.add_argument("--reference-budget", type=float, default=90.0,
                    help="seconds of CPU work for the whole --impl reference run")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--peer-mode", choices=["auto", "store", "mcast", "push"], default="auto",
                    help="how results reach the peers (see featgraph_b200.distributed)")
    ap.add_argument("--schedule", choices=["auto", "overlap", "split", "serial"], default="auto",
                    help="serial: SpMM then SDDMM; overlap: the two side by side in one chain of "
                         "programmatic launches (OverlappedPair); split: the same chain with the "
                         "SDDMM between the SpMM's long rows and its light rows; auto: serial on "
                         "one GPU (where overlapping gains nothing), overlap on several")
    ap.add_argument("--no-l2-probe", action="store_true",
                    help="skip the measurement of the L2 gather peak (roofline_l2)")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="assemble outputs with NCCL collectives instead of peer stores")
    args = ap.parse_args()
    if args.steps < 1:
        raise SystemExit("--steps must be at least 1")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
