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

from featgraph_b200 import graphs  # noqa: E402

FEAT = 64
METRIC = "spmm_plus_sddmm_fp32_feat64_gflops"
UNIT = "GFLOP/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the default workload, from one
# ncu capture (profiles/bench_full_size_launch_list_and_dram.md); other sizes report null.
NCU_TRAFFIC_BYTES = {"spmm": 1843.2e6 + 199.2e6, "sddmm": 1908.2e6 + 891.2e6}
FALLBACK_HBM_GBS = 6650.0


def spmm_alg_bytes(n_rows, nnz, f):
    """indptr + indices + values + every gathered X row + Y."""
    return 4 * (n_rows + 1) + 8 * nnz + 4 * nnz * f + 4 * n_rows * f


def sddmm_alg_bytes(nnz, f, heads=1):
    """row + col + both gathered rows of every edge + out."""
    return 8 * nnz + 8 * nnz * f + 4 * nnz * heads


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
    threads = fg_oracle.max_threads()
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


# ------------------------------------------------------------------------- our GPU arm --

def run_gpu(args):
    import torch.distributed as dist
    from featgraph_b200.distributed import ShardedSDDMM, ShardedSpMM

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
        # NCCL prints its version banner on stdout at NCCL_DEBUG=VERSION; the contract of this
        # script is one JSON line on stdout
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)

    g, x, y2 = make_inputs(args, device)
    adj = g.to_scipy()
    rows_dev = g.coo_rows()
    n, nnz = g.n_rows, g.nnz

    fused = not args.nccl_gather
    spmm = ShardedSpMM(adj, FEAT, device, fused_gather=fused)
    sddmm = ShardedSDDMM(rows_dev, g.indices, n, g.n_cols, FEAT, device, fused_gather=fused,
                         peer_mode=args.peer_mode)
    stream = torch.cuda.current_stream(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def step(events=None):
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
    if spmm.module.device_status() != 0:      # raises if a bounded device-side wait gave up
        raise SystemExit("SpMM reported a device-side error")
    total_ms = events[0][0].elapsed_time(events[-1][-1])
    phases = np.array([[m[i].elapsed_time(m[i + 1]) for i in range(4)] for m in events])
    clocks = sampler.summary(t0, t1)

    # ---- end to end from pinned host buffers, through run_host ----------------------------
    x_host = torch.empty((g.n_cols, FEAT), dtype=torch.float32, pin_memory=True).copy_(x)
    y2_host = torch.empty((g.n_cols, FEAT), dtype=torch.float32, pin_memory=True).copy_(y2)
    y_host = torch.empty((n, FEAT), dtype=torch.float32, pin_memory=True)
    o_host = torch.empty((nnz,), dtype=torch.float32, pin_memory=True)
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        spmm.run_host(x_host, y_host)
        sddmm.run_host(y2_host, x_host, o_host)
    barrier()
    a = _mark(stream)
    for _ in range(e2e_steps):
        spmm.run_host(x_host, y_host)
        sddmm.run_host(y2_host, x_host, o_host)
    b = _mark(stream)
    barrier()
    e2e_ms = a.elapsed_time(b)
    sampler.stop()

    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = float(t[0]), float(t[1])
        ph = torch.tensor(phases.mean(axis=0), device=device, dtype=torch.float64)
        dist.all_reduce(ph, op=dist.ReduceOp.MAX)
        phase_ms = ph.cpu().numpy()
    else:
        phase_ms = phases.mean(axis=0)

    flops_step = 2 * 2.0 * nnz * FEAT
    ms_per_step = total_ms / args.steps
    value = flops_step / (ms_per_step * 1e-3) / 1e9
    e2e_value = flops_step / (e2e_ms / e2e_steps * 1e-3) / 1e9

    if rank == 0:
        peak, peak_kind = measured_peak()
        local_spmm_bytes = spmm_alg_bytes(spmm.row_hi - spmm.row_lo, spmm.local_nnz, FEAT)
        local_sddmm_bytes = sddmm_alg_bytes(sddmm.edge_hi - sddmm.edge_lo, FEAT)
        spmm_ms, sddmm_ms = float(phase_ms[0]), float(phase_ms[2])

        default_size = (world == 1 and n == graphs.REDDIT_NUM_VERTICES
                        and abs(nnz - graphs.REDDIT_NUM_EDGES) < 0.01 * graphs.REDDIT_NUM_EDGES)

        def traffic(kernel):
            return int(NCU_TRAFFIC_BYTES[kernel]) if default_size else None

        def roof(alg_bytes, ms, traffic):
            ach = alg_bytes / (ms * 1e-3) / 1e9
            return {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s",
                    "frac": round(ach / peak, 4), "peak_kind": peak_kind,
                    "frac_of_nominal_8TBs": round(ach / NOMINAL_HBM_GBS, 4),
                    "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": round(ms, 4),
                    "traffic": traffic}

        kernels = {
            "spmm": dict(roof(local_spmm_bytes, spmm_ms, traffic("spmm")),
                         kernels="spmm_giant_kernel + spmm_heavy_kernel + spmm_light_kernel "
                                 "(three concurrent streams)",
                         gflops=round(2.0 * spmm.local_nnz * FEAT / (spmm_ms * 1e-3) / 1e9, 1),
                         gather_ms=round(float(phase_ms[1]), 4)),
            "sddmm": dict(roof(local_sddmm_bytes, sddmm_ms, traffic("sddmm")),
                          kernels="sddmm_tile_kernel",
                          gflops=round(2.0 * (sddmm.edge_hi - sddmm.edge_lo) * FEAT
                                       / (sddmm_ms * 1e-3) / 1e9, 1),
                          gather_ms=round(float(phase_ms[3]), 4)),
        }
        dominant = "sddmm" if sddmm_ms >= spmm_ms else "spmm"
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(g), "graph_seed": graphs.GRAPH_SEED,
                       "degree": g.degree_stats(), "parallelism":
                           "spmm: nnz-balanced row blocks; sddmm: edge ranges; x%d; outputs "
                           "assembled by %s (spmm) / %s (sddmm)" % (world, spmm.gather_mode,
                                                                    sddmm.gather_mode),
                       "l2": "adjacency streams (0.9 GB per kernel) exceed L2 between launches; "
                             "no explicit flush"},
            "e2e": {"value": round(e2e_value, 1), "unit": UNIT,
                    "h2d_bytes_per_step": int(world * 3 * g.n_cols * FEAT * 4),
                    "d2h_bytes_per_step": int(n * FEAT * 4 + nnz * 4),
                    "ms_per_step": round(e2e_ms / e2e_steps, 3), "steps": e2e_steps},
            "gpu_launches": int(args.steps * (spmm.num_launches() + sddmm.num_launches())),
            "clocks": clocks,
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
    del g
    from oracle import fg_oracle
    fg_oracle.build()
    threads = fg_oracle.max_threads()

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
        "config": {"workload": "powerlaw_chung_lu_zipf2.1 N=%d nnz=%d feat_len=%d fp32: CSR "
                               "SpMM + COO SDDMM (synthetic stand-in for the Reddit graph)"
                               % (n_rows, nnz, FEAT),
                   "note": "CPU port of the reference's x86 kernels (TVM v0.7 cannot be "
                           "installed); throughput on a bounded sample of the workload"},
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
    ap.add_argument("--peer-mode", choices=["auto", "store", "push"], default="auto",
                    help="how SDDMM results reach the peers (see ShardedSDDMM)")
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
