#!/usr/bin/env python
"""Benchmark of the composed-format SpMM: GFLOP/s (2 * nnz * N / t) and HBM-roofline fraction.

    python bench.py [--gpus N --steps K --warmup W] [--workload powerlaw|zipf|uniform|skew|blocks]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # SciPy on the host cores, same metric and config

A step is one SpMM C = A B over the whole (row-sharded) matrix with the format and B resident in
HBM.  The default workload is the power-law graph (2^20 rows, N = 128).  Rank 0 prints one JSON
line.  Inputs are synthetic and seeded; B plus the format exceed the 126 MB L2, so consecutive
steps cannot be served from cache.  Without --workload the line also carries a `configs` object
with the other benchmark matrices (uniform N = 64, skew N = 256, blocks float32 / bf16 at
N = 32, 128, 512), each device-timed the same way and checked on sampled rows against SciPy.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from liteform_ae_b200 import synth  # noqa: E402
from oracle.hyb_oracle import spmm_prebuilt as cpu_spmm  # noqa: E402  (CPU legs only: the oracle's SciPy product)

METRIC = "spmm_gflops"
UNIT = "GFLOP/s"

WORKLOADS = {
    # name: (description, generator(rows) -> Csr, full rows, N)
    "zipf": ("config 1: 16384^2 Zipf(1.8) rows, mean 16 nnz/row", lambda m: synth.zipf_rows(M=m), 16384, 32),
    "powerlaw": ("config 2: 2^20 power-law graph, mean 14 nnz/row, row-normalised", lambda m: synth.power_law_graph(M=m), 1 << 20, 128),
    "uniform": ("config 3: 4194304^2, exactly 32 nnz/row", lambda m: synth.uniform_rows(M=m), 1 << 22, 64),
    "skew": ("config 4: 2^20, 64 rows of 100k nnz + log-normal rest", lambda m: synth.skewed_rows(M=m), 1 << 20, 256),
    "blocks": ("config 5: 2097152^2 dense 8x8 blocks on a band (as element CSR)",
               lambda m: synth.bsr_to_csr(*synth.banded_blocks(M=m)), 1 << 21, 128),
}


# ------------------------------------------------------------------------------------------------
def compulsory_bytes(nnz, rows, touched_cols, N):
    """Index 4 B + value 4 B per stored entry, one row id per matrix row, every touched row of B
    once, every row of C once."""
    return nnz * 8 + 4 * (rows + 1) + touched_cols * N * 4 + rows * N * 4


def gather_bytes(nnz, rows, N):
    """Same, but every stored entry fetches its own row of B (no reuse)."""
    return nnz * 8 + 4 * (rows + 1) + nnz * N * 4 + rows * N * 4


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples = []      # (time, sm_mhz, reasons bitmask)
        self.sm_max = None
        self.error = None
        self._halt = threading.Event()

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            while not self._halt.is_set():
                try:
                    reasons = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    reasons = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                self.samples.append((time.perf_counter(), int(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)), reasons))
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report it, do not fail the measurement
            self.error = repr(e)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)

    def summary(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-1:]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "error": self.error or "no samples"}
        bits = 0
        for s in inside:
            bits |= s[2]
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.sm_max,
                "reasons": sorted(v for k, v in self.REASONS.items() if bits & k), "samples": len(inside)}


def physical_gpu_index(local_index):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ------------------------------------------------------------------------------------------------
def time_cpu(A_csr, B, threads, budget_s, reps_min=1):
    """Time SciPy's product on a leading row block sized to fit `budget_s`; returns
    (GFLOP/s, seconds per pass, rows used, nnz used, passes)."""
    from concurrent.futures import ThreadPoolExecutor
    M, N = A_csr.shape[0], B.shape[1]
    probe_rows = max(1, min(M, 1 << 14))
    t0 = time.perf_counter()
    _ = cpu_spmm(A_csr[:probe_rows], B)
    per_nnz = (time.perf_counter() - t0) / max(1, A_csr.indptr[probe_rows]) / max(1, min(threads, 4))
    want_nnz = min(A_csr.nnz, max(1, int(budget_s / max(per_nnz, 1e-12) / max(reps_min, 1))))
    rows = int(np.searchsorted(A_csr.indptr, want_nnz, side="right"))
    rows = max(1, min(M, rows))
    sub = A_csr[:rows]
    cuts = np.searchsorted(sub.indptr, np.linspace(0, sub.nnz, threads + 1)).astype(np.int64)
    cuts[0], cuts[-1] = 0, rows
    parts = [sub[a:b] for a, b in zip(cuts[:-1], cuts[1:]) if b > a]
    times = []
    with ThreadPoolExecutor(max(1, threads)) as ex:
        for _ in range(max(reps_min, 1)):
            t0 = time.perf_counter()
            list(ex.map(lambda P: cpu_spmm(P, B), parts))
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return 2.0 * sub.nnz * N / t / 1e9, t, rows, int(sub.nnz), len(times)


# ------------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """The reference's CPU product (SciPy, what MTX.dot calls) on the host cores."""
    if rank != 0:
        return
    args.workload = args.workload or "powerlaw"
    desc, gen, full_rows, N0 = WORKLOADS[args.workload]
    rows = args.rows or full_rows
    N = args.feat or N0
    csr = gen(rows)
    A = csr.toscipy()
    B = synth.dense_features(csr.shape[1], N, args.seed)
    threads = os.cpu_count() or 1
    total_budget = 150.0
    per_step = total_budget / (args.steps + args.warmup)
    gf0, t_pass, used_rows, used_nnz, _ = time_cpu(A, B, threads, per_step, 1)
    sub = A[:used_rows]
    from concurrent.futures import ThreadPoolExecutor
    cuts = np.searchsorted(sub.indptr, np.linspace(0, sub.nnz, threads + 1)).astype(np.int64)
    cuts[0], cuts[-1] = 0, used_rows
    parts = [sub[a:b] for a, b in zip(cuts[:-1], cuts[1:]) if b > a]
    with ThreadPoolExecutor(threads) as ex:
        for _ in range(args.warmup):
            list(ex.map(lambda P: cpu_spmm(P, B), parts))
        t0 = time.perf_counter()
        for _ in range(args.steps):
            list(ex.map(lambda P: cpu_spmm(P, B), parts))
        t = time.perf_counter() - t0
    value = 2.0 * used_nnz * N * args.steps / t / 1e9
    sample = (f"first {used_rows} of {csr.shape[0]} rows ({used_nnz} of {csr.nnz} nnz) per step, scipy csr @ dense "
              f"(float32) with the rows split over {threads} threads; the reference's own call, MTX.dot, is "
              f"coo.tocsc().dot(B) on one thread (format_matrix_market.py:89-99) and is slower than this")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded)",
        "config": {"workload": f"{args.workload}: {desc}", "rows": csr.shape[0], "cols": csr.shape[1], "nnz": csr.nnz,
                   "N": N},
        "detail": {"format": "scipy csr @ dense on the host (float32)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
class Spec:
    """What one measurement runs on: a workload, its feature width / input type / partition count."""

    def __init__(self, workload, N=0, dtype="f32", parts=1, rows=0, seed=0, fmt="auto", device_B=False):
        self.workload, self.dtype, self.parts, self.seed = workload, dtype, parts, seed
        self.desc, self.gen, full_rows, N0 = WORKLOADS[workload]
        self.rows = rows or full_rows
        self.full_size = self.rows == full_rows
        self.N = N or N0
        self.use_bsr = fmt == "bsr8" or (fmt == "auto" and workload == "blocks")
        self.device_B = device_B       # B drawn on the device (side configurations: no host copy of B is needed)


def make_B(spec, K, dev, torch):
    """(B on the device in float32, host copy or None)."""
    if spec.device_B:
        gen = torch.Generator(device=dev)
        gen.manual_seed(1000 + spec.seed)
        return torch.randn((K, spec.N), generator=gen, device=dev, dtype=torch.float32), None
    host = synth.dense_features(K, spec.N, spec.seed)
    return torch.from_numpy(host).to(dev), host


class HybProblem:
    """Composed-format path: statistics + width search on the whole matrix, per-rank format slice."""
    kernel = "spmm_hyb_kernel"

    def __init__(self, spec, rank, world, dev):
        import torch
        from liteform_ae_b200 import hyb, width_search
        from liteform_ae_b200.sharding import my_range
        self.hyb, self.torch, self.dev, self.spec = hyb, torch, dev, spec
        self.rank, self.world = rank, world
        self.N = N = spec.N
        self.P = P = spec.parts
        t0 = time.perf_counter()
        self.csr = csr = spec.gen(spec.rows)
        self.M, self.K = csr.shape
        self.t_gen = time.perf_counter() - t0
        self.nnz = csr.nnz
        d_csr = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, dev)
        cuts = hyb.shard_rows(d_csr, world)
        self.r0, self.r1 = my_range(cuts, rank)
        ws = hyb.Workspace(dev)
        for attempt in range(2):   # the first pass pays context and module load; report the second
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            stats, hist = hyb.hyb_stats(d_csr, P, workspace=ws)
            self.widths = width_search.search_from_stats(stats, hist, N, P)
            torch.cuda.synchronize(dev)
            self.t_search = time.perf_counter() - t0
            t0 = time.perf_counter()
            self.fmt = hyb.build_hyb_device(d_csr, self.widths, row_range=(self.r0, self.r1), with_mask=False, workspace=ws)
            torch.cuda.synchronize(dev)
            self.t_build = time.perf_counter() - t0
        del d_csr, ws
        self.B, self.B_host = make_B(spec, self.K, dev, torch)
        self.eb = 4
        self.dtype = "f32"
        if spec.dtype == "bf16":       # B in bf16, values / accumulation / C in float32
            self.B = self.B.to(torch.bfloat16)
            self.eb = 2
            self.dtype = "bf16"
        elif spec.dtype != "f32":
            raise SystemExit("the composed-format path takes --dtype f32 or bf16")
        self.C = torch.empty((self.r1 - self.r0, N), dtype=torch.float32, device=dev)
        if self.eb == 4 and self.r1 > self.r0:   # which of the two product kernels the library picks for these operands
            self.kernel = hyb.spmm_hyb_kernel_name(self.fmt, self.B, self.C)
        self.launches_per_step = 1 + (1 if (P == 1 and self.fmt.num_zero_rows > 0) else 0) + (1 if P > 1 else 0)
        self.config = {"workload": f"{spec.workload}: {spec.desc}", "rows": self.M, "cols": self.K, "nnz": self.nnz, "N": N}
        self.detail = {"format": "hyb (composed ELL)", "num_parts": P, "bucket_widths": self.widths,
                       "sharding": f"rows, nnz-balanced, {world} rank(s), B replicated, C left sharded",
                       "l2": "inputs exceed L2 (B %.0f MB + format %.0f MB per rank); no flush between steps" % (
                           self.K * N * self.eb / 1e6, (self.fmt.cols.numel() * 8 + self.fmt.rows.numel() * 4) / 1e6),
                       "thread_blocks": self.launch_shape()}
        self.extra = {"format_build_ms": self.t_build * 1e3, "width_search_ms": self.t_search * 1e3,
                      "generate_s": self.t_gen, "padded_slots": self.fmt.total_slots, "zero_rows": self.fmt.num_zero_rows}

    def launch_shape(self):
        """Thread blocks of one product launch and how many waves of resident blocks that is (the launch
        rule of lf_spmm_hyb_f32: 256 slots per thread group, halved while fewer than 8 waves)."""
        N, fmt = self.N, self.fmt
        if self.spec.dtype == "bf16":
            lanes, chunks, vec = (8, 1, 8) if N <= 64 else (16, 1, 8) if N <= 128 else (32, 1, 8) if N <= 256 else (32, 2, 8)
        else:
            lanes, chunks, vec = ((8, 1, 4) if N <= 32 else (16, 1, 4) if N <= 64 else (32, 1, 4) if N <= 128 else
                                  (32, 2, 4) if N <= 256 else (32, 4, 4))
        gpc = 256 // lanes
        resident = 148 * 3
        tiles = 0
        for spg in (256, 128, 64, 32):
            tiles = sum(-(-int(r) // (max(1, spg // int(w)) * gpc)) for r, w in zip(fmt.ell_rows, fmt.widths) if r)
            if tiles >= resident * 8:
                break
        passes = -(-N // (lanes * chunks * vec))
        return {"per_launch": tiles * passes, "waves_of_444_resident": round(tiles * passes / resident, 2)}

    def step(self):
        self.hyb.spmm_hyb(self.fmt, self.B, out=self.C)

    def bytes_models(self):
        csr, r0, r1 = self.csr, self.r0, self.r1
        my_nnz = int(csr.indptr[r1] - csr.indptr[r0])
        touched = int(np.unique(csr.indices[csr.indptr[r0]:csr.indptr[r1]]).size)
        comp, gath = compulsory_bytes(my_nnz, r1 - r0, touched, self.N), gather_bytes(my_nnz, r1 - r0, self.N)
        if self.eb == 2:               # B rows are half as wide
            comp -= touched * self.N * 2
            gath -= my_nnz * self.N * 2
        return comp, gath

    def sampled_parity(self, C=None, count=2000):
        """Rows of this rank's C (device tensor, or a host array) against SciPy in float64 on the same rows:
        `count` random rows plus the eight longest.  Only the rows of B those rows touch are read back."""
        torch, csr, r0, r1 = self.torch, self.csr, self.r0, self.r1
        if r1 == r0:
            return {"rows_checked": 0, "max_abs_err": 0.0, "max_rel_err": 0.0, "ok": True}
        rng = np.random.default_rng(7 + self.rank)
        lens = np.diff(csr.indptr[r0:r1 + 1])
        pick = np.unique(np.concatenate([rng.integers(r0, r1, count), r0 + np.argsort(lens)[-8:]]))
        ptr = np.concatenate([[0], np.cumsum(np.diff(csr.indptr)[pick])]).astype(np.int64)
        idx = np.concatenate([csr.indices[csr.indptr[r]:csr.indptr[r + 1]] for r in pick])
        val = np.concatenate([csr.data[csr.indptr[r]:csr.indptr[r + 1]] for r in pick]).astype(np.float64)
        cols = np.unique(idx)
        B_rows = self.B[torch.from_numpy(cols).to(self.dev)].double().cpu().numpy()      # what the kernel multiplied
        import scipy.sparse as sp
        want = np.asarray(sp.csr_matrix((val, np.searchsorted(cols, idx), ptr), shape=(len(pick), len(cols))) @ B_rows)
        src = self.C if C is None else C
        local = pick - r0
        got = src[torch.from_numpy(local).to(self.dev)].cpu().numpy() if hasattr(src, "is_cuda") else np.asarray(src)[local]
        return parity_record(got, want, len(pick), "f32 rel 1e-5 / abs 1e-4 vs scipy float64 on the same (rounded) inputs; "
                             "abs part x entries / 4096 for rows longer than 4096 entries", row_nnz=np.diff(csr.indptr)[pick])

    def prepare_e2e(self):
        torch, hyb, fmt = self.torch, self.hyb, self.fmt
        if self.eb != 4 or self.B_host is None:
            raise RuntimeError("the host-memory entry point is float32 only and needs B on the host")
        pin = lambda a: torch.from_numpy(a).pin_memory().numpy()
        if self.world > 1:
            # several ranks: each uploads its format shard and 1/world of B's rows, an all-gather over
            # NVLink completes B on every GPU (sharding.HostShardedSpmm)
            from liteform_ae_b200.sharding import HostShardedSpmm, gpu_numa_node, pinned_empty
            # every rank keeps its host buffers on the NUMA node of its own GPU where the host allows it
            node = gpu_numa_node(self.dev.index)
            self.hs = HostShardedSpmm(fmt, self.N, self.rank, self.world, slots=2, numa_node=node)
            self.B_rows, placed = pinned_empty((self.hs.last - self.hs.first, self.N), torch.float32, node)
            self.B_rows.copy_(torch.from_numpy(self.B_host[self.hs.first:self.hs.last]))
            self.Cp = [pinned_empty((self.r1 - self.r0, self.N), torch.float32, node)[0] for _ in range(2)]
            self.numa = {"gpu_numa_node": node, "host_buffers_bound_to_it": bool(placed)}
            self.format_bytes = self.hs.format_bytes
            return (self.hs.h2d_bytes, self.hs.d2h_bytes,
                    "sharding.HostShardedSpmm: pinned host format shard + 1/world of B in, all-gather of B over "
                    "NVLink, lf_spmm_hyb_f32, C rows out (bytes are per rank)")
        r_nd, c_nd, _, v_nd = fmt.to_nested_numpy(with_values=True)
        ell_rows, row_off, slot_off, h_rows, h_cols, h_vals, h_zero = hyb.HybFormat.host_layout(
            fmt.bucket_widths, r_nd, c_nd, v_nd, self.M, (self.r0, self.r1))
        del r_nd, c_nd, v_nd
        self.h = tuple(pin(a) for a in (h_rows, h_cols, h_vals, h_zero))
        self.Bp = pin(self.B_host)
        self.host_fmt = hyb.HybFormat((self.M, self.K), (self.r0, self.r1), fmt.bucket_widths, ell_rows, row_off,
                                      slot_off, None, None, None, None, self.h[3])
        # two products may be in flight: each slot has its own stream, device workspace and result buffer
        self.Cp = [torch.empty((self.r1 - self.r0, self.N), dtype=torch.float32).pin_memory().numpy() for _ in range(2)]
        self.ws = [torch.empty(hyb.host_workspace_bytes(self.host_fmt, self.N), dtype=torch.uint8, device=self.dev)
                   for _ in range(2)]
        self.e2e_streams = [torch.cuda.Stream(device=self.dev) for _ in range(2)]
        self.format_bytes = sum(a.nbytes for a in self.h)
        h2d = self.format_bytes + self.Bp.nbytes
        return h2d, self.Cp[0].nbytes, "lf_spmm_hyb_f32_host (pinned host format + B in, C out, per rank)"

    def e2e_step(self, slot=0, sync=True, resident=False):
        if self.world > 1:
            self.hs.enqueue(self.B_rows, self.Cp[slot], slot, format_resident=resident)
            if sync:
                self.hs.slots[slot]["stream"].synchronize()
            return
        self.hyb.spmm_hyb_host(self.h, self.host_fmt, self.Bp, self.Cp[slot], self.ws[slot], sync=sync,
                               stream=self.e2e_streams[slot], format_resident=resident)

    def e2e_sync(self):
        if self.world > 1:
            self.hs.synchronize()
            return
        for st in self.e2e_streams:
            st.synchronize()

    def e2e_result(self, slot=0):
        return self.Cp[slot].numpy() if self.world > 1 else self.Cp[slot]

    def e2e_phases(self, reps=5):
        """One call at a time, its phases told apart by CUDA events on the call's stream: uploads
        (format + B), all-gather of B (several ranks), product, download of C.  Milliseconds, median."""
        torch = self.torch
        rec = {"h2d_ms": [], "allgather_B_ms": [], "kernel_ms": [], "d2h_ms": []}
        if self.world > 1:
            for _ in range(reps):
                ev = []
                self.hs.enqueue(self.B_rows, self.Cp[0], 0, events=ev)
                self.hs.slots[0]["stream"].synchronize()
                for k, name in enumerate(("h2d_ms", "allgather_B_ms", "kernel_ms", "d2h_ms")):
                    rec[name].append(ev[k].elapsed_time(ev[k + 1]))
        else:
            # the same copies and the same product as lf_spmm_hyb_f32_host makes, issued one by one
            st = self.e2e_streams[0]
            host = [torch.from_numpy(a) for a in self.h] + [torch.from_numpy(self.Bp)]
            dev_t = [torch.empty_like(h, device=self.dev) for h in host]
            Cd = torch.empty((self.r1 - self.r0, self.N), dtype=torch.float32, device=self.dev)
            Ch = torch.from_numpy(self.Cp[0])
            for _ in range(reps):
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                with torch.cuda.stream(st):
                    ev[0].record()
                    for d, h in zip(dev_t, host):
                        d.copy_(h, non_blocking=True)
                    ev[1].record()
                    self.hyb.spmm_hyb(self.fmt, dev_t[4], out=Cd)
                    ev[2].record()
                    Ch.copy_(Cd, non_blocking=True)
                    ev[3].record()
                st.synchronize()
                rec["h2d_ms"].append(ev[0].elapsed_time(ev[1]))
                rec["kernel_ms"].append(ev[1].elapsed_time(ev[2]))
                rec["d2h_ms"].append(ev[2].elapsed_time(ev[3]))
            rec.pop("allgather_B_ms")
        return {k: statistics.median(v) for k, v in rec.items()}

    def cpu_matrix(self):
        return self.csr.toscipy()

    def time_gather(self, mode, rank, world, steps, barrier):
        """Product followed by / fused with the all-gather of C; checks the gathered C on rank 0
        against a sample of rows computed on the host."""
        import torch
        from liteform_ae_b200.sharding import ShardedSpmm
        torch_, hyb = self.torch, self.hyb
        if not hasattr(self, "_sh"):
            sh = ShardedSpmm.__new__(ShardedSpmm)
            sh.rank, sh.world, sh.fmt = rank, world, self.fmt
            d_ptr = torch_.from_numpy(self.csr.indptr).to(self.dev)
            sh.cuts = hyb.shard_rows(hyb.DeviceCsr(d_ptr, None, None, self.csr.shape), world)
            sh.row_range = (self.r0, self.r1)
            sh.prepare_fused_gather(self.N)
            self._sh = sh
        sh = self._sh
        if mode == "fused":
            run = lambda: sh.spmm_gather_fused(self.B)
        elif mode == "peer":
            run = lambda: sh.gather_peer(hyb.spmm_hyb(self.fmt, self.B, out=self.C))
        else:
            run = lambda: sh.gather(hyb.spmm_hyb(self.fmt, self.B, out=self.C))
        for _ in range(3):
            full = run()
        barrier()
        ev0, ev1 = torch_.cuda.Event(enable_timing=True), torch_.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            full = run()
        ev1.record()
        barrier()
        t = torch_.tensor([ev0.elapsed_time(ev1) / steps], dtype=torch.float64, device=self.dev)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pick = np.unique(np.random.default_rng(5).integers(0, self.M, 4000))
        sub = self.csr.toscipy()[pick]
        want = np.asarray(sub @ self.B_host.astype(np.float64))
        got = full[torch_.from_numpy(pick).to(self.dev)].cpu().numpy()
        return {"ms_per_step": float(t.item()), "gflops": 2.0 * self.nnz * self.N / float(t.item()) / 1e6,
                "gathered_bytes_per_rank": int(self.M * self.N * 4),
                "max_abs_err_sampled_rows": float(np.abs(got - want).max())}

    def per_bucket(self, repeat):
        """Time every bucket on its own (a one-bucket view of the same arenas).  Bytes per bucket:
        compulsory = slots' index+value of real entries, row ids, touched B rows once, C rows once;
        gather = every real entry fetches its own B row."""
        torch, hyb, fmt, N = self.torch, self.hyb, self.fmt, self.N
        cols = fmt.cols.cpu().numpy()
        vals = fmt.vals.cpu().numpy()
        rows = fmt.rows.cpu().numpy()
        out = []
        for i in range(len(fmt.widths)):
            R, w = int(fmt.ell_rows[i]), int(fmt.widths[i])
            if R == 0:
                continue
            so, ro = int(fmt.slot_off[i]), int(fmt.row_off[i])
            sub = hyb.HybFormat(fmt.shape, (fmt.row_begin, fmt.row_end), [[w]], [R], [ro, int(fmt.row_off[i + 1])],
                                [so, int(fmt.slot_off[i + 1])], fmt.rows, fmt.cols, fmt.vals, None, None)
            # accumulate: no clearing launch, every flush is an atomic only where rows are shared
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(repeat + 1)]
            for _ in range(3):
                hyb.spmm_hyb(sub, self.B, out=self.C)
            ev[0].record()
            for k in range(repeat):
                hyb.spmm_hyb(sub, self.B, out=self.C)
                ev[k + 1].record()
            torch.cuda.synchronize(self.dev)
            ms = statistics.median(ev[k].elapsed_time(ev[k + 1]) for k in range(repeat))
            real = vals[so:so + R * w] != 0
            nnz_b = int(real.sum())
            touched = int(np.unique(cols[so:so + R * w][real]).size)
            nrows = int(np.unique(rows[ro:ro + R]).size)
            comp = nnz_b * 8 + 4 * R + touched * N * 4 + nrows * N * 4
            gath = nnz_b * 8 + 4 * R + nnz_b * N * 4 + nrows * N * 4
            out.append({"width": w, "ell_rows": R, "nnz": nnz_b, "ms": ms, "gflops": 2.0 * nnz_b * N / ms / 1e6,
                        "compulsory_gbs": comp / ms / 1e6, "gather_model_gbs": gath / ms / 1e6})
        return out


def parity_record(got, want, rows, tolerance, row_nnz=None):
    """`ok`: |got - want| <= 1e-4 + 1e-5 |want| element-wise; for rows of more than 4096 stored entries the
    absolute part is scaled by entries / 4096 (the error of a chained float32 sum grows that way: the
    100 000-entry rows of the skewed matrix have partial sums near 200, one ulp of which is 1.5e-5, and
    are cut into 400 to 3000 partial sums, depending on the shard size, that atomic adds commit in any order)."""
    err = np.abs(got - want)
    scale = float(np.abs(want).max()) or 1.0
    atol = 1e-4 if row_nnz is None else 1e-4 * np.maximum(1.0, np.asarray(row_nnz, dtype=np.float64) / 4096.0).reshape(-1, 1)
    rec = {"rows_checked": int(rows), "max_abs_err": float(err.max()), "max_rel_err": float(err.max() / scale),
           "ok": bool(np.all(err <= atol + 1e-5 * np.abs(want))), "tolerance": tolerance}
    if row_nnz is not None and np.max(row_nnz) > 4096:
        short = np.asarray(row_nnz) <= 4096
        rec["max_abs_err_rows_up_to_4096_entries"] = float(err[short].max()) if short.any() else 0.0
        rec["longest_row_checked"] = int(np.max(row_nnz))
    return rec


class BsrProblem:
    """8x8 block path (config 5): block rows split evenly over the ranks (every block row holds
    the same number of blocks), B replicated."""

    def __init__(self, spec, rank, world, dev, shared=None):
        import torch
        from liteform_ae_b200 import bsr
        self.bsr, self.torch, self.dev, self.spec = bsr, torch, dev, spec
        self.rank, self.world = rank, world
        self.N = N = spec.N
        t0 = time.perf_counter()
        if shared is None:
            shared = synth.banded_blocks(M=spec.rows)
        indptr, indices, blocks, shape = shared
        self.shared = shared
        self.M, self.K = shape
        self.t_gen = time.perf_counter() - t0
        self.indptr, self.indices, self.blocks = indptr, indices, blocks
        self.nnz = int(blocks.size)
        Mb = self.M // 8
        self.r0, self.r1 = (Mb * rank) // world, (Mb * (rank + 1)) // world   # block rows
        self.tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[spec.dtype]
        self.dtype = spec.dtype
        if spec.dtype == "f32":
            self.kernel = "bsr8_spmm_f32_narrow_kernel" if N <= 32 else "bsr8_spmm_f32_kernel"
        else:
            self.kernel = ("bsr8_spmm_16bit_narrow_kernel" if N <= 32 else
                           "bsr8_spmm_16bit_mid_kernel" if N <= 64 else "bsr8_spmm_16bit_kernel")
        name = {"f32": "float32", "bf16": "bfloat16", "f16": "float16"}[spec.dtype]
        self.a = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, name, dev)
        B32, self.B_host = make_B(spec, self.K, dev, torch)
        self.B = B32.to(self.tdt)
        del B32
        self.C = torch.empty(((self.r1 - self.r0) * 8, N), dtype=torch.float32, device=dev)
        self.launches_per_step = 1
        eb = 4 if spec.dtype == "f32" else 2
        self.eb = eb
        self.config = {"workload": f"{spec.workload}: {spec.desc}", "rows": self.M, "cols": self.K, "nnz": self.nnz, "N": N}
        self.detail = {"format": "bsr 8x8", "input_dtype": spec.dtype, "accumulate": "f32",
                       "sharding": f"block rows, even split, {world} rank(s), B replicated, C left sharded",
                       "l2": "inputs exceed L2 (A %.0f MB + B %.0f MB per rank); no flush between steps" % (
                           self.nnz * eb / 1e6 / world, self.K * N * eb / 1e6)}
        self.extra = {"generate_s": self.t_gen}

    def time_device_builder(self):
        """CSR -> 8x8 blocks on the device (lf_bsr8_plan + lf_bsr8_fill), timed on the element CSR form
        of this matrix.  The CSR arrays are laid out on the device from the block arrays (every block
        row of the synthetic matrix holds the same number of blocks, so this is a reshape)."""
        torch = self.torch
        from liteform_ae_b200 import hyb
        dtype_name = {"f32": "float32", "bf16": "bfloat16", "f16": "float16"}[self.spec.dtype]
        per = np.diff(self.indptr)
        if per.size == 0 or not (per == per[0]).all():
            return {}
        k, Mb = int(per[0]), self.M // 8
        cols = (self.a.indices.view(Mb, 1, k, 1).to(torch.int32) * 8 +
                torch.arange(8, dtype=torch.int32, device=self.dev).view(1, 1, 1, 8)).expand(Mb, 8, k, 8).reshape(-1)
        vals = self.a.blocks.view(Mb, k, 8, 8).permute(0, 2, 1, 3).reshape(-1).float().contiguous()
        ptr = torch.arange(self.M + 1, dtype=torch.int64, device=self.dev) * (8 * k)
        csr = hyb.DeviceCsr(ptr, cols.contiguous(), vals, (self.M, self.K))
        times = []
        for _ in range(4):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            built = self.bsr.DeviceBsr8.from_csr_device(csr, dtype_name)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
        same = bool(torch.equal(built.indptr, self.a.indptr) and torch.equal(built.indices, self.a.indices) and
                    torch.equal(built.blocks, self.a.blocks))
        if not same:
            raise RuntimeError("the device-built blocks differ from the generator's")
        return {"format_build_ms": statistics.median(times[1:]) * 1e3,
                "format_build": "CSR (device) -> 8x8 blocks (device), lf_bsr8_plan + lf_bsr8_fill, checked equal to the generated blocks"}

    def step(self):
        self.bsr.spmm_bsr8(self.a, self.B, out=self.C, block_row_range=(self.r0, self.r1))

    def bytes_models(self):
        nb = int(self.indptr[self.r1] - self.indptr[self.r0])
        rows = (self.r1 - self.r0) * 8
        touched = int(np.unique(self.indices[self.indptr[self.r0]:self.indptr[self.r1]]).size) * 8
        comp = nb * 64 * self.eb + 4 * nb + 8 * (self.r1 - self.r0 + 1) + touched * self.N * self.eb + rows * self.N * 4
        gath = nb * 64 * self.eb + 4 * nb + 8 * (self.r1 - self.r0 + 1) + nb * 8 * self.N * self.eb + rows * self.N * 4
        return comp, gath

    def sampled_parity(self, C=None, count=300):
        """Block rows of this rank's C against SciPy's BSR product in float64 of the operands as the
        kernel sees them (rounded to the input type)."""
        import scipy.sparse as sp
        torch = self.torch
        if self.r1 == self.r0:
            return {"rows_checked": 0, "max_abs_err": 0.0, "max_rel_err": 0.0, "ok": True}
        rng = np.random.default_rng(9 + self.rank)
        pick = np.unique(np.concatenate([rng.integers(self.r0, self.r1, count), [self.r0, self.r1 - 1]]))
        ip = self.indptr.astype(np.int64)
        sel = np.concatenate([np.arange(ip[I], ip[I + 1]) for I in pick])
        J = np.unique(self.indices[sel])
        ptr = np.concatenate([[0], np.cumsum(np.diff(ip)[pick])]).astype(np.int64)
        blk = self.a.blocks[torch.from_numpy(sel).to(self.dev)].double().cpu().numpy()
        b_rows = torch.from_numpy((J[:, None].astype(np.int64) * 8 + np.arange(8)[None, :]).reshape(-1)).to(self.dev)
        want = np.asarray(sp.bsr_matrix((blk, np.searchsorted(J, self.indices[sel]).astype(np.int32), ptr),
                                        shape=(len(pick) * 8, len(J) * 8)) @ self.B[b_rows].double().cpu().numpy())
        rows = ((pick - self.r0)[:, None] * 8 + np.arange(8)[None, :]).reshape(-1)
        src = self.C if C is None else C
        got = src[torch.from_numpy(rows).to(self.dev)].cpu().numpy() if hasattr(src, "is_cuda") else np.asarray(src)[rows]
        return parity_record(got, want, len(rows), "rel 1e-5 / abs 1e-4 vs scipy float64 on the same (rounded) inputs")

    def prepare_e2e(self):
        torch = self.torch
        if self.B_host is None:
            raise RuntimeError("the end-to-end leg needs B on the host")
        s, e = int(self.indptr[self.r0]), int(self.indptr[self.r1])
        conv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.tdt).pin_memory()
        self.h_ptr = torch.from_numpy((self.indptr[self.r0:self.r1 + 1] - s).astype(np.int64)).pin_memory()
        self.h_idx = torch.from_numpy(self.indices[s:e].astype(np.int32)).pin_memory()
        self.h_blk = conv(self.blocks[s:e])
        self.h_B = conv(self.B_host)
        # two products may be in flight: each slot has its own stream, device buffers and result buffer
        self.h_C = [torch.empty(((self.r1 - self.r0) * 8, self.N), dtype=torch.float32).pin_memory() for _ in range(2)]
        host = (self.h_ptr, self.h_idx, self.h_blk, self.h_B)
        self.d_in = [tuple(torch.empty_like(h, device=self.dev) for h in host) for _ in range(2)]
        self.d_C = [torch.empty_like(self.h_C[0], device=self.dev) for _ in range(2)]
        self.e2e_streams = [torch.cuda.Stream(device=self.dev) for _ in range(2)]
        self.format_bytes = sum(t.numel() * t.element_size() for t in host[:3])
        h2d = sum(t.numel() * t.element_size() for t in host)
        return h2d, self.h_C[0].numel() * 4, "spmm_bsr8 on buffers copied from/to pinned host memory every step"

    def e2e_step(self, slot=0, sync=True, resident=False):
        torch = self.torch
        with torch.cuda.stream(self.e2e_streams[slot]):
            pairs = list(zip(self.d_in[slot], (self.h_ptr, self.h_idx, self.h_blk, self.h_B)))
            for d, h in (pairs[3:] if resident else pairs):
                d.copy_(h, non_blocking=True)
            d_ptr, d_idx, d_blk, d_B = self.d_in[slot]
            a = self.bsr.DeviceBsr8(d_ptr, d_idx, d_blk, ((self.r1 - self.r0) * 8, self.K))
            self.bsr.spmm_bsr8(a, d_B, out=self.d_C[slot])
            self.h_C[slot].copy_(self.d_C[slot], non_blocking=True)
        if sync:
            self.e2e_streams[slot].synchronize()

    def e2e_sync(self):
        for st in self.e2e_streams:
            st.synchronize()

    def e2e_result(self, slot=0):
        return self.h_C[slot].numpy()

    def e2e_phases(self, reps=5):
        return None

    def cpu_matrix(self):
        import scipy.sparse as sp
        return sp.bsr_matrix((self.blocks, self.indices, self.indptr), shape=(self.M, self.K)).tocsr()


def pin_to_gpu_numa_node(local_rank):
    """Keep this process (and with it the pinned host buffers it will touch first) on the CPUs that are
    local to its GPU, where the topology is visible and the allowed CPU set contains any of them.
    Read-only queries plus the process's own affinity; nothing outlasts the process."""
    info = {"applied": False}
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(local_rank))
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        dom, rest = bus.split(":", 1)
        path = f"/sys/bus/pci/devices/{int(dom, 16):04x}:{rest.lower()}/local_cpulist"
        with open(path) as f:
            text = f.read().strip()
        local = set()
        for part in text.split(","):
            if part:
                a, _, b = part.partition("-")
                local.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0)
        both = allowed & local
        info.update({"gpu_local_cpus": text, "allowed_cpus": len(allowed)})
        if both and both != allowed:
            os.sched_setaffinity(0, both)
            info["applied"] = True
        info["cpus_used"] = len(both or allowed)
    except Exception as exc:
        info["error"] = repr(exc)[:200]
    return info


def measure(prob, steps, warmup, barrier, dist, world, dev):
    """W warm-up steps, then K timed steps bracketed by barrier + synchronize; CUDA events around every
    step on the launching stream.  Returns the record of one configuration (max over ranks)."""
    import torch
    for _ in range(warmup):
        prob.step()
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t_wall0 = time.perf_counter()
    ev[0].record()
    for i in range(steps):
        prob.step()
        ev[i + 1].record()
    barrier()
    t_wall1 = time.perf_counter()
    total_ms = ev[0].elapsed_time(ev[-1])
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
    alg, gath = prob.bytes_models()
    mine = torch.tensor([total_ms, statistics.fmean(step_ms), float(alg), float(gath)], dtype=torch.float64, device=dev)
    if world > 1:
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        every = torch.stack(every).cpu().numpy()
    else:
        every = mine.cpu().numpy()[None, :]
    parity = prob.sampled_parity()
    ok = torch.tensor([1.0 if parity["ok"] else 0.0, parity["max_abs_err"], parity["max_rel_err"]], dtype=torch.float64, device=dev)
    if world > 1:
        allok = [torch.empty_like(ok) for _ in range(world)]
        dist.all_gather(allok, ok)
        allok = torch.stack(allok).cpu().numpy()
        parity = {"rows_checked_per_rank": parity["rows_checked"], "max_abs_err": float(allok[:, 1].max()),
                  "max_rel_err": float(allok[:, 2].max()), "ok": bool(allok[:, 0].min() > 0.5), "tolerance": parity.get("tolerance")}
    return {"total_ms_max": float(every[:, 0].max()), "rank_total_ms": [float(x) for x in every[:, 0]],
            "launch_ms_rank0": float(every[0, 1]), "launch_ms_max": float(every[:, 1].max()),
            "step_ms_rank0": step_ms, "alg_bytes_rank": [float(x) for x in every[:, 2]],
            "gather_bytes_rank": [float(x) for x in every[:, 3]], "parity": parity, "wall": (t_wall0, t_wall1)}


def roofline_of(prob, rec, world):
    """Roofline object of one configuration.  Per rank: algorithmic bytes of the rank's shard / the rank's
    mean launch time; the job's figure divides the whole matrix's bytes by the slowest rank's time and
    compares with `world` times the measured single-GPU peak."""
    peak, peak_kind = measured_peak_gbs()
    steps = len(rec["step_ms_rank0"])
    launch_ms = rec["total_ms_max"] / steps if world > 1 else rec["launch_ms_rank0"]
    alg = sum(rec["alg_bytes_rank"])
    gath = sum(rec["gather_bytes_rank"])
    achieved = alg / (launch_ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peak * world, "unit": "GB/s", "frac": achieved / (peak * world),
            "traffic": None, "peak_kind": f"of {peak_kind}" + (f" x {world} GPUs" if world > 1 else ""),
            "kernel": prob.kernel, "algorithmic_bytes_per_launch": int(alg), "launch_ms": launch_ms,
            "launch_ms_median": statistics.median(rec["step_ms_rank0"]),
            "gather_model_bytes_per_launch": int(gath), "gather_model_gbs": gath / (launch_ms * 1e-3) / 1e9,
            # bytes every stored entry / block pulls out of L2 or HBM, per clock and SM at 148 SMs x 1965 MHz: the
            # scattered-row gathers of these kernels top out near 30 (measured on the block workload)
            "gather_model_bytes_per_clk_per_sm": gath / (launch_ms * 1e-3) / (148 * world * 1.965e9)}


KERNEL_SOURCES = {"hyb": ("lf_spmm_hyb.cu", "lf_common.cuh"), "bsr8": ("lf_spmm_bsr8.cu", "lf_bsr8_mma.cuh")}


def kernel_source_hash(family):
    """sha256 (first 16 hex digits) over the CUDA sources of one kernel family: a traffic figure captured
    under ncu is only reported while the kernel is the one it was captured on."""
    import hashlib
    h = hashlib.sha256()
    for f in KERNEL_SOURCES[family]:
        with open(os.path.join(ROOT, "liteform_ae_b200", "csrc", f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def attach_traffic(roofline, spec, world):
    key = (spec.workload, "bsr8" if spec.use_bsr else "hyb", spec.dtype, spec.N, spec.parts, world)
    entry = TRAFFIC_BYTES_PER_LAUNCH.get(key) if spec.full_size else None
    if entry is None:
        roofline["traffic_source"] = "no ncu capture for this configuration"
        return
    nbytes, source, src_hash = entry
    if src_hash != kernel_source_hash(key[1]):
        roofline["traffic_source"] = f"stale: {source} was captured on other kernel sources ({src_hash})"
        return
    roofline["traffic"] = nbytes
    roofline["traffic_source"] = source
    roofline["dram_gbs_from_traffic"] = nbytes / (roofline["launch_ms"] * 1e-3) / 1e9


def run_side_configs(args, rank, world, dev, barrier, dist):
    """The other benchmark configurations, device-timed like the headline and checked on sampled rows."""
    import torch
    out = {}
    side_steps, side_warm = max(3, min(args.steps, args.side_steps)), 3
    plan = [("config3_uniform_f32_n64", Spec("uniform", 64, "f32", device_B=True)),
            ("config4_skew_f32_n256", Spec("skew", 256, "f32", device_B=True))]
    for name, spec in plan:
        try:
            prob = HybProblem(spec, rank, world, dev)
            rec = measure(prob, side_steps, side_warm, barrier, dist, world, dev)
            out[name] = side_record(prob, spec, rec, world, side_steps)
            del prob
        except Exception as exc:
            out[name] = {"error": repr(exc)[:300]}
        torch.cuda.empty_cache()
    shared = None
    try:
        shared = synth.banded_blocks()
    except Exception as exc:
        out["config5_blocks"] = {"error": repr(exc)[:300]}
    if shared is not None:
        for dtype in ("f32", "bf16"):
            for N in (128, 32, 512):
                name = f"config5_blocks_{dtype}_n{N}"
                try:
                    spec = Spec("blocks", N, dtype, device_B=True)
                    prob = BsrProblem(spec, rank, world, dev, shared=shared)
                    rec = measure(prob, side_steps, side_warm, barrier, dist, world, dev)
                    out[name] = side_record(prob, spec, rec, world, side_steps)
                    del prob
                except Exception as exc:
                    out[name] = {"error": repr(exc)[:300]}
                torch.cuda.empty_cache()
    return out


def side_record(prob, spec, rec, world, steps):
    roof = roofline_of(prob, rec, world)
    attach_traffic(roof, spec, world)
    ms = rec["total_ms_max"] / steps
    return {"config": prob.config, "dtype": prob.dtype, "steps": steps, "ms": ms,
            "gflops": 2.0 * prob.nnz * prob.N / ms / 1e6,
            "rank_ms_min": min(rec["rank_total_ms"]) / steps, "rank_ms_max": max(rec["rank_total_ms"]) / steps,
            "roofline": {k: roof.get(k) for k in ("frac", "achieved", "peak", "algorithmic_bytes_per_launch", "kernel",
                                                  "traffic", "traffic_source", "dram_gbs_from_traffic", "gather_model_gbs",
                                                  "gather_model_bytes_per_clk_per_sm")},
            "parity": rec["parity"], "detail": {k: v for k, v in prob.detail.items() if k != "l2"},
            "build": {k: prob.extra[k] for k in ("format_build_ms", "width_search_ms", "generate_s") if k in prob.extra}}


def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.bsr_engine or args.bsr_shape:
        from liteform_ae_b200 import _cabi
        _cabi.check(_cabi.load().lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, args.bsr_engine))
        _cabi.check(_cabi.load().lf_set_option(_cabi.LF_OPT_BSR_PIPE_SHAPE, args.bsr_shape))
    numa = pin_to_gpu_numa_node(local_rank)
    spec = Spec(args.workload or "powerlaw", args.feat, args.dtype, args.parts, args.rows, args.seed, args.format)
    prob = (BsrProblem if spec.use_bsr else HybProblem)(spec, rank, world, dev)
    if spec.use_bsr and not args.no_build_timing:
        prob.extra.update(prob.time_device_builder())
    N = prob.N

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    rec = measure(prob, args.steps, args.warmup, barrier, dist, world, dev)
    sampler.stop()
    total_ms_max = rec["total_ms_max"]
    clocks = sampler.summary(*rec["wall"])

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region ----------
    try:
        if args.no_e2e:
            raise RuntimeError("skipped (--no-e2e)")
        h2d, d2h, call = prob.prepare_e2e()
        e2e_steps = max(4, min(args.steps, 20))
        e2e_steps += e2e_steps % 2
        for _ in range(2):
            prob.e2e_step()
        # (1) one call at a time, each synchronised before the next starts: the latency of a call
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            prob.e2e_step()
        barrier()
        t_one = (time.perf_counter() - t0) / e2e_steps

        def two_in_flight(resident):
            for slot in (0, 1):
                prob.e2e_step(slot, sync=False, resident=resident)
            prob.e2e_sync()
            barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                prob.e2e_step(i % 2, sync=False, resident=resident)
            prob.e2e_sync()
            barrier()
            return (time.perf_counter() - t0) / e2e_steps

        # (2) two calls in flight on two streams (own workspace and result buffer each): the result
        # of one step crosses the bus while the operands of the next one come in.  Every step still
        # copies all its inputs in and its whole result out inside the timed region.
        t_two = two_in_flight(False)
        e2e_parity = [prob.sampled_parity(C=prob.e2e_result(k)) for k in (0, 1)]
        # (3) as (2), but the format stays in the device workspace after the first call: only B goes in
        t_res = two_in_flight(True)
        res_parity = [prob.sampled_parity(C=prob.e2e_result(k)) for k in (0, 1)]
        phases = prob.e2e_phases()
        te = torch.tensor([t_one, t_two, t_res], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        t_one, t_two, t_res = (float(x) for x in te.cpu())
        e2e = {"value": 2.0 * prob.nnz * N / min(t_one, t_two) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": min(t_one, t_two) * 1e3, "steps": e2e_steps, "call": call,
               "mode": "two calls in flight on two streams" if t_two < t_one else "one call at a time",
               "ms_per_step_one_call_at_a_time": t_one * 1e3, "ms_per_step_two_in_flight": t_two * 1e3,
               "parity_sampled_rows": {"max_abs_err": max(p["max_abs_err"] for p in e2e_parity),
                                       "max_rel_err": max(p["max_rel_err"] for p in e2e_parity),
                                       "ok": all(p["ok"] for p in e2e_parity), "rows_checked": e2e_parity[0]["rows_checked"]},
               "format_resident": {"ms_per_step": t_res * 1e3, "value": 2.0 * prob.nnz * N / t_res / 1e9,
                                   "h2d_bytes_per_step": int(h2d - prob.format_bytes),
                                   "note": "LF_SPMM_FORMAT_RESIDENT: the format stays in the device workspace after the "
                                           "first call, B in and C out every step; not the headline (the reference uploads "
                                           "the format on every call)",
                                   "parity_ok": all(p["ok"] for p in res_parity)},
               "phases_one_call_ms": phases, "host_affinity": dict(numa, **getattr(prob, "numa", {}))}
    except Exception as exc:  # keep the device-resident numbers, say what went wrong
        e2e = {"value": None, "unit": UNIT, "error": repr(exc)}

    # ---- the whole C on every rank: padded NCCL all-gather, ragged peer-store gather, fused epilogue ----
    gather = None
    if args.gather != "none" and world > 1 and isinstance(prob, HybProblem) and prob.eb == 4 and prob.B_host is not None:
        gather = {}
        for mode in (("nccl", "peer", "fused") if args.gather == "all" else (args.gather,)):
            try:
                gather[mode] = prob.time_gather(mode, rank, world, max(3, min(args.steps, 30)), barrier)
            except Exception as exc:
                gather[mode] = {"error": repr(exc)[:300]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        A = prob.cpu_matrix()
        gf, t_pass, used_rows, used_nnz, passes = time_cpu(A, prob.B_host, 1, 12.0, 2)
        cpu = {"value": gf, "unit": UNIT, "cores": 1, "kind": "port",
               "sample": f"scipy csr @ dense (float32), first {used_rows} of {prob.M} rows ({used_nnz} nnz), median of {passes} passes, {t_pass:.2f} s per pass"}
        threads = os.cpu_count() or 1
        if threads > 1:
            gfm, tm, ur, un, ps = time_cpu(A, prob.B_host, threads, 6.0, 2)
            cpu["all_cores"] = {"value": gfm, "cores": threads, "sample": f"{ur} rows split over {threads} threads, {tm:.2f} s per pass"}
        del A

    roofline = roofline_of(prob, rec, world)
    attach_traffic(roofline, spec, world)
    headline_detail, headline_extra = prob.detail, prob.extra
    line = {
        "metric": METRIC, "value": 2.0 * prob.nnz * N * args.steps / (total_ms_max * 1e-3) / 1e9, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms_max / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": prob.dtype,
        "data": "synthetic (seeded, numpy default_rng)", "config": prob.config, "detail": headline_detail,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
        "gpu_launches": prob.launches_per_step * args.steps,
        "parity_sampled_rows": rec["parity"],
        "rank_ms_min": min(rec["rank_total_ms"]) / args.steps, "rank_ms_max": max(rec["rank_total_ms"]) / args.steps,
    }
    line.update(headline_extra)
    if gather is not None:
        line["gather"] = gather
    if args.per_bucket and hasattr(prob, "per_bucket"):
        line["per_bucket"] = prob.per_bucket(20)
    del prob
    torch.cuda.empty_cache()
    if args.workload is None and not args.no_side:
        t0 = time.perf_counter()
        line["configs"] = run_side_configs(args, rank, world, dev, barrier, dist)
        line["configs_wall_s"] = time.perf_counter() - t0
    if rank == 0:
        print(json.dumps(line), flush=True)


# DRAM bytes (read + write) of one launch of the dominant kernel from an ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum), keyed by (workload, format, dtype, N, num_parts,
# n_gpus) at full size: (bytes, where the figure comes from, hash of the CUDA sources it was
# captured on).  The figure is reported only while kernel_source_hash() still matches.
_NCU = "ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum -c 2 on `bench.py --workload %s --steps 2 --warmup 3 --no-cpu --no-e2e`"
TRAFFIC_BYTES_PER_LAUNCH = {
    ("powerlaw", "hyb", "f32", 128, 1, 1): (3139579392 + 542627840, _NCU % "powerlaw" + ", full size", "10e0a7d22469db01"),
    ("powerlaw", "hyb", "f32", 128, 2, 1): (3419856384 + 971848960, _NCU % "powerlaw --parts 2" + ", full size", "10e0a7d22469db01"),
    ("powerlaw", "hyb", "f32", 128, 4, 1): (3236526848 + 1477323520, _NCU % "powerlaw --parts 4" + ", full size", "10e0a7d22469db01"),
    ("powerlaw", "hyb", "f32", 128, 8, 1): (3311143168 + 1991411456, _NCU % "powerlaw --parts 8" + ", full size", "10e0a7d22469db01"),
    ("uniform", "hyb", "f32", 64, 1, 1): (32675725824 + 1073462016, _NCU % "uniform" + ", full size", "10e0a7d22469db01"),
    ("skew", "hyb", "f32", 256, 1, 1): (19900642816 + 1108303360, _NCU % "skew" + ", full size", "10e0a7d22469db01"),
    ("blocks", "bsr8", "f32", 128, 1, 1): (2 * (931068672 + 508342528), "ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum -c 2 on `bench.py --workload blocks --rows 1048576 --steps 2 --warmup 3 --no-cpu --no-e2e --no-build-timing`: "
                                           "captured at 2^20 rows, doubled (traffic is proportional to the rows at a fixed band)", "0805c80c8db254c0"),
    ("blocks", "bsr8", "bf16", 128, 1, 1): (2 * (484701184 + 493565184), "ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum -c 2 on `bench.py --workload blocks --dtype bf16 --rows 1048576 --steps 2 --warmup 3 --no-cpu --no-e2e --no-build-timing`: "
                                            "captured at 2^20 rows, doubled (traffic is proportional to the rows at a fixed band)", "0805c80c8db254c0"),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="default: powerlaw as the headline plus the other benchmark matrices in `configs`")
    ap.add_argument("--no-side", action="store_true", help="skip the `configs` object (the other benchmark matrices)")
    ap.add_argument("--side-steps", type=int, default=20, help="timed steps of each side configuration")
    ap.add_argument("--rows", type=int, default=0, help="override the matrix dimension (tests)")
    ap.add_argument("--feat", type=int, default=0, help="override the feature width N")
    ap.add_argument("--parts", type=int, default=1, help="number of column partitions")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--format", default="auto", choices=["auto", "hyb", "bsr8"],
                    help="auto: 8x8 block kernels for the block workload, composed format otherwise")
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16", "f16"], help="input type of the block path")
    ap.add_argument("--per-bucket", action="store_true", help="also time every ELL bucket on its own")
    ap.add_argument("--gather", default="all", choices=["none", "all", "nccl", "peer", "fused"],
                    help="multi-GPU only: also time product + full C on every rank (padded NCCL all-gather, ragged "
                         "peer-store gather lf_allgather_rows, fused epilogue lf_spmm_hyb_f32_bcast)")
    ap.add_argument("--bsr-engine", type=int, default=0, help="block path: LF_OPT_BSR_COPY_ENGINE (0 = library default)")
    ap.add_argument("--bsr-shape", type=int, default=0, help="block path, engines 4 and 5: LF_OPT_BSR_PIPE_SHAPE")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-build-timing", action="store_true", help="block path: skip timing the device CSR -> blocks builder")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-memory end-to-end leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    elif args.gpus > 1:
        print(f"bench.py: --gpus {args.gpus} needs torchrun (one process per GPU); running 1 rank", file=sys.stderr)
    try:
        run_ours(args, rank, local_rank, world)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
