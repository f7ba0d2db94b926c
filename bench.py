#!/usr/bin/env python
"""Benchmark of the composed-format SpMM: GFLOP/s (2 * nnz * N / t) and HBM-roofline fraction.

    python bench.py [--gpus N --steps K --warmup W] [--workload powerlaw|zipf|uniform|skew|blocks]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # SciPy on the host cores, same metric and config

A step is one SpMM C = A B over the whole (row-sharded) matrix with the format and B resident in
HBM.  The default workload is the power-law graph (2^20 rows, N = 128).  Rank 0 prints one JSON
line.  Inputs are synthetic and seeded; B plus the format exceed the 126 MB L2, so consecutive
steps cannot be served from cache.
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
    sample = f"first {used_rows} of {csr.shape[0]} rows ({used_nnz} of {csr.nnz} nnz) per step, scipy csr @ dense split over {threads} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded)",
        "config": {"workload": f"{args.workload}: {desc}", "format": "scipy csr on the host", "rows": csr.shape[0],
                   "cols": csr.shape[1], "nnz": csr.nnz, "N": N},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
class HybProblem:
    """Composed-format path: statistics + width search on the whole matrix, per-rank format slice."""
    kernel = "spmm_hyb_kernel"

    def __init__(self, args, rank, world, dev):
        import torch
        from liteform_ae_b200 import hyb, width_search
        from liteform_ae_b200.sharding import my_range
        self.hyb, self.torch, self.dev = hyb, torch, dev
        self.rank, self.world = rank, world
        desc, gen, full_rows, N0 = WORKLOADS[args.workload]
        self.N = N = args.feat or N0
        self.P = P = args.parts
        t0 = time.perf_counter()
        self.csr = csr = gen(args.rows or full_rows)
        self.M, self.K = csr.shape
        self.B_host = synth.dense_features(self.K, N, args.seed)
        self.t_gen = time.perf_counter() - t0
        self.nnz = csr.nnz
        d_csr = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, dev)
        cuts = hyb.shard_rows(d_csr, world)
        self.r0, self.r1 = my_range(cuts, rank)
        for attempt in range(2):   # the first pass pays context and module load; report the second
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            stats, hist = hyb.hyb_stats(d_csr, P)
            self.widths = width_search.search_from_stats(stats, hist, N, P)
            torch.cuda.synchronize(dev)
            self.t_search = time.perf_counter() - t0
            t0 = time.perf_counter()
            self.fmt = hyb.build_hyb_device(d_csr, self.widths, row_range=(self.r0, self.r1), with_mask=False)
            torch.cuda.synchronize(dev)
            self.t_build = time.perf_counter() - t0
        del d_csr
        self.B = torch.from_numpy(self.B_host).to(dev)
        self.eb = 4
        self.dtype = "f32"
        if args.dtype == "bf16":       # B in bf16, values / accumulation / C in float32
            self.B = self.B.to(torch.bfloat16)
            self.eb = 2
            self.dtype = "bf16"
        elif args.dtype != "f32":
            raise SystemExit("the composed-format path takes --dtype f32 or bf16")
        self.C = torch.empty((self.r1 - self.r0, N), dtype=torch.float32, device=dev)
        self.launches_per_step = 1 + (1 if (P == 1 and self.fmt.num_zero_rows > 0) else 0) + (1 if P > 1 else 0)
        self.config = {"workload": f"{args.workload}: {desc}", "format": "hyb (composed ELL)", "rows": self.M,
                       "cols": self.K, "nnz": self.nnz, "N": N, "num_parts": P, "bucket_widths": self.widths,
                       "sharding": f"rows, nnz-balanced, {world} rank(s), B replicated, C left sharded",
                       "l2": "inputs exceed L2 (B %.0f MB + format %.0f MB per rank); no flush between steps" % (
                           self.B_host.nbytes / 1e6, (self.fmt.cols.numel() * 8 + self.fmt.rows.numel() * 4) / 1e6)}
        self.extra = {"format_build_ms": self.t_build * 1e3, "width_search_ms": self.t_search * 1e3,
                      "generate_s": self.t_gen, "padded_slots": self.fmt.total_slots, "zero_rows": self.fmt.num_zero_rows}

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

    def prepare_e2e(self):
        torch, hyb, fmt = self.torch, self.hyb, self.fmt
        if self.eb != 4:
            raise RuntimeError("the host-memory entry point is float32 only")
        pin = lambda a: torch.from_numpy(a).pin_memory().numpy()
        if self.world > 1:
            # several ranks: each uploads its format shard and 1/world of B's rows, an all-gather over
            # NVLink completes B on every GPU (sharding.HostShardedSpmm)
            from liteform_ae_b200.sharding import HostShardedSpmm
            self.hs = HostShardedSpmm(fmt, self.N, self.rank, self.world, slots=2)
            self.B_rows = torch.from_numpy(self.B_host[self.hs.first:self.hs.last]).pin_memory()
            self.Cp = [torch.empty((self.r1 - self.r0, self.N), dtype=torch.float32).pin_memory() for _ in range(2)]
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
        h2d = sum(a.nbytes for a in self.h) + self.Bp.nbytes
        return h2d, self.Cp[0].nbytes, "lf_spmm_hyb_f32_host (pinned host format + B in, C out, per rank)"

    def e2e_step(self, slot=0, sync=True):
        if self.world > 1:
            self.hs.enqueue(self.B_rows, self.Cp[slot], slot)
            if sync:
                self.hs.slots[slot]["stream"].synchronize()
            return
        self.hyb.spmm_hyb_host(self.h, self.host_fmt, self.Bp, self.Cp[slot], self.ws[slot], sync=sync,
                               stream=self.e2e_streams[slot])

    def e2e_sync(self):
        if self.world > 1:
            self.hs.synchronize()
            return
        for st in self.e2e_streams:
            st.synchronize()

    def e2e_result(self, slot=0):
        return self.Cp[slot].numpy() if self.world > 1 else self.Cp[slot]

    def cpu_matrix(self):
        return self.csr.toscipy()

    def time_gather(self, mode, rank, world, steps, barrier):
        """Product followed by / fused with the all-gather of C; checks the gathered C on rank 0
        against a sample of rows computed on the host."""
        import torch
        from liteform_ae_b200.sharding import ShardedSpmm
        torch_, hyb = self.torch, self.hyb
        sh = ShardedSpmm.__new__(ShardedSpmm)
        sh.rank, sh.world, sh.fmt = rank, world, self.fmt
        d_ptr = torch_.from_numpy(self.csr.indptr).to(self.dev)
        sh.cuts = hyb.shard_rows(hyb.DeviceCsr(d_ptr, None, None, self.csr.shape), world)
        if mode == "fused":
            sh.prepare_fused_gather(self.N)
            run = lambda: sh.spmm_gather_fused(self.B)
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
        t = torch_.tensor([ev0.elapsed_time(ev1) / steps], dtype=torch_.float64, device=self.dev)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pick = np.unique(np.random.default_rng(5).integers(0, self.M, 4000))
        sub = self.csr.toscipy()[pick]
        want = np.asarray(sub @ self.B_host.astype(np.float64))
        got = full[torch_.from_numpy(pick).to(self.dev)].cpu().numpy()
        return {"mode": mode, "ms_per_step": float(t.item()), "gflops": 2.0 * self.nnz * self.N / float(t.item()) / 1e6,
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


class BsrProblem:
    """8x8 block path (config 5): block rows split evenly over the ranks (every block row holds
    the same number of blocks), B replicated."""

    def __init__(self, args, rank, world, dev):
        import torch
        from liteform_ae_b200 import bsr
        self.bsr, self.torch, self.dev = bsr, torch, dev
        desc, _, full_rows, N0 = WORKLOADS[args.workload]
        self.N = N = args.feat or N0
        t0 = time.perf_counter()
        indptr, indices, blocks, shape = synth.banded_blocks(M=args.rows or full_rows)
        self.M, self.K = shape
        self.B_host = synth.dense_features(self.K, N, args.seed)
        self.t_gen = time.perf_counter() - t0
        self.indptr, self.indices, self.blocks = indptr, indices, blocks
        self.nnz = int(blocks.size)
        Mb = self.M // 8
        self.r0, self.r1 = (Mb * rank) // world, (Mb * (rank + 1)) // world   # block rows
        self.tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.dtype]
        self.dtype = args.dtype
        if args.dtype == "f32":
            self.kernel = "bsr8_spmm_f32_narrow_kernel" if N <= 32 else "bsr8_spmm_f32_kernel"
        else:
            self.kernel = ("bsr8_spmm_16bit_narrow_kernel" if N <= 32 else
                           "bsr8_spmm_16bit_mid_kernel" if N <= 64 else "bsr8_spmm_16bit_kernel")
        name = {"f32": "float32", "bf16": "bfloat16", "f16": "float16"}[args.dtype]
        self.a = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, name, dev)
        self.B = torch.from_numpy(self.B_host).to(dev).to(self.tdt)
        self.C = torch.empty(((self.r1 - self.r0) * 8, N), dtype=torch.float32, device=dev)
        self.launches_per_step = 1
        eb = 4 if args.dtype == "f32" else 2
        self.eb = eb
        self.config = {"workload": f"{args.workload}: {desc}", "format": "bsr 8x8", "rows": self.M, "cols": self.K,
                       "nnz": self.nnz, "N": N, "input_dtype": args.dtype, "accumulate": "f32",
                       "sharding": f"block rows, even split, {world} rank(s), B replicated, C left sharded",
                       "l2": "inputs exceed L2 (A %.0f MB + B %.0f MB per rank); no flush between steps" % (
                           self.nnz * eb / 1e6 / world, self.B_host.size * eb / 1e6)}
        self.extra = {"generate_s": self.t_gen}
        if not args.no_build_timing:
            self.extra.update(self.time_device_builder(name))

    def time_device_builder(self, dtype_name):
        """CSR -> 8x8 blocks on the device (lf_bsr8_plan + lf_bsr8_fill), timed on the element CSR form
        of this matrix.  The CSR arrays are laid out on the device from the block arrays (every block
        row of the synthetic matrix holds the same number of blocks, so this is a reshape)."""
        torch = self.torch
        from liteform_ae_b200 import hyb
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

    def prepare_e2e(self):
        torch = self.torch
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
        h2d = sum(t.numel() * t.element_size() for t in host)
        return h2d, self.h_C[0].numel() * 4, "spmm_bsr8 on buffers copied from/to pinned host memory every step"

    def e2e_step(self, slot=0, sync=True):
        torch = self.torch
        with torch.cuda.stream(self.e2e_streams[slot]):
            for d, h in zip(self.d_in[slot], (self.h_ptr, self.h_idx, self.h_blk, self.h_B)):
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

    def cpu_matrix(self):
        import scipy.sparse as sp
        return sp.bsr_matrix((self.blocks, self.indices, self.indptr), shape=(self.M, self.K)).tocsr()


def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    use_bsr = args.format == "bsr8" or (args.format == "auto" and args.workload == "blocks")
    prob = (BsrProblem if use_bsr else HybProblem)(args, rank, world, dev)
    N = prob.N

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    for _ in range(args.warmup):
        prob.step()
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    t_wall0 = time.perf_counter()
    ev[0].record()
    for i in range(args.steps):
        prob.step()
        ev[i + 1].record()
    barrier()
    t_wall1 = time.perf_counter()
    sampler.stop()
    total_ms = ev[0].elapsed_time(ev[-1])
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max = float(t.item())
    clocks = sampler.summary(t_wall0, t_wall1)

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
        # (2) two calls in flight on two streams (own workspace and result buffer each): the result
        # of one step crosses the bus while the operands of the next one come in.  Every step still
        # copies all its inputs in and its whole result out inside the timed region.
        for slot in (0, 1):
            prob.e2e_step(slot, sync=False)
        prob.e2e_sync()
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            prob.e2e_step(i % 2, sync=False)
        prob.e2e_sync()
        barrier()
        t_two = (time.perf_counter() - t0) / e2e_steps
        te = torch.tensor([t_one, t_two], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        t_one, t_two = float(te[0].item()), float(te[1].item())
        resident = prob.C.cpu().numpy()
        e2e = {"value": 2.0 * prob.nnz * N / min(t_one, t_two) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": min(t_one, t_two) * 1e3, "steps": e2e_steps, "call": call,
               "mode": "two calls in flight on two streams" if t_two < t_one else "one call at a time",
               "ms_per_step_one_call_at_a_time": t_one * 1e3, "ms_per_step_two_in_flight": t_two * 1e3,
               "max_abs_diff_vs_resident_run": float(max(np.abs(prob.e2e_result(k) - resident).max() for k in (0, 1)))}
    except Exception as exc:  # keep the device-resident numbers, say what went wrong
        e2e = {"value": None, "unit": UNIT, "error": repr(exc)}

    # ---- optional: the whole C on every rank (NCCL all-gather after the product, or fused) -----
    gather = None
    if args.gather != "none" and world > 1 and isinstance(prob, HybProblem):
        try:
            gather = prob.time_gather(args.gather, rank, world, max(3, min(args.steps, 30)), barrier)
        except Exception as exc:
            gather = {"mode": args.gather, "error": repr(exc)}

    if rank != 0:
        return
    peak, peak_kind = measured_peak_gbs()
    launch_ms = statistics.fmean(step_ms)
    alg, gath = prob.bytes_models()
    achieved = alg / (launch_ms * 1e-3) / 1e9
    key = (args.workload, "bsr8" if use_bsr else "hyb", prob.dtype, N, args.parts, world)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(key),
                "peak_kind": f"of {peak_kind}", "kernel": prob.kernel,
                "algorithmic_bytes_per_launch": int(alg), "launch_ms": launch_ms,
                "launch_ms_median": statistics.median(step_ms),
                "gather_model_bytes_per_launch": int(gath),
                "gather_model_gbs": gath / (launch_ms * 1e-3) / 1e9}
    if roofline["traffic"]:
        roofline["dram_gbs_from_traffic"] = roofline["traffic"] / (launch_ms * 1e-3) / 1e9

    cpu = None
    if world == 1 and not args.no_cpu:
        A = prob.cpu_matrix()
        gf, t_pass, used_rows, used_nnz, passes = time_cpu(A, prob.B_host, 1, 12.0, 2)
        cpu = {"value": gf, "unit": UNIT, "cores": 1, "kind": "port",
               "sample": f"scipy csr @ dense (float32), first {used_rows} of {prob.M} rows ({used_nnz} nnz), median of {passes} passes, {t_pass:.2f} s per pass"}
        threads = os.cpu_count() or 1
        if threads > 1:
            gfm, tm, ur, un, ps = time_cpu(A, prob.B_host, threads, 6.0, 2)
            cpu["all_cores"] = {"value": gfm, "cores": threads, "sample": f"{ur} rows split over {threads} threads, {tm:.2f} s per pass"}

    line = {
        "metric": METRIC, "value": 2.0 * prob.nnz * N * args.steps / (total_ms_max * 1e-3) / 1e9, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms_max / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": prob.dtype,
        "data": "synthetic (seeded, numpy default_rng)", "config": prob.config,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
        "gpu_launches": prob.launches_per_step * args.steps,
    }
    line.update(prob.extra)
    if gather is not None:
        line["gather"] = gather
    if args.per_bucket and hasattr(prob, "per_bucket"):
        line["per_bucket"] = prob.per_bucket(20)
    print(json.dumps(line), flush=True)


# DRAM bytes (read + write) of one launch of the dominant kernel, taken from the ncu captures
# summarised under profiles/; keyed by (workload, format, dtype, N, num_parts, n_gpus).  Absent
# entries are reported as null.
TRAFFIC_BYTES_PER_LAUNCH = {
    # profiles/spmm_hyb_powerlaw_n128.md (full-size capture)
    ("powerlaw", "hyb", "f32", 128, 1, 1): 3124605000 + 543989248,
    # profiles/spmm_hyb_uniform_n64_skew_n256.md (full-size captures)
    ("uniform", "hyb", "f32", 64, 1, 1): 33724907264 + 1074169856,
    ("skew", "hyb", "f32", 256, 1, 1): 21397719552 + 1109027072,
    # profiles/spmm_bsr8_blocks_n128.md (captured at 2^20 rows, scaled x2 to the 2^21-row matrix)
    ("blocks", "bsr8", "f32", 128, 1, 1): 2 * (918607360 + 508638720),
    ("blocks", "bsr8", "bf16", 128, 1, 1): 2 * (494361600 + 492801280),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="powerlaw", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="override the matrix dimension (tests)")
    ap.add_argument("--feat", type=int, default=0, help="override the feature width N")
    ap.add_argument("--parts", type=int, default=1, help="number of column partitions")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--format", default="auto", choices=["auto", "hyb", "bsr8"],
                    help="auto: 8x8 block kernels for the block workload, composed format otherwise")
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16", "f16"], help="input type of the block path")
    ap.add_argument("--per-bucket", action="store_true", help="also time every ELL bucket on its own")
    ap.add_argument("--gather", default="none", choices=["none", "nccl", "fused"],
                    help="multi-GPU only: also time product + full C on every rank (NCCL all-gather or fused epilogue)")
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
