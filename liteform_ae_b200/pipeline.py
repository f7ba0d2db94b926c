"""The caller of the hot path: the reference's end-to-end driver as a library.

``playground_pipline/proc05.spmm.end-to-end.py`` is a script: for every matrix it asks a
classifier whether the composed format ("CELL") pays off (lines 65-79), and then either
  * asks a second classifier for the number of column partitions (82-97), searches the bucket
    widths, builds the format and times the product for N in 32..512 (136-188), or
  * pads the matrix to a square multiple of 32, converts it to 32x32 fp16 blocks and times the
    block product, falling back to the CSR product when that fails (190-257),
and collects one table row per (matrix, N) (260-273).  The functions here do the same steps
with the same decisions and the same column names, on this package's device paths: row
statistics from ``lf_row_stats``, width search / format / product from the composed-format
entry points, blocks cut on the device, CSR product as the last resort.

The two classifiers are scikit-learn models the reference ships as pickles; they are not part
of this package.  Pass anything with a ``predict`` method (``joblib.load`` of the reference's
files works); ``clf_partition=None`` falls back to this package's own chooser
(``format_algos.suggest_num_parts``), which is not the reference's model.
"""
from __future__ import annotations

import math
import sys
import time
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

from . import format_algos as fa
from .format_matrix_market import MTX

FORMAT_SELECTION_FEATURES = ["num_rows", "num_cols", "nnz", "avg_nnz_per_row", "min_nnz_per_row",
                             "max_nnz_per_row", "std_dev_nnz_per_row"]
NUM_PARTITIONS_FEATURES = ["num_rows", "num_cols", "nnz", "avg_nnz_density_per_row", "min_nnz_density_per_row",
                           "max_nnz_density_per_row", "std_dev_nnz_density_per_row"]
FEAT_SIZES = (32, 64, 128, 256, 512)
TABLE_COLUMNS = ["name", "format", "feat_size", "num_parts", "time_select(s)", "time_num_parts(s)",
                 "time_bucket(s)", "time_exe_our(ms)"]


def _features(g: MTX, device) -> Dict[str, float]:
    return g.matrix_features_device(device) if device is not None else g.matrix_features()


def get_X_for_format_selection(g: MTX, device="cuda"):
    """Feature vector of the format classifier (proc05:26-47): one row, seven columns."""
    f = _features(g, device)
    return [np.array([f[k] for k in FORMAT_SELECTION_FEATURES])]


def get_X_for_num_partitions(g: MTX, num_features: int, device="cuda"):
    """Feature vector of the partition-count model (proc05:50-62): densities plus N."""
    f = _features(g, device)
    return [np.array([f[k] for k in NUM_PARTITIONS_FEATURES] + [num_features])]


def predict_format_selection(g: MTX, clf, device="cuda"):
    """``("CELL" | "BCSR", seconds)``; class 1 means the composed format (proc05:65-79)."""
    X = get_X_for_format_selection(g, device)
    t0 = time.perf_counter()
    y = clf.predict(X)
    dt = time.perf_counter() - t0
    return ("CELL" if y[0] == 1 else "BCSR"), dt


def predict_num_partitions(g: MTX, clf, num_features: int, device="cuda"):
    """``(num_parts, seconds)`` (proc05:82-97).  ``clf=None``: this package's own chooser."""
    if clf is None:
        t0 = time.perf_counter()
        parts = fa.suggest_num_parts(g, num_features, device=device)
        parts = parts[0] if isinstance(parts, tuple) else parts
        return int(parts), time.perf_counter() - t0
    X = get_X_for_num_partitions(g, num_features, device)
    t0 = time.perf_counter()
    y = clf.predict(X)
    return int(y[0]), time.perf_counter() - t0


def _time_composed(g: MTX, num_features: int, num_parts: int, device, repeat: int):
    import torch
    t0 = time.perf_counter()
    cfg = fa.CostModelSettings(feat_size=num_features, num_parts=num_parts)
    widths = fa.search_bucket_config(g, num_parts, cfg, device=device)
    t_bucket = time.perf_counter() - t0
    fmt = fa.build_hyb_format_device(g, widths, device=device, with_mask=False)
    x = torch.ones((g.num_dst_nodes(), num_features))
    ms = fa.bench_hyb_with_config(g, x, None, feat_size=num_features, bucket_widths=widths, bucketing_format=fmt,
                                  coarsening_factor=2, num_col_parts=num_parts, use_implicit_unroll=True,
                                  device=device, repeat=repeat)
    return t_bucket, ms, widths


def _time_blocks(g: MTX, num_features: int, block_size: int, device, repeat: int):
    """The reference pads to a square multiple of the block size (proc05:196-208) and uses fp16."""
    import torch
    from . import bsr
    from .timing import profile_ms
    side = max(g.num_src_nodes(), g.num_dst_nodes())
    side = -(-side // block_size) * block_size
    a = g.tobsr_device(shape=(side, side), dtype="float16", device=device)
    x = torch.rand(side, num_features).half().to(device)
    out = bsr.spmm_bsr8(a, x)
    return profile_ms(lambda: bsr.spmm_bsr8(a, x, out=out), warmup=min(10, repeat), repeat=repeat)


def _time_csr(g: MTX, num_features: int, device, repeat: int):
    import torch
    x = torch.rand((g.num_dst_nodes(), num_features))
    return fa.bench_naive(g, x, None, feat_size=num_features, coarsening_factor=2, device=device, repeat=repeat)


def run_matrix(g: MTX, clf_selection, clf_partition=None, feat_sizes: Iterable[int] = FEAT_SIZES,
               block_size: int = 32, device="cuda", repeat: int = 100,
               num_parts_override: Optional[int] = None, log=None) -> List[dict]:
    """One table row per feature size for one matrix, following proc05:127-257."""
    log = log or (lambda *a, **k: None)
    fmt_name, t_select = predict_format_selection(g, clf_selection, device)
    log(f"name: {g.name} format: {fmt_name} time(s): {t_select}")
    rows = []
    for n in feat_sizes:
        rec = {"name": g.name, "format": fmt_name, "feat_size": int(n), "num_parts": 0, "time_select(s)": t_select,
               "time_num_parts(s)": 0, "time_bucket(s)": 0, "time_exe_our(ms)": 0}
        if fmt_name == "CELL":
            parts, t_parts = predict_num_partitions(g, clf_partition, n, device)
            if num_parts_override is not None:
                parts = int(num_parts_override)
            rec.update({"num_parts": parts, "time_num_parts(s)": t_parts})
            try:
                t_bucket, ms, widths = _time_composed(g, n, parts, device, repeat)
                rec.update({"time_bucket(s)": t_bucket, "time_exe_our(ms)": ms})
                log(f"name: {g.name} format: CELL feat_size: {n} num_partitions: {parts} bucket_config: {widths} exe_time: {ms}")
            except Exception as exc:   # the driver records a failed run as an infinite time (proc05:178-180)
                print(exc, file=sys.stderr)
                rec["time_exe_our(ms)"] = math.inf
        else:
            rec["format"] = "BSR"
            try:
                rec["time_exe_our(ms)"] = _time_blocks(g, n, block_size, device, repeat)
            except Exception as exc:
                print(exc, file=sys.stderr)
                try:                       # blocks did not work out: plain CSR (proc05:232-246)
                    rec["format"] = "CSR"
                    rec["time_exe_our(ms)"] = _time_csr(g, n, device, repeat)
                except Exception as exc2:  # proc05:247-253
                    print(exc2, file=sys.stderr)
                    rec.update({"format": "CRASHED", "time_exe_our(ms)": 0})
            log(f"name: {g.name} format: {rec['format']} feat_size: {n} exe_time: {rec['time_exe_our(ms)']}")
        rows.append(rec)
    return rows


def run(matrices: Sequence[MTX], clf_selection, clf_partition=None, **kwargs) -> Dict[str, list]:
    """The driver's result table (proc05:260-269) as a dict of columns, ready for
    ``pandas.DataFrame(data=table)``."""
    table: Dict[str, list] = {c: [] for c in TABLE_COLUMNS}
    for g in matrices:
        for rec in run_matrix(g, clf_selection, clf_partition, **kwargs):
            for c in TABLE_COLUMNS:
                table[c].append(rec[c])
    return table
