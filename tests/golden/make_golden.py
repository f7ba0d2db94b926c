"""Generate ``tests/golden/hyb_golden.json`` by running the UNMODIFIED reference.

Needs a checkout of johnpzh/liteform_ae, named by the environment variable
``LITEFORM_REFERENCE_ROOT``.  For every case it feeds a seeded matrix to the reference's
``search_bucket_config`` (playground_pipline/format_algos.py:988-1032) and ``build_hyb_format``
(format_algos.py:226-385) and records the chosen widths and a sha256 digest of the int32-cast
output arrays; tiny hand-made cases also keep the arrays themselves.  The tests then require
the CPU oracle and the CUDA library to reproduce these values on any machine.

    python tests/golden/make_golden.py            # small + medium cases (about a minute)
    python tests/golden/make_golden.py --full     # adds the full-size benchmark matrices
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time
import warnings

import numpy as np
import scipy.sparse as sp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from liteform_ae_b200 import synth  # noqa: E402
from oracle import hyb_oracle as ho  # noqa: E402
from oracle import reference_shim as rs  # noqa: E402

OUT = os.path.join(HERE, "hyb_golden.json")


def csr_digest(indptr, indices, data) -> str:
    h = hashlib.sha256()
    h.update(np.ascontiguousarray(indptr, dtype=np.int64).tobytes())
    h.update(np.ascontiguousarray(indices, dtype=np.int32).tobytes())
    h.update(np.ascontiguousarray(data, dtype=np.float32).tobytes())
    return h.hexdigest()


# ---- seeded generator cases: name -> (callable returning synth.Csr, [(P, N), ...]) ----------
def generator_cases(full: bool):
    cases = {
        "zipf_16384_s0": (lambda: synth.zipf_rows(), [(1, 32), (2, 32), (4, 32), (8, 32), (16, 32)]),
        "zipf_2048_s5": (lambda: synth.zipf_rows(M=2048, seed=5), [(1, 32), (3, 32), (1, 512), (3, 512)]),
        "powerlaw_8192_s1": (lambda: synth.power_law_graph(M=8192, seed=1), [(1, 128), (4, 128)]),
        "uniform32_4096_s2": (lambda: synth.uniform_rows(M=4096, seed=2), [(1, 64), (4, 64)]),
        "skew_8192_s3": (lambda: synth.skewed_rows(M=8192, seed=3), [(1, 256), (2, 256)]),
        "blocks_4096_s4": (lambda: synth.bsr_to_csr(*synth.banded_blocks(M=4096, seed=4)), [(1, 64), (2, 64)]),
    }
    if full:
        cases.update({
            "powerlaw_1048576_s1": (lambda: synth.power_law_graph(), [(1, 128), (8, 128)]),
            "skew_1048576_s3": (lambda: synth.skewed_rows(), [(1, 256)]),
            "uniform32_4194304_s2": (lambda: synth.uniform_rows(), [(1, 64)]),
            # config 5 as element CSR (every row holds 64 entries): the composed format of the block matrix
            "blocks_2097152_s4": (lambda: synth.bsr_to_csr(*synth.banded_blocks()), [(1, 128)]),
        })
    return cases


# ---- hand-made edge cases --------------------------------------------------------------------
def _rows_to_csr(rows, K):
    indptr = np.zeros(len(rows) + 1, dtype=np.int64)
    np.cumsum([len(r) for r in rows], out=indptr[1:])
    indices = np.asarray([c for r in rows for c in sorted(r)], dtype=np.int32)
    return indptr, indices, np.ones(len(indices), dtype=np.float32), (len(rows), K)


def edge_cases():
    rng = np.random.default_rng(99)
    K = 64
    out = {}
    # a row of degree 11 forced into width 2: six ELL rows with one row id
    out["deg11_width2"] = dict(csr=_rows_to_csr([list(range(11)), [3]], K), P=1, N=32, force_widths=[[2]])
    # a column partition without entries -> [] for that partition
    out["empty_partition"] = dict(csr=_rows_to_csr([[0, 1, 2], [1, 5], [2, 3, 4, 6]], K), P=4, N=32)
    # a partition holding exactly one nonzero -> ValueError
    out["single_nnz_partition"] = dict(csr=_rows_to_csr([[0, 1, 40], [1, 2], [2, 3]], K), P=2, N=32)
    # empty rows never show up in the format
    out["empty_rows"] = dict(csr=_rows_to_csr([[], [1, 2], [], [], [0, 5, 9, 11], []], K), P=1, N=32)
    # 20 rows of degree 2, one of degree 7, 10 of degree 16: an EMPTY bucket of width 4 appears
    rows = [sorted(rng.choice(K, 2, replace=False).tolist()) for _ in range(20)]
    rows.append(sorted(rng.choice(K, 7, replace=False).tolist()))
    rows += [sorted(rng.choice(K, 16, replace=False).tolist()) for _ in range(10)]
    out["lone_row_fixup"] = dict(csr=_rows_to_csr(rows, K), P=1, N=32)
    # a lone width-1 row next to wider buckets: moved UP to the next width of the snapshot
    rows = [[5]] + [sorted(rng.choice(K, 4, replace=False).tolist()) for _ in range(6)] + \
           [sorted(rng.choice(K, 8, replace=False).tolist()) for _ in range(3)]
    out["lone_width1_row"] = dict(csr=_rows_to_csr(rows, K), P=1, N=64)
    # lone width-1 row whose next snapshot width was itself moved away just before
    rows = [[7]] + [sorted(rng.choice(K, 13, replace=False).tolist())]
    out["lone_width1_and_lone_wide"] = dict(csr=_rows_to_csr(rows, K), P=1, N=32)
    # a row far beyond the widest class (degree 3000 -> class 1024 counted 4 times)
    big = 4096
    rows = [sorted(rng.choice(big, 3000, replace=False).tolist())] + \
           [sorted(rng.choice(big, int(d), replace=False).tolist()) for d in rng.integers(1, 40, 200)]
    out["deg3000"] = dict(csr=_rows_to_csr(rows, big), P=1, N=128)
    out["deg3000_p3"] = dict(csr=_rows_to_csr(rows, big), P=3, N=128)
    return out


def run_reference(fa, g, P, N, force_widths=None):
    rec = {"P": P, "N": N}
    try:
        widths = force_widths if force_widths is not None else fa.search_bucket_config(g, P, fa.CostModelSettings(N, P))
    except ValueError as e:
        rec["error"] = str(e)
        return rec, None
    rec["widths"] = [[int(w) for w in ws] for ws in widths]
    rec["forced"] = force_widths is not None
    rows, cols, mask = fa.build_hyb_format(g, widths)
    rec["digest"] = ho.digest_hyb(widths, rows, cols, mask)
    rec["ell_rows"] = [[int(r.shape[0]) for r in rp] for rp in rows]
    return rec, (rows, cols, mask)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--full", action="store_true")
    ap.add_argument("--only", default=None, help="comma-separated case names to (re)generate")
    args = ap.parse_args()
    warnings.simplefilter("ignore")
    fa, _ = rs.load_reference()
    golden = json.load(open(OUT)) if os.path.isfile(OUT) else {"generated": {}, "edge": {}}
    only = set(args.only.split(",")) if args.only else None

    for name, (make, runs) in generator_cases(args.full).items():
        if only and name not in only:
            continue
        if not only and name in golden["generated"] and not args.full:
            pass
        t0 = time.time()
        csr = make()
        g = rs.reference_mtx(csr.tocoo(), name)
        entry = {"shape": list(csr.shape), "nnz": csr.nnz,
                 "csr_digest": csr_digest(csr.indptr, csr.indices, csr.data), "runs": []}
        for P, N in runs:
            rec, _ = run_reference(fa, g, P, N)
            entry["runs"].append(rec)
            print(f"{name} P={P} N={N}: {rec.get('widths', rec.get('error'))} ({time.time() - t0:.1f}s)", flush=True)
        golden["generated"][name] = entry
        json.dump(golden, open(OUT, "w"), indent=1, sort_keys=True)

    for name, case in edge_cases().items():
        if only and name not in only:
            continue
        indptr, indices, data, shape = case["csr"]
        coo = sp.csr_matrix((data, indices, indptr), shape=shape).tocoo()
        g = rs.reference_mtx(coo, name)
        rec, arrays = run_reference(fa, g, case["P"], case["N"], case.get("force_widths"))
        rec["shape"] = list(shape)
        rec["indptr"] = indptr.tolist()
        rec["indices"] = indices.tolist()
        if arrays is not None and len(indices) < 400:
            rows, cols, mask = arrays
            rec["rows"] = [[np.asarray(a).astype(int).tolist() for a in rp] for rp in rows]
            rec["cols"] = [[np.asarray(a).astype(int).tolist() for a in cp] for cp in cols]
            rec["mask"] = [[np.asarray(a).astype(int).tolist() for a in mp] for mp in mask]
        golden["edge"][name] = rec
        print(f"edge {name}: {rec.get('widths', rec.get('error'))}")
    json.dump(golden, open(OUT, "w"), indent=1, sort_keys=True)
    print("wrote", OUT)


if __name__ == "__main__":
    main()
