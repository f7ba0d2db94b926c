"""Matrix container with the surface of the reference's ``format_matrix_market`` module.

``MTX`` keeps one ``scipy.sparse.coo_matrix`` in ``coo_mtx`` exactly like the reference
(playground_pipline/format_matrix_market.py:40-205) and adds cached canonical-CSR views on
the host and on the device, which the CUDA path consumes.  ``Bucket`` is kept for API
compatibility (format_matrix_market.py:12-37); the width search here works on counters.
"""
from __future__ import annotations

from os.path import basename, splitext

import numpy as np
from scipy import sparse as sp

__all__ = ["MTX", "Bucket"]

_DGL_NAMES = ['cora', 'citeseer', 'pubmed', 'ppi', 'arxiv', 'proteins', 'reddit']


class Bucket:
    def __init__(self, bucket_width: int, num_rows: int, nnz: int, row_indices: list, col_indices: set):
        self.bucket_width = bucket_width
        self.num_rows = num_rows
        self.nnz = nnz
        self.row_indices = row_indices
        self.col_indices = col_indices

    def __str__(self):
        head = (f"Bucket(bucket_width={self.bucket_width}, num_rows={self.num_rows}, nnz={self.nnz}, "
                f"len(row_indices)={len(self.row_indices)}, ")
        if len(self.row_indices) < 11 and len(self.col_indices) < 11:
            return head + (f"row_indices={self.row_indices}, len(col_indices)={len(self.col_indices)}, "
                           f"col_indices={self.col_indices})")
        return head + f"len(col_indices)={len(self.col_indices)})"


class MTX:
    def __init__(self, filename=None) -> None:
        self._csr_cache = None      # (id(coo_mtx), scipy csr)
        self._dev_cache = {}        # device -> (id(coo_mtx), DeviceCsr)
        if filename is None:
            # empty shell: assign ``coo_mtx`` afterwards (format_matrix_market.py:44-46)
            self.name = None
            self.coo_mtx = None
        elif filename in _DGL_NAMES:
            # The reference fetches these seven graphs through DGL/OGB (format_matrix_market.py:47-56).
            # Here they are read from local files: <LITEFORM_DATA_DIR>/<name>.npz (scipy.sparse.save_npz
            # of the adjacency matrix) or <name>.mtx; data is set to ones as the reference does (:53).
            import os
            root = os.environ.get("LITEFORM_DATA_DIR", "")
            self.name = filename
            npz, mtx = os.path.join(root, filename + ".npz"), os.path.join(root, filename + ".mtx")
            if root and os.path.isfile(npz):
                self.coo_mtx = sp.coo_matrix(sp.load_npz(npz))
            elif root and os.path.isfile(mtx):
                from scipy.io import mmread
                self.coo_mtx = sp.coo_matrix(mmread(mtx))
            else:
                raise RuntimeError(
                    f"dataset '{filename}' is downloaded through DGL/OGB by the reference "
                    "(format_matrix_market.py:47-56); there is no network here. Put <name>.npz or <name>.mtx "
                    "into the directory named by LITEFORM_DATA_DIR, build the matrix with MTX.from_csr / "
                    "MTX.from_coo, or load a .mtx file by path.")
            self.coo_mtx.data = np.ones(len(self.coo_mtx.data))
        else:
            from scipy.io import mmread
            self.name = splitext(basename(filename))[0]
            self.coo_mtx = sp.coo_matrix(mmread(filename))
            self.coo_mtx.data = np.ones(len(self.coo_mtx.data))  # format_matrix_market.py:63-64

    # ---- constructors for in-memory matrices (new) ---------------------------------------
    @classmethod
    def from_coo(cls, coo, name="matrix") -> "MTX":
        g = cls(None)
        g.name = name
        g.coo_mtx = sp.coo_matrix(coo)
        return g

    @classmethod
    def from_csr(cls, indptr, indices, data, shape, name="matrix") -> "MTX":
        g = cls(None)
        g.name = name
        csr = sp.csr_matrix((np.asarray(data), np.asarray(indices), np.asarray(indptr)), shape=shape)
        g.coo_mtx = csr.tocoo()
        if csr.has_sorted_indices:
            g._csr_cache = (id(g.coo_mtx), csr)
        return g

    # ---- the reference's methods -----------------------------------------------------------
    def adj_tensors(self, format: str):
        if format == "coo":
            return self.coo_mtx.row, self.coo_mtx.col
        elif format == "csc":
            csc = self.coo_mtx.tocsc()
            return csc.indptr, csc.indices, csc.data
        elif format == "csr":
            csr = self.csr_host()
            return csr.indptr, csr.indices, csr.data
        raise TypeError(F"Format {format} is not suppoted.")

    def num_src_nodes(self):
        return self.coo_mtx.shape[0]

    def num_dst_nodes(self):
        return self.coo_mtx.shape[1]

    def num_edges(self):
        return self.coo_mtx.nnz

    def dot(self, B):
        """A * B with SciPy (CSC times dense), the reference's golden product."""
        return self.coo_mtx.tocsc().dot(B)

    def tobsr(self, blocksize=None, copy=False):
        return self.coo_mtx.tobsr(blocksize=blocksize, copy=copy)

    def tobsr_with_padding(self, shape, blocksize=None):
        """BSR copy with fp16 block data on a padded shape (format_matrix_market.py:116-138).
        Current SciPy refuses to construct float16 sparse matrices, so the matrix is assembled in
        float32 and its block array is narrowed afterwards."""
        data = np.array(self.coo_mtx.data, dtype=np.float32)
        ij = [self.coo_mtx.row, self.coo_mtx.col]
        bsr = sp.bsr_matrix((data, ij), blocksize=blocksize, shape=shape)
        bsr.sort_indices()
        bsr.data = bsr.data.astype(np.float16)
        return bsr

    def tobsr_device(self, shape=None, dtype="float16", device="cuda"):
        """Device-side counterpart of ``tobsr_with_padding`` for 8x8 blocks: the CSR form is
        uploaded once (and cached), the blocks are cut on the device.  Returns ``bsr.DeviceBsr8``."""
        from .bsr import DeviceBsr8
        return DeviceBsr8.from_csr_device(self.csr_device(device), dtype=dtype, padded_shape=shape)

    def tocsr(self, copy=False):
        return self.coo_mtx.tocsr(copy=copy)

    def matrix_features(self):
        num_rows, num_cols = self.coo_mtx.shape
        indptr, _, _ = self.adj_tensors("csr")
        assert len(indptr) == num_rows + 1, \
            F"len(indptr) {len(indptr)} is not equal to num_rows + 1 ({num_rows + 1})."
        nnz_per_row = np.diff(indptr)
        avg = np.mean(nnz_per_row)
        lo, hi = nnz_per_row.min(), nnz_per_row.max()
        return {
            "name": self.name,
            "num_rows": num_rows,
            "num_cols": num_cols,
            "nnz": self.coo_mtx.nnz,
            "avg_nnz_per_row": avg,
            "min_nnz_per_row": lo,
            "max_nnz_per_row": hi,
            "std_dev_nnz_per_row": np.std(nnz_per_row),
            "avg_nnz_density_per_row": avg / num_cols,
            "min_nnz_density_per_row": lo / num_cols,
            "max_nnz_density_per_row": hi / num_cols,
            "std_dev_nnz_density_per_row": np.std(nnz_per_row / num_cols),
        }

    def matrix_features_device(self, device="cuda"):
        """Same dictionary as ``matrix_features`` with the per-row pass done on the device
        (``lf_row_stats``).  Sums are exact integers, so the means and extrema are identical to the
        host version and the standard deviations agree to rounding (the reference sums squared
        deviations in floating point; here the variance is formed from exact integer moments)."""
        import math
        from fractions import Fraction
        from .hyb import row_length_stats
        num_rows, num_cols = self.coo_mtx.shape
        n, total, squares, lo, hi = row_length_stats(self.csr_device(device))
        avg = total / n
        var = Fraction(n * squares - total * total, n * n)
        std = math.sqrt(var)
        return {
            "name": self.name, "num_rows": num_rows, "num_cols": num_cols, "nnz": self.coo_mtx.nnz,
            "avg_nnz_per_row": avg, "min_nnz_per_row": lo, "max_nnz_per_row": hi, "std_dev_nnz_per_row": std,
            "avg_nnz_density_per_row": avg / num_cols, "min_nnz_density_per_row": lo / num_cols,
            "max_nnz_density_per_row": hi / num_cols, "std_dev_nnz_density_per_row": std / num_cols,
        }

    def __str__(self):
        return str(self.coo_mtx)

    # ---- cached canonical views (new) ------------------------------------------------------
    def csr_host(self):
        """Canonical CSR (sorted columns, duplicates merged) of ``coo_mtx``, cached."""
        if self._csr_cache is None or self._csr_cache[0] != id(self.coo_mtx):
            csr = self.coo_mtx.tocsr()
            csr.sort_indices()
            self._csr_cache = (id(self.coo_mtx), csr)
        return self._csr_cache[1]

    def has_duplicates(self) -> bool:
        """True if ``coo_mtx`` stores a (row, col) pair more than once.  The reference counts
        degrees on COO entries (format_algos.py:249-252) but takes entries from the merged CSR
        (format_algos.py:254), so its output on such input is not a valid format."""
        return self.csr_host().nnz != self.coo_mtx.nnz

    def csr_device(self, device="cuda"):
        from .hyb import DeviceCsr
        key = str(device)
        hit = self._dev_cache.get(key)
        if hit is None or hit[0] != id(self.coo_mtx):
            if self.has_duplicates():
                raise ValueError("the matrix holds duplicate (row, col) entries; merge them first "
                                 "(coo.sum_duplicates())")
            csr = self.csr_host()
            dev = DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, device)
            self._dev_cache[key] = (id(self.coo_mtx), dev)
            hit = self._dev_cache[key]
        return hit[1]
