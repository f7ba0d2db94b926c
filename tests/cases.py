"""Seeded matrices shared by the CPU and GPU tests (names match tests/golden/hyb_golden.json)."""
import numpy as np

from liteform_ae_b200 import synth

GENERATORS = {
    "zipf_16384_s0": lambda: synth.zipf_rows(),
    "zipf_2048_s5": lambda: synth.zipf_rows(M=2048, seed=5),
    "powerlaw_8192_s1": lambda: synth.power_law_graph(M=8192, seed=1),
    "uniform32_4096_s2": lambda: synth.uniform_rows(M=4096, seed=2),
    "skew_8192_s3": lambda: synth.skewed_rows(M=8192, seed=3),
    "blocks_4096_s4": lambda: synth.bsr_to_csr(*synth.banded_blocks(M=4096, seed=4)),
    "powerlaw_1048576_s1": lambda: synth.power_law_graph(),
    "skew_1048576_s3": lambda: synth.skewed_rows(),
    "uniform32_4194304_s2": lambda: synth.uniform_rows(),
    "blocks_2097152_s4": lambda: synth.bsr_to_csr(*synth.banded_blocks()),
}
SMALL = ["zipf_16384_s0", "zipf_2048_s5", "powerlaw_8192_s1", "uniform32_4096_s2", "skew_8192_s3",
         "blocks_4096_s4"]
FULL = ["powerlaw_1048576_s1", "skew_1048576_s3", "uniform32_4194304_s2", "blocks_2097152_s4"]

_cache = {}


def matrix(name):
    if name not in _cache:
        if len(_cache) > 6:
            _cache.clear()
        _cache[name] = GENERATORS[name]()
    return _cache[name]


def edge_csr(rec):
    indptr = np.asarray(rec["indptr"], dtype=np.int64)
    indices = np.asarray(rec["indices"], dtype=np.int32)
    data = np.ones(len(indices), dtype=np.float32)
    return synth.Csr(indptr, indices, data, tuple(rec["shape"]), "edge")


def csr_digest(csr):
    import hashlib
    h = hashlib.sha256()
    h.update(np.ascontiguousarray(csr.indptr, dtype=np.int64).tobytes())
    h.update(np.ascontiguousarray(csr.indices, dtype=np.int32).tobytes())
    h.update(np.ascontiguousarray(csr.data, dtype=np.float32).tobytes())
    return h.hexdigest()
