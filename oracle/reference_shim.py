"""TEST INFRASTRUCTURE ONLY -- loader for the unmodified LiteForm reference modules.

The reference's ``playground_pipline/format_algos.py`` and
``playground_pipline/format_matrix_market.py`` are pure Python, but they import
packages that do not exist in this image (``tvm``, ``sparsetir_artifact``,
``dgl``, ``ogb``) and one that fails to import under current scikit-learn
(its own ``utils`` module).  ``load_reference()`` installs inert stand-ins for
those imports and returns the two modules exactly as they lie on disk, so the
format side of the path (``search_bucket_config`` format_algos.py:988-1032,
``build_hyb_format`` format_algos.py:226-385) can be executed as the ground truth
for the restatement in ``hyb_oracle.py`` and to generate ``tests/golden``.

Nothing in the shipped package imports this file.  It only works where a checkout
of the reference is present and the environment variable ``LITEFORM_REFERENCE_ROOT`` names it;
``reference_available()`` says whether that is the case.
"""
from __future__ import annotations

import os
import sys
import types
from unittest.mock import MagicMock

# The checkout's location comes from the environment only; without it the reference is "absent".
_DEFAULT_ROOT = os.environ.get("LITEFORM_REFERENCE_ROOT", "")
_SUBDIR = "playground_pipline"
_ABSENT = ["tvm", "tvm.testing", "tvm.tir", "tvm.script", "tvm.sparse",
           "sparsetir_artifact", "dgl", "dgl.data", "ogb", "ogb.nodeproppred"]
_cache = {}


def reference_available(root: str = _DEFAULT_ROOT) -> bool:
    return bool(root) and os.path.isfile(os.path.join(root, _SUBDIR, "format_algos.py"))


def load_reference(root: str = _DEFAULT_ROOT):
    """Return ``(format_algos, format_matrix_market)`` of the reference checkout."""
    if root in _cache:
        return _cache[root]
    if not reference_available(root):
        raise FileNotFoundError(f"no LiteForm reference under {root!r} (set LITEFORM_REFERENCE_ROOT to the checkout)")
    import numpy as np

    saved = {k: sys.modules.get(k) for k in _ABSENT + ["utils", "format_algos", "format_matrix_market"]}
    for name in _ABSENT:
        sys.modules[name] = MagicMock(name=name)
    stub_utils = types.ModuleType("utils")

    def _no_dataset(name):
        raise KeyError(f"dataset download is not available: {name}")

    stub_utils.get_dataset = _no_dataset
    sys.modules["utils"] = stub_utils
    had_np_str = hasattr(np, "str")
    if not had_np_str:
        np.str = str  # format_algos.py:50 evaluates ``np.str`` in an annotation
    path = os.path.join(root, _SUBDIR)
    sys.path.insert(0, path)
    try:
        sys.modules.pop("format_algos", None)
        sys.modules.pop("format_matrix_market", None)
        import format_algos as fa  # type: ignore
        import format_matrix_market as mm  # type: ignore
    finally:
        sys.path.remove(path)
        # the reference modules stay reachable through the returned objects only
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    _cache[root] = (fa, mm)
    return fa, mm


def reference_mtx(coo, name="synthetic", root: str = _DEFAULT_ROOT):
    """Wrap a scipy COO matrix in the reference's ``MTX`` container (format_matrix_market.py:44-46)."""
    _, mm = load_reference(root)
    g = mm.MTX(None)
    g.name = name
    g.coo_mtx = coo
    return g
