"""CUDA-event timing with a cold L2, the protocol of the reference's timing helper
(playground_pipline/format_algos.py:164-202: a 256 MB buffer is rewritten before every timed
run, events bracket the call) with real warm-up and repeat counts."""
from __future__ import annotations

import statistics
from typing import Callable, List

_FLUSH_BYTES = 512 * 1024 * 1024   # > 4x the 126 MB L2 of a B200
_flush_buf = {}


def _flush_buffer(torch, device):
    key = str(device)
    if key not in _flush_buf:
        _flush_buf[key] = torch.empty(_FLUSH_BYTES, dtype=torch.int8, device=device)
    return _flush_buf[key]


def time_ms(fn: Callable[[], None], warmup: int = 10, repeat: int = 100, flush_l2: bool = True,
            device=None) -> List[float]:
    """Per-iteration device times (ms) of ``fn`` on the current stream."""
    import torch
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    buf = _flush_buffer(torch, device) if flush_l2 else None
    for _ in range(warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(repeat)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(repeat)]
    torch.cuda.synchronize(device)
    for i in range(repeat):
        if buf is not None:
            buf.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize(device)
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def profile_ms(fn: Callable[[], None], warmup: int = 10, repeat: int = 100, flush_l2: bool = True) -> float:
    """Mean time in ms (what the reference's ``profile_tvm_ms`` returns, format_algos.py:601)."""
    return statistics.fmean(time_ms(fn, warmup, repeat, flush_l2))


def median_ms(fn: Callable[[], None], warmup: int = 10, repeat: int = 100, flush_l2: bool = True) -> float:
    return statistics.median(time_ms(fn, warmup, repeat, flush_l2))
