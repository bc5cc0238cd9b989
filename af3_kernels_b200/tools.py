"""Small host utilities with the reference's names (src/af3_kernels/tools.py)."""
from __future__ import annotations

from functools import wraps
from os import environ

import torch

DO_PROFILE = environ.get("DO_PROFILE", "0") == "1"
USE_DIST = environ.get("USE_DIST", "0") == "1"


# Per-operator device time, gathered when DO_PROFILE=1 or AF3K_TIMERS=1: name -> [calls, [(start, end) CUDA
# events not yet folded in], milliseconds folded in].  The reference keeps per-thread rdtsc
# timers per TPP category (src/csrc/timing.h:232-265) and prints them with print_debug_timers
# (src/csrc/init.cpp:145-216); on the GPU the unit that can be timed from the host is the operator.
DO_TIMERS = DO_PROFILE or environ.get("AF3K_TIMERS", "0") == "1"
op_timers: dict = {}


def _fold(entry) -> None:
    pending = entry[1]
    if pending:
        pending[-1][1].synchronize()
        entry[2] += sum(a.elapsed_time(b) for a, b in pending)
        pending.clear()


def reset_op_timers() -> None:
    op_timers.clear()


def op_timer_totals() -> dict:
    """name -> (calls, total milliseconds on the device); waits for the recorded events."""
    out = {}
    for name, entry in op_timers.items():
        _fold(entry)
        out[name] = (entry[0], entry[2])
    return out


def profile(name: str = None):
    """With DO_PROFILE=1: wraps a function in a torch.profiler range (reference: tools.py:20-33)
    and an NVTX range, and brackets it with CUDA events on the current stream so that
    ``print_debug_timers`` can print per-operator device time.  With AF3K_TIMERS=1 only the
    events are recorded.  Otherwise the function is returned unchanged (no overhead)."""

    def decorator(func):
        if not DO_TIMERS:
            return func
        label = func.__name__ if name is None else name

        @wraps(func)
        def wrapper(*args, **kwargs):
            cuda = torch.cuda.is_available()
            if cuda:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                torch.cuda.nvtx.range_push(label)
            try:
                if DO_PROFILE:
                    with torch.profiler.record_function(label):
                        return func(*args, **kwargs)
                return func(*args, **kwargs)
            finally:
                if cuda:
                    torch.cuda.nvtx.range_pop()
                    end.record()
                    entry = op_timers.setdefault(label, [0, [], 0.0])
                    entry[0] += 1
                    entry[1].append((start, end))
                    if len(entry[1]) >= 256:
                        _fold(entry)

        return wrapper

    return decorator


comm_time_counters: dict = {}


def _rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def record_comm_time(name: str, seconds: float, size: int = 0) -> None:
    """Accumulates seconds and gigabytes per collective name on rank 0 when USE_DIST=1
    (reference: tools.py:39-45)."""
    if USE_DIST and _rank() == 0:
        c = comm_time_counters.setdefault(name, [0.0, 0.0])
        c[0] += seconds
        c[1] += size / 1e9


def print_comm_time() -> None:
    if USE_DIST and _rank() == 0:
        for name, (secs, gb) in comm_time_counters.items():
            rate = gb / secs if secs > 0 else float("nan")
            print(f"{name}\t:\t{secs:.4f} s\t{rate:.4f} GB/s\t{gb:.4f} GB")


def pad_to_size(tensor: torch.Tensor, size: int, dim: int = 0) -> torch.Tensor:
    """Zero-pads ``dim`` up to ``size`` (reference: tools.py:55-61)."""
    if tensor.shape[dim] == size:
        return tensor.contiguous()
    shape = list(tensor.shape)
    shape[dim] = size - tensor.shape[dim]
    pad = torch.zeros(shape, device=tensor.device, dtype=tensor.dtype)
    return torch.cat([tensor, pad], dim=dim).contiguous()
