"""Small host utilities with the reference's names (src/af3_kernels/tools.py)."""
from __future__ import annotations

from functools import wraps
from os import environ

import torch

DO_PROFILE = environ.get("DO_PROFILE", "0") == "1"
USE_DIST = environ.get("USE_DIST", "0") == "1"


def profile(name: str = None):
    """Wraps a function in a torch.profiler range when DO_PROFILE=1 (reference: tools.py:20-33)."""

    def decorator(func):
        if not DO_PROFILE:
            return func

        @wraps(func)
        def wrapper(*args, **kwargs):
            with torch.profiler.record_function(func.__name__ if name is None else name):
                return func(*args, **kwargs)

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
