"""B200 (sm_100a) drop-in for the attention hot path of HPC-SJTU/af3_kernels.

The public names and signatures follow the reference's ``src/af3_kernels/__init__.py``.  Only
the biased, key-masked dot-product attention path (hand-written CUDA behind ``libaf3k.so``) and
the two blocks and modules that wrap it are implemented; the reference's unrelated operators
(GLU / Linear, triangle multiplication) are importable but raise ``NotImplementedError``.  Nothing here computes on the CPU.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _capi
from .dpa import dot_product_attention, dot_product_attention_host, read_status
from . import tools
from .tools import pad_to_size, print_comm_time, profile, record_comm_time
from .distributed import RowShardedAttention, row_partition
from .fused_ops import attention_block, self_attention_block
from .Attention import GridSelfAttentionCpp, DistributedGridSelfAttentionCpp

__all__ = [
    "dot_product_attention_cpp",
    "dot_product_attention",
    "dot_product_attention_host",
    "RowShardedAttention",
    "row_partition",
    "GridSelfAttentionCpp",
    "DistributedGridSelfAttentionCpp",
    "attention_block",
    "self_attention_block",
    "gated_linear_unit_cpp",
    "_attention_cpp",
    "self_attention_cpp",
    "pad_and_align_tensor",
    "vnni_repack_tensor",
    "reset_debug_timers",
    "print_debug_timers",
    "print_debug_thread_imbalance",
    "Linear",
    "TriangleMultiplicationCpp",
    "DistributedTriangleMultiplicationCpp",
    "read_status",
]


@profile("dot_product_attention")
def dot_product_attention_cpp(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: torch.Tensor,
    bias: torch.Tensor,
    use_flash_attention: bool = False,
    BLK_SZ: int = 128,
    FLASH_SZ: int = 1024,
    *,
    q_scale: Optional[torch.Tensor] = None,
    k_scale: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Same positional signature as the reference (src/af3_kernels/__init__.py:31-40).

    ``use_flash_attention``, ``BLK_SZ`` and ``FLASH_SZ`` are accepted and checked but do not
    select code: the CUDA kernel always runs an online softmax over 128-key tiles.  Unlike the
    reference the call never writes to ``q`` and a 1-D mask broadcasts over the batch.
    ``q_scale`` / ``k_scale`` (keyword-only) enable float8_e4m3fn q and k.  CUDA tensors are
    computed in place on their device; host tensors (what the reference takes) go through
    ``dot_product_attention_host`` and come back as a host tensor.
    """
    if int(BLK_SZ) <= 0 or int(FLASH_SZ) <= 0:
        raise ValueError("BLK_SZ and FLASH_SZ must be positive")
    if not q.is_cuda:
        # host tensors, as the reference takes them: pipelined over PCIe, computed on the GPU,
        # result in host memory
        return dot_product_attention_host(q, k, v, mask, bias, q_scale=q_scale, k_scale=k_scale)
    return dot_product_attention(q, k, v, mask, bias, q_scale=q_scale, k_scale=k_scale)


def _not_built(name: str):
    raise NotImplementedError(
        f"{name} is outside the attention hot path this package implements on B200"
    )


def gated_linear_unit_cpp(x, weight, vnni_repacked=False, M_BLK=128, N_BLK=128):
    _not_built("gated_linear_unit_cpp")


def _attention_cpp(
    pair: torch.Tensor,
    mask: torch.Tensor,
    bias: torch.Tensor,
    q_proj: torch.Tensor,
    k_proj: torch.Tensor,
    v_proj: torch.Tensor,
    gating_query: torch.Tensor,
    out_proj: torch.Tensor,
    head: int,
    use_flash_attention: bool = False,  # unused, as in the reference
    BLK_SZ: int = 128,
    FLASH_SZ: int = 1024,  # unused, as in the reference
) -> torch.Tensor:
    """Grid / triangle self-attention block, same signature as the reference
    (src/af3_kernels/__init__.py:55-80): q/k/v/gate projections, biased key-masked attention,
    sigmoid gating, output projection.  Weights are ``[in, out]`` (``linear.weight.T``)."""
    return attention_block(pair, mask, bias, q_proj, k_proj, v_proj, gating_query, out_proj, head)


def self_attention_cpp(
    pair: torch.Tensor,
    mask: torch.Tensor,
    bias: torch.Tensor,
    q_proj: torch.Tensor,
    q_bias: torch.Tensor,
    k_proj: torch.Tensor,
    v_proj: torch.Tensor,
    gating_query: torch.Tensor,
    head: int,
    use_flash_attention: bool = False,  # unused, as in the reference
    BLK_SZ: int = 128,
    FLASH_SZ: int = 1024,  # unused, as in the reference
) -> torch.Tensor:
    """Single / diffusion attention block over one token sequence, same signature as the
    reference (src/af3_kernels/__init__.py:83-105): ``pair`` is ``x [N, C]``, ``mask [N]``."""
    return self_attention_block(pair, mask, bias, q_proj, q_bias, k_proj, v_proj, gating_query, head)


def pad_and_align_tensor(x: torch.Tensor, shape, need_init: bool = True, init: float = 0.0,
                         alignment: int = 64) -> torch.Tensor:
    """Device-side stand-in for the reference helper (src/csrc/tools.cpp:42-124): returns ``x``
    itself when it already has ``shape`` and is contiguous, else a new tensor of ``shape`` holding
    ``x`` in its leading corner and ``init`` elsewhere.  The kernel needs no padding (TMA
    zero-fills out-of-range tiles); this exists for callers that used the helper directly."""
    shape = tuple(int(s) for s in shape)
    if tuple(x.shape) == shape and x.is_contiguous():
        return x
    if len(shape) != x.dim() or any(a > b for a, b in zip(x.shape, shape)):
        raise ValueError(f"cannot pad {tuple(x.shape)} to {shape}")
    out = torch.full(shape, init, dtype=x.dtype, device=x.device) if need_init else \
        torch.empty(shape, dtype=x.dtype, device=x.device)
    out[tuple(slice(0, s) for s in x.shape)] = x
    return out


def vnni_repack_tensor(x: torch.Tensor, type: int = 2, BLK_SZ: int = 0) -> torch.Tensor:
    """The reference re-orders a weight into the VNNI layout of its CPU GEMM
    (src/csrc/tools.cpp:151-176).  No such layout exists on the GPU (TMA swizzled tiles and cuBLAS
    take the plain matrix), so the weight is returned unchanged; callers that repack before
    ``_attention_cpp`` / ``self_attention_cpp`` keep working."""
    return x


def reset_debug_timers():
    """The reference resets its per-thread rdtsc timers (src/csrc/init.cpp:102-143); here the
    per-operator CUDA-event totals gathered by the ``profile`` wrapper are cleared."""
    tools.reset_op_timers()


def print_debug_timers(tid=0, detailed=True):
    """Prints per-operator call counts and device milliseconds (CUDA events around every wrapped
    operator; gathered when DO_PROFILE=1 or AF3K_TIMERS=1).  The reference prints per-TPP-category
    CPU-thread timers (src/csrc/init.cpp:145-216); ``tid`` selects a CPU thread there and is
    ignored here."""
    totals = tools.op_timer_totals()
    if not totals:
        print("af3k timers: nothing recorded (set DO_PROFILE=1 or AF3K_TIMERS=1 before importing)")
        return
    print(f"{'operator':<32}{'calls':>8}{'total ms':>12}{'ms/call':>12}")
    for name, (calls, ms) in sorted(totals.items()):
        print(f"{name:<32}{calls:>8}{ms:>12.3f}{(ms / calls if calls else 0.0):>12.4f}")


def print_debug_thread_imbalance():
    """The reference prints the spread of its OpenMP threads' timers (src/csrc/init.cpp:218-309).
    A kernel launch has no host threads to compare; the per-operator table is printed instead."""
    print_debug_timers()


class Linear(torch.nn.Module):
    """Bias-free linear layer with the reference's constructor (src/af3_kernels/__init__.py:138-165).
    Outside the attention hot path: a plain cuBLAS GEMM on the tensor's device, no VNNI repack."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 M_BLK: int = 128, N_BLK: int = 128) -> None:
        super().__init__()
        assert bias is False
        self.in_features = in_features
        self.out_features = out_features
        self.weight = torch.nn.Parameter(torch.empty((out_features, in_features), device=device, dtype=dtype))
        self.register_parameter("bias", None)
        self.M_BLK = M_BLK
        self.N_BLK = N_BLK

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(input, self.weight)


class TriangleMultiplicationCpp(torch.nn.Module):
    """Importable for code that names it (src/af3_kernels/TriangleMultiplication.py:22-76); the
    triangle multiplication is a different operator from the attention path built here."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__()
        _not_built("TriangleMultiplicationCpp")


class DistributedTriangleMultiplicationCpp(torch.nn.Module):
    """See TriangleMultiplicationCpp (src/af3_kernels/TriangleMultiplication.py:79-192)."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__()
        _not_built("DistributedTriangleMultiplicationCpp")
