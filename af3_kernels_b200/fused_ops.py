"""The two attention blocks that wrap the core operator in the reference.

* ``attention_block`` stands in for ``_C._attention`` (src/csrc/dot_product_attention.cpp:200-378,
  wrapper src/af3_kernels/__init__.py:55-80): grid / triangle self-attention over the rows of the
  pair representation - q, k, v and gate projections, the biased key-masked core, sigmoid gating
  and the output projection.
* ``self_attention_block`` stands in for ``_C.self_attention`` (:380-543, wrapper :83-105): single /
  diffusion attention over one token sequence with a query bias and gating, no output projection.

The projections are plain GEMMs and go through torch (cuBLAS); the core is the hand-written kernel
behind ``libaf3k.so``.  q, k and v are never rearranged in memory: the ``[.., N, H*D]`` projection
outputs are handed to the kernel as strided ``[.., H, N, D]`` views, and the kernel writes its
result straight into the ``[.., N, H*D]`` layout the gating needs.

Weights are taken the way the reference passes them: ``[in_features, out_features]``
(``linear.weight.T.contiguous()``; the reference additionally VNNI-repacks them for its CPU GEMM,
which has no meaning here - ``vnni_repack_tensor`` returns its input unchanged).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _capi
from .dpa import dot_product_attention


def _as_bf16(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)


def sigmoid_gate(weighted: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """weighted * sigmoid(gate) for two bf16 CUDA tensors of the same shape, in one pass
    (``af3k_sigmoid_gate``; reference: the SigmoidFwdTPP + MulTPP pair behind the core,
    src/csrc/dot_product_attention.cpp:339-345).  Shapes the kernel does not take (element count
    not a multiple of 8, non-contiguous) go through torch."""
    n = weighted.numel()
    if (weighted.dtype != torch.bfloat16 or gate.dtype != torch.bfloat16 or n % 8 != 0 or n == 0
            or not weighted.is_contiguous() or not gate.is_contiguous()
            or weighted.data_ptr() % 16 != 0 or gate.data_ptr() % 16 != 0):
        return weighted * torch.sigmoid(gate)
    out = torch.empty_like(weighted)
    with torch.cuda.device(weighted.device):
        _capi.check(_capi.load().af3k_sigmoid_gate(weighted.data_ptr(), gate.data_ptr(), out.data_ptr(), n,
                                                   torch.cuda.current_stream().cuda_stream))
    return out


def attention_block(
    pair: torch.Tensor,
    mask: torch.Tensor,
    bias: torch.Tensor,
    q_proj: torch.Tensor,
    k_proj: torch.Tensor,
    v_proj: torch.Tensor,
    gating_query: torch.Tensor,
    out_proj: torch.Tensor,
    head: int,
) -> torch.Tensor:
    """pair [R, N, C] (already layer-normed); mask [R, N] or [N], True = attend; bias [head, N, N];
    all weights [C, C] as [in, out].  Returns [R, N, C] in ``pair.dtype``."""
    if pair.dim() != 3:
        raise ValueError("pair must be [rows, N, c_pair]")
    if not pair.is_cuda:
        raise RuntimeError("af3_kernels_b200 runs on CUDA tensors only (no CPU fallback)")
    R, N, C = pair.shape
    if C % head != 0:
        raise ValueError("c_pair must be divisible by the number of heads")
    D = C // head
    x = _as_bf16(pair)
    q = torch.matmul(x, _as_bf16(q_proj)).view(R, N, head, D).permute(0, 2, 1, 3)
    k = torch.matmul(x, _as_bf16(k_proj)).view(R, N, head, D).permute(0, 2, 1, 3)
    v = torch.matmul(x, _as_bf16(v_proj)).view(R, N, head, D).permute(0, 2, 1, 3)
    weighted = torch.empty((R, N, head, D), dtype=torch.bfloat16, device=pair.device)
    dot_product_attention(q, k, v, mask, bias, out=weighted.permute(0, 2, 1, 3))
    gated = sigmoid_gate(weighted.view(R, N, C), torch.matmul(x, _as_bf16(gating_query)))
    return torch.matmul(gated, _as_bf16(out_proj)).to(pair.dtype)


def self_attention_block(
    x: torch.Tensor,
    mask: Optional[torch.Tensor],
    bias: torch.Tensor,
    q_proj: torch.Tensor,
    q_bias: torch.Tensor,
    k_proj: torch.Tensor,
    v_proj: torch.Tensor,
    gating_query: torch.Tensor,
    head: int,
) -> torch.Tensor:
    """x [N, C]; mask [N], True = attend; bias [head, N, N]; weights [C, C] as [in, out]; q_bias
    [C] (or [head, D]).  Returns [N, C] in ``x.dtype``."""
    if x.dim() != 2:
        raise ValueError("x must be [num_tokens, channels]")
    if not x.is_cuda:
        raise RuntimeError("af3_kernels_b200 runs on CUDA tensors only (no CPU fallback)")
    N, C = x.shape
    if C % head != 0:
        raise ValueError("channels must be divisible by the number of heads")
    D = C // head
    xb = _as_bf16(x)
    q = (torch.matmul(xb, _as_bf16(q_proj)) + _as_bf16(q_bias).reshape(C)).view(1, N, head, D).permute(0, 2, 1, 3)
    k = torch.matmul(xb, _as_bf16(k_proj)).view(1, N, head, D).permute(0, 2, 1, 3)
    v = torch.matmul(xb, _as_bf16(v_proj)).view(1, N, head, D).permute(0, 2, 1, 3)
    weighted = torch.empty((1, N, head, D), dtype=torch.bfloat16, device=x.device)
    m = None if mask is None else mask.reshape(-1)
    dot_product_attention(q, k, v, m, bias, out=weighted.permute(0, 2, 1, 3))
    return sigmoid_gate(weighted.view(N, C), torch.matmul(xb, _as_bf16(gating_query))).to(x.dtype)
