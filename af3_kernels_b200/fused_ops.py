"""The two attention blocks that wrap the core operator in the reference.

* ``attention_block`` stands in for ``_C._attention`` (src/csrc/dot_product_attention.cpp:200-378,
  wrapper src/af3_kernels/__init__.py:55-80): grid / triangle self-attention over the rows of the
  pair representation - q, k, v and gate projections, the biased key-masked core, sigmoid gating
  and the output projection.
* ``self_attention_block`` stands in for ``_C.self_attention`` (:380-543, wrapper :83-105): single /
  diffusion attention over one token sequence with a query bias and gating, no output projection.

For the grid block at c_pair = 128 the four input projections are one hand-written pass over the
pair (``af3k_qkvg_projection``: q, k, v leave head-major and q pre-scaled); the output projection
is a plain GEMM through torch (cuBLAS), as are all projections of other widths, whose
``[.., N, H*D]`` outputs are handed to the attention kernel as strided ``[.., H, N, D]`` views.  The
kernel writes its result straight into the ``[.., N, H*D]`` layout the gating needs.

Weights are taken the way the reference passes them: ``[in_features, out_features]``
(``linear.weight.T.contiguous()``; the reference additionally VNNI-repacks them for its CPU GEMM,
which has no meaning here - ``vnni_repack_tensor`` returns its input unchanged).
"""
from __future__ import annotations

from typing import Optional

import torch

import ctypes

from . import _capi
from .dpa import _status_buffer, dot_product_attention


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


_w4_cache: dict = {}


def _stacked_projection_weights(q_proj, k_proj, v_proj, gating_query) -> torch.Tensor:
    """[512, 128] bf16: the four [in, out] projection weights as stacked [out, in] rows (q, k, v,
    gate), which is the K-major B operand the projection kernel reads.  Built once per set of
    weight tensors (keyed by their storage and version)."""
    key = tuple((w.data_ptr(), w._version, w.dtype, tuple(w.stride())) for w in (q_proj, k_proj, v_proj, gating_query))
    w4 = _w4_cache.get(key)
    if w4 is None:
        if len(_w4_cache) >= 16:
            _w4_cache.clear()
        w4 = torch.cat([_as_bf16(w.detach()).t() for w in (q_proj, k_proj, v_proj, gating_query)], dim=0).contiguous()
        _w4_cache[key] = w4
    return w4


def qkvg_projection(x: torch.Tensor, w4: torch.Tensor, head: int, q_scale: float):
    """x [R, N, 128] bf16 contiguous, w4 [512, 128] bf16 -> (q, k, v [R, head, N, 128 / head], gate
    [R, N, 128]), all bf16, q pre-multiplied by ``q_scale`` (``af3k_qkvg_projection``)."""
    R, N, C = x.shape
    D = C // head
    q = torch.empty((R, head, N, D), dtype=torch.bfloat16, device=x.device)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    g = torch.empty((R, N, C), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _capi.check(_capi.load().af3k_qkvg_projection(
            x.data_ptr(), w4.data_ptr(), R, N, head, ctypes.c_float(q_scale), q.data_ptr(), k.data_ptr(),
            v.data_ptr(), g.data_ptr(), _status_buffer(x.device).data_ptr(), torch.cuda.current_stream().cuda_stream))
    return q, k, v, g


def _fused_projection_ok(x: torch.Tensor, head: int) -> bool:
    C = x.shape[-1]
    return (C == 128 and C % head == 0 and (C // head) % 8 == 0 and x.dtype == torch.bfloat16
            and x.is_contiguous() and x.data_ptr() % 16 == 0 and x.numel() > 0)


def pair_front(pair: torch.Tensor, ln_weight: torch.Tensor, ln_bias: torch.Tensor, eps: float,
               bias_weight: torch.Tensor, w4: torch.Tensor, head: int, q_scale: float):
    """The whole front of the grid block in one pass over the RAW pair [R, N, 128] bf16
    (``af3k_pair_front``): LayerNorm, the pair-bias projection + permute, and the q / k / v / gate
    projections.  Returns (bias [Hb, R, N] bf16 view with 16-byte aligned rows, q, k, v
    [R, head, N, 128 / head], gate [R, N, 128]); the normalised pair itself never reaches HBM."""
    R, N, C = pair.shape
    D = C // head
    dev = pair.device
    Hb = bias_weight.shape[0]
    gamma = ln_weight.detach().to(device=dev, dtype=torch.float32).contiguous()
    beta = ln_bias.detach().to(device=dev, dtype=torch.float32).contiguous()
    bw = bias_weight.detach().to(device=dev, dtype=torch.float32).contiguous()
    pitch = (N + 7) // 8 * 8
    bias = torch.empty((Hb, R, pitch), dtype=torch.bfloat16, device=dev)
    q = torch.empty((R, head, N, D), dtype=torch.bfloat16, device=dev)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    g = torch.empty((R, N, C), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _capi.check(_capi.load().af3k_pair_front(
            pair.data_ptr(), gamma.data_ptr(), beta.data_ptr(), ctypes.c_float(eps), bw.data_ptr(), Hb,
            w4.data_ptr(), R, N, head, ctypes.c_float(q_scale), bias.data_ptr(), pitch, q.data_ptr(), k.data_ptr(),
            v.data_ptr(), g.data_ptr(), _status_buffer(dev).data_ptr(), torch.cuda.current_stream().cuda_stream))
    return bias[:, :, :N], q, k, v, g


def pair_front_ok(pair: torch.Tensor, head: int, bias_heads: int) -> bool:
    return pair.is_cuda and pair.dim() == 3 and _fused_projection_ok(pair, head) and 1 <= bias_heads <= 4


def grid_block_from_raw_pair(pair, mask, ln_weight, ln_bias, eps, bias_weight, q_proj, k_proj, v_proj,
                             gating_query, out_proj, head: int) -> torch.Tensor:
    """LayerNorm + pair bias + ``attention_block`` for a raw bf16 pair [R, N, 128]: the fused front,
    the attention core, the sigmoid gate and the output projection."""
    R, N, C = pair.shape
    D = C // head
    w4 = _stacked_projection_weights(q_proj, k_proj, v_proj, gating_query)
    bias, q, k, v, gate = pair_front(pair, ln_weight, ln_bias, eps, bias_weight, w4, head, D ** -0.5)
    weighted = torch.empty((R, N, head, D), dtype=torch.bfloat16, device=pair.device)
    dot_product_attention(q, k, v, mask, bias, softmax_scale=1.0, out=weighted.permute(0, 2, 1, 3))
    gated = sigmoid_gate(weighted.view(R, N, C), gate)
    return torch.matmul(gated, _as_bf16(out_proj))


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
    if _fused_projection_ok(x, head):
        # c_pair = 128: one pass over x for all four projections; q, k, v leave head-major with q
        # already scaled, so the attention core reads unit-stride rows and scales nothing
        w4 = _stacked_projection_weights(q_proj, k_proj, v_proj, gating_query)
        q, k, v, gate = qkvg_projection(x, w4, head, D ** -0.5)
        weighted = torch.empty((R, N, head, D), dtype=torch.bfloat16, device=pair.device)
        dot_product_attention(q, k, v, mask, bias, softmax_scale=1.0, out=weighted.permute(0, 2, 1, 3))
        gated = sigmoid_gate(weighted.view(R, N, C), gate)
        return torch.matmul(gated, _as_bf16(out_proj)).to(pair.dtype)
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
