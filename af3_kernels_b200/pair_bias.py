"""Pair-bias producer: LayerNorm over the channels of the pair representation, the per-head bias
projection and the permute to ``[H, N, N]`` in one pass over the pair (``af3k_pair_bias``).

Stands in for the two statements in front of the attention core in the reference's modules
(src/af3_kernels/Attention.py:51-52 and :152-153)::

    pair = self.act_norm(pair)
    bias = self.pair_bias_projection(pair).permute(2, 0, 1)
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import _capi

CHANNELS = 128
MAX_HEADS = 16


def supported(pair: torch.Tensor, num_head: int) -> bool:
    """The fused kernel covers c_pair = 128 (AlphaFold3's pair width) and up to 16 heads."""
    return pair.is_cuda and pair.dim() == 3 and pair.shape[-1] == CHANNELS and 1 <= num_head <= MAX_HEADS


def layernorm_pair_bias(
    pair: torch.Tensor,
    ln_weight: torch.Tensor,
    ln_bias: torch.Tensor,
    proj_weight: torch.Tensor,
    eps: float = 1e-5,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """pair [R, N, 128] (bf16 or fp32, CUDA); ln_weight / ln_bias [128]; proj_weight [H, 128]
    (``nn.Linear.weight``).  Returns (normalised pair [R, N, 128] bf16, bias [H, R, N] bf16); the
    bias is a view with 16-byte aligned rows, which the attention kernel reads in place."""
    if not pair.is_cuda:
        raise RuntimeError("af3_kernels_b200 runs on CUDA tensors only (no CPU fallback)")
    if pair.dim() != 3 or pair.shape[-1] != CHANNELS:
        raise ValueError(f"pair must be [R, N, {CHANNELS}]")
    H = proj_weight.shape[0]
    if proj_weight.shape != (H, CHANNELS) or not 1 <= H <= MAX_HEADS:
        raise ValueError(f"proj_weight must be [H, {CHANNELS}] with 1 <= H <= {MAX_HEADS}")
    if pair.dtype not in (torch.bfloat16, torch.float32):
        pair = pair.to(torch.float32)
    pair = pair.contiguous()
    R, N, C = pair.shape
    dev = pair.device
    gamma = ln_weight.detach().to(device=dev, dtype=torch.float32).contiguous()
    beta = ln_bias.detach().to(device=dev, dtype=torch.float32).contiguous()
    proj = proj_weight.detach().to(device=dev, dtype=torch.float32).contiguous()
    normed = torch.empty((R, N, C), dtype=torch.bfloat16, device=dev)
    pitch = (N + 7) // 8 * 8
    bias = torch.empty((H, R, pitch), dtype=torch.bfloat16, device=dev)
    lib = _capi.load()
    with torch.cuda.device(dev):
        code = lib.af3k_pair_bias(
            pair.data_ptr(),
            _capi.AF3K_BF16 if pair.dtype == torch.bfloat16 else _capi.AF3K_F32,
            R, N, C, H,
            gamma.data_ptr(), beta.data_ptr(), proj.data_ptr(), ctypes.c_float(eps),
            normed.data_ptr(), bias.data_ptr(), pitch,
            torch.cuda.current_stream().cuda_stream,
        )
    _capi.check(code)
    return normed, bias[:, :, :N]
