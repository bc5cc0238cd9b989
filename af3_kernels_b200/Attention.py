"""Grid (triangle) self-attention modules with the reference's names, constructor arguments and
parameter names (src/af3_kernels/Attention.py), so that a checkpoint of the reference's modules
loads unchanged.  The forward passes run on CUDA through ``attention_block``.
"""
from __future__ import annotations

from math import ceil

import torch
import torch.distributed as dist
import torch.nn as nn

from . import pair_bias
from .fused_ops import attention_block, grid_block_from_raw_pair, pair_front_ok
from .tools import profile


class GridSelfAttentionCpp(nn.Module):
    """Reference: src/af3_kernels/Attention.py:23-82.  pair [N, N, c_pair], mask [N, N]."""

    def __init__(self, c_pair: int = 128, num_head: int = 4, transpose: bool = False):
        super().__init__()
        self.c_pair = c_pair
        self.num_head = num_head
        self.qkv_dim = self.c_pair // self.num_head
        self.transpose = transpose
        self.act_norm = nn.LayerNorm(self.c_pair)
        self.pair_bias_projection = nn.Linear(self.c_pair, self.num_head, bias=False)
        self.q_projection = nn.Linear(self.c_pair, self.c_pair, bias=False)
        self.k_projection = nn.Linear(self.c_pair, self.c_pair, bias=False)
        self.v_projection = nn.Linear(self.c_pair, self.c_pair, bias=False)
        self.gating_query = nn.Linear(self.c_pair, self.c_pair, bias=False)
        self.output_projection = nn.Linear(self.c_pair, self.c_pair, bias=False)

    # One pass over the raw pair for LayerNorm + pair bias + q/k/v/gate projections (af3k_pair_front).
    # Off by default: at N = 768 it takes 0.232 ms against 0.073 + 0.140 ms for the two kernels it
    # replaces - it saves the normalised pair's round trip through HBM, but only two tiles per SM are
    # being normalised at a time (against five CTAs of the stand-alone producer), and the row walks are
    # latency-bound.
    fused_front = False

    def _weights(self):
        # [in, out] views of the Linear weights: what the reference hands to its operator
        return (self.q_projection.weight.T, self.k_projection.weight.T, self.v_projection.weight.T,
                self.gating_query.weight.T, self.output_projection.weight.T)

    def _norm_and_bias(self, pair: torch.Tensor):
        # c_pair = 128: one fused pass (LayerNorm, bias projection, permute); other widths go
        # through PyTorch's LayerNorm and Linear on the same device
        if pair_bias.supported(pair, self.num_head):
            return pair_bias.layernorm_pair_bias(pair, self.act_norm.weight, self.act_norm.bias,
                                                 self.pair_bias_projection.weight, self.act_norm.eps)
        pair = self.act_norm(pair)
        bias = self.pair_bias_projection(pair).permute(2, 0, 1)     # [H, N, N]
        return pair, bias

    @profile("B200 GridSelfAttention")
    def forward(self, pair: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        dtype = pair.dtype
        if self.fused_front and not self.transpose and pair_front_ok(pair, self.num_head, self.num_head):
            # bf16 pair, c_pair = 128, up to four heads: LayerNorm, pair bias and the four projections
            # in one pass over the raw pair
            return grid_block_from_raw_pair(pair, mask, self.act_norm.weight, self.act_norm.bias, self.act_norm.eps,
                                            self.pair_bias_projection.weight, *self._weights(), self.num_head).to(dtype)
        pair, bias = self._norm_and_bias(pair)
        if self.transpose:
            pair = pair.permute(1, 0, 2)
        out = attention_block(pair, mask, bias, *self._weights(), self.num_head)
        if self.transpose:
            out = out.permute(1, 0, 2)
        return out.to(dtype)


class DistributedGridSelfAttentionCpp(GridSelfAttentionCpp):
    """Reference: src/af3_kernels/Attention.py:85-203.  Every rank holds the whole ``pair`` and
    computes the rows ``[rank * ceil(N / ws), (rank + 1) * ceil(N / ws))``; the bias is computed
    redundantly on every rank from the replicated pair, the mask is sliced by row, and the row
    blocks are exchanged in ``COMM_SPLIT`` pieces.  The reference overlaps gather *i* with the
    compute of piece *i + 1* from a helper thread; here the exchange runs on side CUDA streams
    (``RowShardedAttention.gather_rows``: peer copies into symmetric memory, or NCCL)."""

    def __init__(self, c_pair: int = 128, num_head: int = 4, transpose: bool = False):
        super().__init__(c_pair, num_head, transpose)
        self._sharder = None

    @profile("B200 Distributed GridSelfAttention")
    def forward(self, pair: torch.Tensor, mask: torch.Tensor, COMM_SPLIT: int = 4) -> torch.Tensor:
        from .distributed import RowShardedAttention
        rk, ws = dist.get_rank(), dist.get_world_size()
        dtype = pair.dtype
        seq_len = pair.shape[0]
        split_size = ceil(seq_len / ws)
        rows = slice(split_size * rk, split_size * (rk + 1))
        local_mask = mask[rows]

        pair, bias = self._norm_and_bias(pair)
        bias = bias.contiguous()
        if self.transpose:
            pair = pair.permute(1, 0, 2)
        chunk = pair[rows]
        if self._sharder is None:
            self._sharder = RowShardedAttention()
        self._sharder.comm_split = COMM_SPLIT
        weights = self._weights()

        def compute(lo, hi, slot, kw):
            # this rank's piece goes straight into its slot of the result; the other ranks' pieces
            # arrive in place while the next piece is computed (RowShardedAttention.gather_rows)
            slot.copy_(attention_block(chunk[lo:hi], local_mask[lo:hi], bias, *weights, self.num_head))

        out = self._sharder.gather_rows(seq_len, tuple(pair.shape[1:]), pair.dtype, pair.device, compute)
        if self.transpose:
            out = out.permute(1, 0, 2)
        return out.contiguous().to(dtype)
