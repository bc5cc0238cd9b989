"""Row-sharded attention over the GPUs of one node.

Every (pair row, head) is an independent attention problem, so the rows of the pair
representation are split into contiguous blocks, one per rank, exactly as the reference's
``DistributedGridSelfAttentionCpp`` does (src/af3_kernels/Attention.py:145-156): rank ``r`` owns
rows ``[r * ceil(rows / ws), (r + 1) * ceil(rows / ws))``; the bias is replicated and the mask is
sliced by row.  No collective sits on the data path of the kernel.  The optional gather of the
output is cut into ``comm_split`` pieces and issued on a side stream, so the exchange of piece
``i`` overlaps the kernel of piece ``i + 1`` (the reference does this with a helper thread and a
queue around ``dist.all_gather``, Attention.py:162-195).
"""
from __future__ import annotations

import time
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from .tools import pad_to_size, record_comm_time


def row_partition(rows: int, world_size: int, rank: int) -> Tuple[int, int, int]:
    """-> (begin, end, split_size): the row block of ``rank`` and the padded block size."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad world_size / rank")
    split = (rows + world_size - 1) // world_size
    begin = min(rows, split * rank)
    end = min(rows, begin + split)
    return begin, end, split


class RowShardedAttention:
    """Shards ``dot_product_attention`` by pair row over a process group.

    ``attention_fn(q, k, v, mask, bias) -> out`` defaults to the CUDA operator; tests running on
    CPU ranks (gloo) pass a stand-in so that the partition / gather logic is exercised without a GPU.
    """

    def __init__(self, group=None, comm_split: int = 8, attention_fn: Optional[Callable] = None,
                 comm_sms: int = 8):
        if comm_split < 1:
            raise ValueError("comm_split must be >= 1")
        self.group = group
        self.comm_split = comm_split
        # The attention kernel is persistent, one CTA per SM, each taking the SM's whole shared
        # memory and TMEM: a collective launched beside it finds no SM until it ends, and the
        # gather of piece i then runs after kernel i + 1 instead of under it.  So the kernels of a
        # gathered forward leave `comm_sms` SMs free (0 = use all).  Measured on two GPUs (2 048 rows of
        # N = 2 048, fp8 q/k): 7.17 ms with every SM and four pieces, 6.97 ms with eight SMs left free
        # and eight pieces; capping NCCL's own CTAs (NCCL_MAX_CTAS) only made the transfers slower.
        self.comm_sms = comm_sms
        # How the pieces travel on CUDA ranks: "copy" (peer-to-peer copies into the peers' result buffers,
        # which live in symmetric memory: copy engines move the data, no SM is taken from the attention
        # kernel), "sendrecv" (grouped NCCL point-to-point, in place), "broadcast" (one per rank, in
        # place), "allgather" (one collective into a staging buffer + a copy); "auto" = "copy" where
        # symmetric memory can be set up, else "sendrecv".
        self.exchange = "auto"
        self.copy_streams = 0           # streams the peer copies of a piece are spread over (0 = one per peer:
                                        # on 8 GPUs 2.67 ms per forward against 3.06 with four and 3.62 with two)
        self._symm = {}
        self._copy_streams = None
        self.last_exchange = None       # what the last forward used
        self.symm_error = None          # why symmetric memory could not be set up, if it could not
        # the CUDA operator writes into a caller-provided ``out``; a stand-in (CPU tests) returns its result
        self.writes_in_place = attention_fn is None
        if attention_fn is None:
            from .dpa import dot_product_attention as attention_fn
        self.attention_fn = attention_fn
        self._comm_stream = None

    # ------------------------------------------------------------------ helpers
    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group)

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group)

    def broadcast_shared(self, bias: torch.Tensor, mask: Optional[torch.Tensor], src: int = 0):
        """Broadcasts the replicated operands (bias, full mask) once from ``src`` into each
        rank's own memory.  Returns the work handles' results already waited on."""
        dist.broadcast(bias, src=src, group=self.group)
        if mask is not None:
            m = mask.view(torch.uint8) if mask.dtype == torch.bool else mask
            dist.broadcast(m, src=src, group=self.group)
        return bias, mask

    def shard(self, full: torch.Tensor, rows: int) -> torch.Tensor:
        """This rank's contiguous row block of a tensor whose first dimension is the pair row."""
        b, e, _ = row_partition(rows, self.world_size, self.rank)
        return full[b:e]

    def _symmetric_result(self, shape, dtype, device):
        """One of two result buffers in symmetric memory (alternating per call, so that a result stays
        valid until the call after the next starts) with the peers' views of it, or None when
        symmetric memory is not available."""
        key = (tuple(shape), dtype, device.index)
        ent = self._symm.get(key)
        if ent is None:
            try:
                import torch.distributed._symmetric_memory as symm_mem
                group = self.group if self.group is not None else dist.group.WORLD
                bufs = []
                for _ in range(2):
                    t = symm_mem.empty(shape, dtype=dtype, device=device)
                    hdl = symm_mem.rendezvous(t, group)
                    peers = [t if r == self.rank else hdl.get_buffer(r, shape, dtype) for r in range(self.world_size)]
                    bufs.append((t, hdl, peers))
                ent = {"bufs": bufs, "turn": 0}
            except Exception as exc:    # no symmetric memory on this system / build: NCCL carries the pieces
                self.symm_error = f"{type(exc).__name__}: {exc}"
                ent = {"bufs": None, "turn": 0}
            # two result shapes are kept (each costs two full-size buffers); an older one is dropped
            while len(self._symm) >= 2:
                self._symm.pop(next(iter(self._symm)))
            self._symm[key] = ent
        if ent["bufs"] is None:
            return None
        ent["turn"] ^= 1
        return ent["bufs"][ent["turn"]]

    # ------------------------------------------------------------------ compute
    def forward_local(self, q, k, v, mask, bias) -> torch.Tensor:
        """Attention over this rank's rows only; the output stays row-sharded."""
        return self.attention_fn(q, k, v, mask, bias)

    def forward(self, q, k, v, mask, bias, rows: int, timeout_s: float = 60.0) -> torch.Tensor:
        """q, k, v, mask: this rank's row block (``shard`` of the full tensors).  Returns the
        full ``[rows, H, N, D]`` output on every rank (see ``gather_rows`` for how the pieces travel
        and how long the result stays valid)."""
        ws, rank = self.world_size, self.rank
        b, e, split = row_partition(rows, ws, rank)
        local_rows = e - b
        if q.shape[0] != local_rows:
            raise ValueError(f"rank {rank} expected {local_rows} local rows, got {q.shape[0]}")
        _, H, N, D = q.shape
        out_dtype = torch.bfloat16 if q.is_cuda else q.dtype

        def compute(lo, hi, slot, kw):
            m = None
            if mask is not None:
                m = mask[lo:hi] if mask.dim() >= 2 and mask.shape[0] == local_rows else mask
            if self.writes_in_place:
                self.attention_fn(q[lo:hi], k[lo:hi], v[lo:hi], m, bias, out=slot, **kw)
            else:
                slot.copy_(self.attention_fn(q[lo:hi], k[lo:hi], v[lo:hi], m, bias))

        return self.gather_rows(rows, (H, N, D), out_dtype, q.device, compute, timeout_s)

    def gather_rows(self, rows: int, tail, dtype, device, compute, timeout_s: float = 60.0) -> torch.Tensor:
        """Runs ``compute(lo, hi, slot, kw)`` for the pieces ``[lo, hi)`` of this rank's row block -
        it must fill ``slot`` (``[hi - lo, *tail]``), passing ``kw`` on to the attention operator - and
        returns the full ``[rows, *tail]`` result on every rank.

        The result buffer is laid out ``[rank, row in block, *tail]``, which is the row order of the
        full problem, so every rank computes each piece of its block straight into its own slot and
        the pieces of the other ranks arrive in place while the next piece is computed.  Nothing is
        copied after the exchange.  With ``exchange`` "copy" (the default where symmetric memory
        works) the result is a view of one of two buffers that alternate per call: it stays valid
        until the call after the next one."""
        ws, rank = self.world_size, self.rank
        b, e, split = row_partition(rows, ws, rank)
        local_rows = e - b
        tail = tuple(tail)
        on_gpu = device.type == "cuda"
        piece = (split + self.comm_split - 1) // self.comm_split
        exchange = self.exchange
        symm = None
        if on_gpu and ws > 1 and exchange in ("auto", "copy"):
            symm = self._symmetric_result((ws, split) + tail, dtype, device)
            if symm is None and exchange == "copy":
                raise RuntimeError("exchange='copy' needs symmetric memory, which could not be set up")
        if exchange == "auto":
            exchange = "copy" if symm is not None else "sendrecv"
        self.last_exchange = exchange
        if exchange == "copy":
            full, hdl, peer_full = symm
            # nobody may still be writing into (or, two calls back, reading from) this buffer
            hdl.barrier(channel=0)
            n_cs = self.copy_streams if self.copy_streams > 0 else max(1, ws - 1)
            if self._copy_streams is None or len(self._copy_streams) != n_cs:
                self._copy_streams = [torch.cuda.Stream(device=device) for _ in range(n_cs)]
        else:
            full = torch.empty((ws, split) + tail, dtype=dtype, device=device)
        if local_rows < split:
            full[rank, local_rows:].zero_()        # the padded tail of a ragged split, dropped at the end
        roots = [dist.get_global_rank(self.group, r) if self.group is not None else r for r in range(ws)]

        use_streams = on_gpu
        if use_streams and self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=device)
        kw = {}
        if on_gpu and ws > 1 and self.comm_sms > 0 and exchange != "copy":
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            kw["max_ctas"] = max(1, sms - self.comm_sms)
        works = []
        t0 = time.time()
        for p0 in range(0, split, piece):
            p1 = min(split, p0 + piece)
            lo, hi = min(p0, local_rows), min(p1, local_rows)
            if hi > lo:
                compute(lo, hi, full[rank, lo:hi], kw)
            if use_streams and exchange == "copy":
                # this rank's piece into every peer's buffer, one stream per peer so that several
                # copy engines work at once.  Every rank starts with its right-hand neighbour: with
                # all ranks going through the peers in the same order, everybody's first copy lands
                # on the same GPU (measured on 8 GPUs, copies alone: 204 GB/s out of every GPU
                # against 700 GB/s in this order).
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(device))
                for kk in range(1, ws):
                    if p1 > p0:
                        r = (rank + kk) % ws
                        cs = self._copy_streams[(kk - 1) % len(self._copy_streams)]
                        cs.wait_event(ev)
                        with torch.cuda.stream(cs):
                            peer_full[r][rank, p0:p1].copy_(full[rank, p0:p1], non_blocking=True)
            elif use_streams:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(device))
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ev)
                    if exchange == "sendrecv":
                        # one grouped launch per piece: this rank's slot goes to every peer while
                        # theirs arrive, both directions of every link busy at once
                        ops = []
                        for r in range(ws):
                            if r != rank:
                                ops.append(dist.P2POp(dist.isend, full[rank, p0:p1], roots[r], group=self.group))
                                ops.append(dist.P2POp(dist.irecv, full[r, p0:p1], roots[r], group=self.group))
                        if ops:
                            for w in dist.batch_isend_irecv(ops):
                                w.wait()       # orders the comm stream behind the transfer; the host does not block
                    elif exchange == "allgather":
                        # one collective per piece into a staging buffer, then one strided copy into place
                        tmp = torch.empty((ws, p1 - p0) + tail, dtype=dtype, device=device)
                        dist.all_gather_into_tensor(tmp, full[rank, p0:p1].contiguous(), group=self.group)
                        full[:, p0:p1].copy_(tmp)
                        tmp.record_stream(self._comm_stream)
                    else:
                        for r in range(ws):
                            dist.broadcast(full[r, p0:p1], src=roots[r], group=self.group)
            else:
                for r in range(ws):
                    works.append(dist.broadcast(full[r, p0:p1], src=roots[r], group=self.group, async_op=True))
        for w in works:
            if not w.wait(timeout=_timedelta(timeout_s)):
                raise RuntimeError("broadcast of an output piece did not complete")
        if use_streams and exchange == "copy":
            # every rank's copies are behind it when it reaches the barrier, so past the barrier every
            # rank's buffer is complete
            cur = torch.cuda.current_stream(device)
            for cs in self._copy_streams:
                cur.wait_stream(cs)
            hdl.barrier(channel=1)
        elif use_streams:
            torch.cuda.current_stream(device).wait_stream(self._comm_stream)
            full.record_stream(self._comm_stream)
        record_comm_time("AG Attn", time.time() - t0, full.numel() * full.element_size())
        return full.view((ws * split,) + tail)[:rows]


def _timedelta(seconds: float):
    import datetime

    return datetime.timedelta(seconds=seconds)
