"""world_size-2 gloo runs of the row-sharded path on CPU ranks.  The attention function is
replaced by the CPU oracle so that only the partition / gather logic is under test."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_fn(q, k, v, mask, bias):
    from oracle.attention_oracle import oracle_fp32
    return oracle_fp32(q, k, v, mask, bias).to(q.dtype)


def _worker(rank, ws, port, rows, comm_split, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=60))
    try:
        from af3_kernels_b200.distributed import RowShardedAttention
        g = torch.Generator().manual_seed(7)
        H, N, D = 2, 24, 8
        q = torch.randn(rows, H, N, D, generator=g)
        k = torch.randn(rows, H, N, D, generator=g)
        v = torch.randn(rows, H, N, D, generator=g)
        bias = torch.randn(H, N, N, generator=g)
        mask = torch.rand(rows, N, generator=g) >= 0.2
        op = RowShardedAttention(comm_split=comm_split, attention_fn=_oracle_fn)
        # replicated operands start zeroed on rank 1 and arrive by broadcast
        if rank != 0:
            bias = torch.zeros_like(bias)
        mask_u8 = mask.view(torch.uint8).clone()
        if rank != 0:
            mask_u8.zero_()
        op.broadcast_shared(bias, mask_u8)
        mask_b = mask_u8.view(torch.bool)
        full = op.forward(op.shard(q, rows), op.shard(k, rows), op.shard(v, rows),
                          op.shard(mask_b, rows), bias, rows)
        single = _oracle_fn(q, k, v, mask, torch.randn(H, N, N, generator=torch.Generator().manual_seed(0))
                            if False else bias)
        ok = full.shape == single.shape and torch.equal(full, single)
        local = op.forward_local(op.shard(q, rows), op.shard(k, rows), op.shard(v, rows),
                                 op.shard(mask_b, rows), bias)
        b, e = (rows + ws - 1) // ws * rank, min(rows, (rows + ws - 1) // ws * (rank + 1))
        ok = ok and torch.equal(local, single[b:e])
        # the gather on its own, with another row payload and a caller-supplied piece function
        # (what the distributed grid module does with its whole block per piece)
        table = torch.arange(rows * 15, dtype=torch.float32).reshape(rows, 5, 3)
        mine = table[b:e]
        seen = []

        def compute(lo, hi, slot, kw):
            seen.append((lo, hi))
            slot.copy_(mine[lo:hi] * 2.0)

        got = op.gather_rows(rows, (5, 3), torch.float32, torch.device("cpu"), compute)
        ok = ok and torch.equal(got, table * 2.0)
        ok = ok and sum(hi - lo for lo, hi in seen) == max(e - b, 0) and all(hi > lo for lo, hi in seen)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,comm_split", [(8, 1), (8, 4), (7, 2), (5, 4), (1, 1)])
def test_row_sharded_equals_single(rows, comm_split):
    ws = 2
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(ws, port, rows, comm_split, ret), nprocs=ws, join=True)
    assert all(ret.get(r) for r in range(ws)), dict(ret)


def _bad_worker(rank, ws, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=5))
    try:
        from af3_kernels_b200.distributed import RowShardedAttention
        op = RowShardedAttention(comm_split=1, attention_fn=_oracle_fn)
        q = torch.zeros(3, 1, 4, 8)      # 3 local rows, but a rank owns 2 of 4
        try:
            op.forward(q, q, q, None, torch.zeros(1, 4, 4), rows=4)
            ret[rank] = "no error"
        except ValueError:
            ret[rank] = "ValueError"
    finally:
        dist.destroy_process_group()


def test_wrong_local_shard_is_rejected_before_any_collective():
    ws = 2
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_bad_worker, args=(ws, port, ret), nprocs=ws, join=True)
    assert dict(ret) == {0: "ValueError", 1: "ValueError"}


def _lost_rank_worker(rank, ws, port, ret):
    """Rank 1 leaves between steps (never joins the gather); rank 0's collective must end with an
    error after the short process-group timeout instead of waiting forever."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=3))
    from af3_kernels_b200.distributed import RowShardedAttention
    if rank == 1:
        ret[rank] = "left"
        return
    op = RowShardedAttention(comm_split=1, attention_fn=_oracle_fn)
    q = torch.zeros(2, 1, 4, 8)
    try:
        op.forward(q, q, q, None, torch.zeros(1, 4, 4), rows=4, timeout_s=3.0)
        ret[rank] = "no error"
    except Exception as e:  # gloo reports a timeout / connection error
        ret[rank] = "error"


def test_lost_rank_ends_the_gather_with_an_error():
    ws = 2
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_lost_rank_worker, args=(ws, port, ret), nprocs=ws, join=True)
    assert ret[1] == "left" and ret[0] == "error", dict(ret)
