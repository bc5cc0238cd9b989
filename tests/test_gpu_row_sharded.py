"""Row-sharded attention on two or more GPUs of one node (NCCL): the gathered output must equal
the single-GPU output bit for bit, for an even and a ragged row split.  Needs at least two CUDA
devices; skipped otherwise (the partition / gather logic itself is covered on CPU ranks in
test_distributed_cpu.py).  Ranks are child processes; NVLS is switched off."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, ws, port, rows, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import datetime
    import torch.distributed as dist
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from af3_kernels_b200.distributed import RowShardedAttention
        from af3_kernels_b200.dpa import dot_product_attention, read_status
        g = torch.Generator(device=dev).manual_seed(3)          # same seed: identical on every rank
        H, N, D = 4, 300, 32
        q = torch.randn(rows, H, N, D, generator=g, device=dev).to(torch.bfloat16)
        k = torch.randn(rows, H, N, D, generator=g, device=dev).to(torch.bfloat16)
        v = torch.randn(rows, H, N, D, generator=g, device=dev).to(torch.bfloat16)
        bias = torch.randn(H, N, N, generator=g, device=dev)
        mask = torch.rand(rows, N, generator=g, device=dev) >= 0.1
        single = dot_product_attention(q, k, v, mask, bias)
        op = RowShardedAttention(comm_split=3)
        # replicated operands arrive by broadcast from rank 0
        b_in = bias.clone() if rank == 0 else torch.zeros_like(bias)
        m_in = (mask.clone() if rank == 0 else torch.zeros_like(mask)).view(torch.uint8)
        op.broadcast_shared(b_in, m_in)
        ok, used = True, []
        # every form of the exchange, the default first ("auto": peer copies into symmetric memory
        # where that can be set up); two calls each, since the result buffers alternate
        for exchange in ("auto", "sendrecv", "broadcast", "allgather"):
            op.exchange = exchange
            for _ in range(2):
                full = op.forward(op.shard(q, rows), op.shard(k, rows), op.shard(v, rows),
                                  op.shard(m_in.view(torch.bool), rows), b_in, rows)
                torch.cuda.synchronize()
                ok = ok and full.shape == single.shape and torch.equal(full, single) and read_status(dev)[0] == 0
            used.append(op.last_exchange)
        ret[rank] = bool(ok) and used[1:] == ["sendrecv", "broadcast", "allgather"]
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("rows", [8, 7])
def test_sharded_output_equals_single_gpu(cuda_device, rows):
    ws = min(torch.cuda.device_count(), 4)
    if ws < 2:
        pytest.skip("needs at least two CUDA devices")
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, ws, port, rows, ret)) for r in range(ws)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all(ret.get(r) for r in range(ws)), dict(ret)



def _module_worker(rank, ws, port, n, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import datetime
    import torch.distributed as dist
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        import af3_kernels_b200 as A
        torch.manual_seed(11)                                    # same weights on every rank
        plain = A.GridSelfAttentionCpp(128, 4).to(dev).to(torch.bfloat16).eval()
        shard = A.DistributedGridSelfAttentionCpp(128, 4).to(dev).to(torch.bfloat16).eval()
        shard.load_state_dict(plain.state_dict())
        g = torch.Generator(device=dev).manual_seed(12)
        pair = torch.randn(n, n, 128, generator=g, device=dev).to(torch.bfloat16)
        mask = torch.rand(n, n, generator=g, device=dev) >= 0.1
        with torch.no_grad():
            ref = plain(pair, mask)
            ok = True
            for _ in range(2):                                   # the result buffers alternate per call
                out = shard(pair, mask, COMM_SPLIT=3)
                torch.cuda.synchronize()
                # row blocks of other sizes may take another GEMM kernel in the output projection:
                # equal to a bf16 ulp of the largest value, not bit for bit
                tol = 2.0 ** -7 * ref.float().abs().max().item()
                ok = ok and out.shape == ref.shape and (out.float() - ref.float()).abs().max().item() <= tol
        ret[rank] = bool(ok)
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [160, 135])
def test_distributed_grid_module_equals_plain_module(cuda_device, n):
    """DistributedGridSelfAttentionCpp on two or more GPUs against GridSelfAttentionCpp on one, for a
    row count the ranks share evenly and one they do not."""
    ws = min(torch.cuda.device_count(), 4)
    if ws < 2:
        pytest.skip("needs at least two CUDA devices")
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_module_worker, args=(r, ws, port, n, ret)) for r in range(ws)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all(ret.get(r) for r in range(ws)), dict(ret)
