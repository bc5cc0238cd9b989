"""GPU parity of the two attention blocks and the grid modules (projections through cuBLAS, core
through libaf3k.so) against golden outputs of the reference's PyTorch models and the fp32 block
oracles.  The blocks compute in bf16, so errors are judged against the size of the outputs:
max-abs <= 4 % of the largest reference magnitude, mean-abs <= 2 % of the mean magnitude (four
bf16 roundings in a row: projections, P, gated product, output projection)."""
import os
import socket

import pytest
import torch

import af3_kernels_b200 as A
from af3_kernels_b200.dpa import read_status
from oracle import attention_oracle as O
from test_blocks_oracle import blocks, grid_args, self_args  # noqa: F401  (fixture + helpers)

pytestmark = pytest.mark.gpu


def _close(out, ref, what):
    o, r = out.float().cpu(), ref.float()
    err = (o - r).abs()
    assert torch.isfinite(o).all(), what
    assert err.max().item() <= 0.04 * r.abs().max().item(), (what, err.max().item(), r.abs().max().item())
    assert err.mean().item() <= 0.02 * r.abs().mean().item(), (what, err.mean().item(), r.abs().mean().item())


def _grid_module(c, dev, cls=None):
    N, C, H, T = (int(v) for v in c["meta"])
    m = (cls or A.GridSelfAttentionCpp)(C, H, bool(T))
    m.load_state_dict({k[2:]: v for k, v in c.items() if k.startswith("w/")})
    return m.to(dev).eval()


def test_grid_module_matches_reference_model(cuda_device, blocks):
    for tag, c in blocks.items():
        if not tag.startswith("grid"):
            continue
        m = _grid_module(c, cuda_device)
        with torch.no_grad():
            out = m(c["pair"].to(cuda_device), c["mask"].to(cuda_device))
        assert out.shape == c["out"].shape and out.dtype == torch.float32
        _close(out, c["out"], tag)
    assert read_status(cuda_device)[0] == 0


def test_attention_cpp_operator_signature_path(cuda_device, blocks):
    c = blocks["grid_n24_c64_h2"]
    dev = cuda_device
    pair, mask, ln_w, ln_b, w_bias, w_q, w_k, w_v, w_g, w_o = (t.to(dev) for t in grid_args(c))
    x = torch.nn.functional.layer_norm(pair, (pair.shape[-1],), ln_w, ln_b)
    bias = torch.nn.functional.linear(x, w_bias).permute(2, 0, 1)
    rep = lambda w: A.vnni_repack_tensor(w.T.contiguous(), 2, 32)     # what the reference module does
    out = A._attention_cpp(x.to(torch.bfloat16), mask, bias, rep(w_q), rep(w_k), rep(w_v), rep(w_g),
                           w_o.T.contiguous(), 2, False, 64, 0)
    assert out.dtype == torch.bfloat16
    _close(out, c["out"], "_attention_cpp")


def test_self_attention_cpp_matches_reference_model(cuda_device, blocks):
    dev = cuda_device
    for tag, c in blocks.items():
        if not tag.startswith("self"):
            continue
        N, C, H = (int(v) for v in c["meta"])
        x, mask, logits, w_q, b_q, w_k, w_v, w_g = (t.to(dev) for t in self_args(c))
        out = A.self_attention_cpp(x, mask, logits, w_q.T.contiguous(), b_q, w_k.T.contiguous(),
                                   w_v.T.contiguous(), w_g.T.contiguous(), H)
        assert out.shape == (N, C) and out.dtype == torch.float32
        _close(out, c["out"], tag)


def test_grid_module_larger_shape_against_oracle(cuda_device):
    torch.manual_seed(3)
    N, C, H = 200, 128, 4
    m = A.GridSelfAttentionCpp(C, H, False)
    with torch.no_grad():
        for lin in (m.q_projection, m.k_projection):
            lin.weight.mul_(4.0)
        m.pair_bias_projection.weight.mul_(8.0)
    pair = torch.randn(N, N, C)
    mask = torch.rand(N, N) >= 0.05
    sd = m.state_dict()
    ref = O.grid_block_fp32(pair, mask, sd["act_norm.weight"], sd["act_norm.bias"],
                            sd["pair_bias_projection.weight"], sd["q_projection.weight"],
                            sd["k_projection.weight"], sd["v_projection.weight"],
                            sd["gating_query.weight"], sd["output_projection.weight"], H)
    m = m.to(cuda_device).eval()
    with torch.no_grad():
        out = m(pair.to(cuda_device), mask.to(cuda_device))
        again = m(pair.to(cuda_device), mask.to(cuda_device))
    _close(out, ref, "grid N=200")
    assert torch.equal(out, again)


def test_distributed_module_single_rank_equals_plain_module(cuda_device, blocks):
    import torch.distributed as dist
    c = blocks["grid_n36_c48_h2_t"]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                            device_id=cuda_device)
    try:
        plain = _grid_module(c, cuda_device)
        sharded = _grid_module(c, cuda_device, A.DistributedGridSelfAttentionCpp)
        pair, mask = c["pair"].to(cuda_device), c["mask"].to(cuda_device)
        with torch.no_grad():
            a = plain(pair, mask)
            b = sharded(pair, mask, COMM_SPLIT=3)
        assert a.shape == b.shape
        # same math on row pieces; the projection GEMMs may pick another tiling for another M
        assert (a - b).abs().max().item() <= 2e-2 * a.abs().max().item()
    finally:
        dist.destroy_process_group()


def test_fused_projection_kernel_matches_plain_gemms(cuda_device):
    """af3k_qkvg_projection: q, k, v head-major with q pre-scaled, gate row-major, against fp32
    matmuls of the same bf16 operands (bf16 rounding of the result only), on a ragged row count and
    for every head count the kernel takes."""
    from af3_kernels_b200.fused_ops import _stacked_projection_weights, qkvg_projection
    from af3_kernels_b200.dpa import read_status
    dev = cuda_device
    g = torch.Generator().manual_seed(3)
    for R, N, H in ((3, 200, 4), (1, 37, 2), (2, 129, 16), (5, 256, 8)):
        C, D = 128, 128 // H
        x = torch.randn(R, N, C, generator=g).to(torch.bfloat16).to(dev)
        ws = [(torch.randn(C, C, generator=g) * 0.1).to(torch.bfloat16).to(dev) for _ in range(4)]   # [in, out]
        w4 = _stacked_projection_weights(*ws)
        assert w4.shape == (4 * C, C)
        scale = D ** -0.5
        q, k, v, gate = qkvg_projection(x, w4, H, scale)
        torch.cuda.synchronize()
        assert read_status(dev)[0] == 0
        ref = [x.float() @ w.float() for w in ws]
        ref[0] = ref[0] * scale
        for got, want in zip((q, k, v), ref[:3]):
            want = want.view(R, N, H, D).permute(0, 2, 1, 3)
            assert got.shape == want.shape
            assert (got.float() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item()), (R, N, H)
        assert (gate.float() - ref[3]).abs().max().item() <= 2e-2 * max(1.0, ref[3].abs().max().item())


def test_self_block_replays_from_a_cuda_graph(cuda_device):
    """The block is a handful of short launches (four GEMMs, the attention kernel, the gate); its
    calls into the library allocate nothing the graph allocator cannot serve and never synchronise,
    so the whole block can be captured once and replayed - with results identical to the eager call."""
    dev = cuda_device
    g = torch.Generator().manual_seed(31)
    N, C, H = 200, 64, 4
    x = torch.randn(N, C, generator=g).to(torch.bfloat16).to(dev)
    ws = [(torch.randn(C, C, generator=g) * C ** -0.5).to(torch.bfloat16).to(dev) for _ in range(4)]
    qb = (torch.randn(C, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    bias = torch.randn(H, N, N, generator=g).to(torch.bfloat16).to(dev)
    mask = (torch.arange(N) < N - 17).to(dev)
    call = lambda: A.self_attention_cpp(x, mask, bias, ws[0], qb, ws[1], ws[2], ws[3], H)
    with torch.no_grad():
        ref = call()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            call()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out = call()
        torch.cuda.current_stream(dev).wait_stream(side)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize(dev)
    assert torch.equal(out, ref)
    assert read_status(dev)[0] == 0


def test_fused_front_matches_the_two_kernels_it_replaces(cuda_device):
    """af3k_pair_front (LayerNorm + pair bias + q/k/v/gate projections from the raw pair) against
    af3k_pair_bias followed by af3k_qkvg_projection: both round the normalised pair to bf16 before
    the projections; odd sizes cover tiles that straddle pair rows and the ragged last tile."""
    from af3_kernels_b200.fused_ops import _stacked_projection_weights, pair_front, qkvg_projection
    from af3_kernels_b200.pair_bias import layernorm_pair_bias
    dev = cuda_device
    for R, N, H, Hb in ((5, 200, 4, 4), (3, 128, 4, 2), (2, 37, 8, 1), (130, 130, 4, 4)):
        g = torch.Generator().manual_seed(100 + N)
        pair = (torch.randn(R, N, 128, generator=g) * 2.0 + 0.3).to(torch.bfloat16).to(dev)
        ln_w = (1.0 + 0.2 * torch.randn(128, generator=g)).to(dev)
        ln_b = (0.1 * torch.randn(128, generator=g)).to(dev)
        bw = (torch.randn(Hb, 128, generator=g) * 0.3).to(dev)
        ws = [(torch.randn(128, 128, generator=g) * 128 ** -0.5).to(torch.bfloat16).to(dev) for _ in range(4)]
        w4 = _stacked_projection_weights(*ws)
        D = 128 // H
        normed, bias_ref = layernorm_pair_bias(pair, ln_w, ln_b, bw)
        q_ref, k_ref, v_ref, g_ref = qkvg_projection(normed, w4, H, D ** -0.5)
        bias, q, k, v, gate = pair_front(pair, ln_w, ln_b, 1e-5, bw, w4, H, D ** -0.5)
        torch.cuda.synchronize(dev)
        assert read_status(dev)[0] == 0
        # the two LayerNorms order their arithmetic differently, so a normalised value may land on the
        # neighbouring bf16 now and then: the projections agree to a few bf16 ulps of their scale
        for a, b in ((q, q_ref), (k, k_ref), (v, v_ref), (gate, g_ref)):
            s_ = b.float().abs().max().item()
            assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -6 * s_
            assert (a.float() - b.float()).abs().mean().item() <= 2.0 ** -10 * s_
        scale = bias_ref.float().abs().max().item()
        assert (bias.float() - bias_ref.float()).abs().max().item() <= 2.0 ** -7 * scale + 1e-3
