"""GPU parity of the fused pair-bias producer (LayerNorm + bias projection + permute) against the
fp32 restatement of the reference's two PyTorch statements, through the C ABI.

Tolerances: the kernel writes bf16.  The normalised pair is compared with the fp32 LayerNorm at
bf16 resolution (one ulp, relative 2^-7 at most); the bias additionally with the bias recomputed in fp32 from the
kernel's own bf16 normalised pair, where only the summation order and the final bf16 rounding
differ (relative 2^-7 of the largest bias plus a small absolute term)."""
import pytest
import torch

from af3_kernels_b200 import _capi
from af3_kernels_b200.pair_bias import layernorm_pair_bias
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def _case(R, N, H, dtype, seed, dev):
    g = torch.Generator().manual_seed(seed)
    pair = (torch.randn(R, N, 128, generator=g) * 3.0 + 0.5).to(dtype)
    ln_w = 1.0 + 0.2 * torch.randn(128, generator=g)
    ln_b = 0.1 * torch.randn(128, generator=g)
    w = torch.randn(H, 128, generator=g) * 0.3
    normed, bias = layernorm_pair_bias(pair.to(dev), ln_w.to(dev), ln_b.to(dev), w.to(dev))
    torch.cuda.synchronize()
    assert bias.stride(2) == 1 and (bias.stride(1) * 2) % 16 == 0      # rows TMA can read in place
    return pair, ln_w, ln_b, w, normed.cpu(), bias.cpu()


@pytest.mark.parametrize("R,N,H,dtype", [(5, 37, 4, torch.float32), (3, 128, 4, torch.bfloat16),
                                         (2, 300, 16, torch.bfloat16), (3, 200, 8, torch.bfloat16),
                                         (1, 129, 5, torch.bfloat16), (1, 1, 1, torch.float32),
                                         (7, 264, 8, torch.float32)])
def test_pair_bias_matches_oracle(cuda_device, R, N, H, dtype):
    pair, ln_w, ln_b, w, normed, bias = _case(R, N, H, dtype, 11 + N, cuda_device)
    x_ref, b_ref = O.pair_bias_fp32(pair, ln_w, ln_b, w)
    assert normed.shape == (R, N, 128) and normed.dtype == torch.bfloat16
    assert bias.shape == (H, R, N) and bias.dtype == torch.bfloat16
    assert ((normed.float() - x_ref).abs() <= 2.0 ** -7 * x_ref.abs() + 1e-6).all()      # one bf16 ulp
    # the projection as the kernel defines it: from the bf16 normalised pair
    b_same = torch.nn.functional.linear(normed.float(), w).permute(2, 0, 1)
    scale = b_same.abs().max().item()
    assert (bias.float() - b_same).abs().max().item() <= 2.0 ** -7 * scale + 1e-3
    # and against the all-fp32 oracle
    assert (bias.float() - b_ref).abs().max().item() <= 2e-2 * max(1.0, scale)
    assert _capi.load().af3k_last_launch_count() == 1
    import ctypes
    st = (ctypes.c_int32 * 4)()
    assert _capi.load().af3k_pair_bias_status(st) == 0 and list(st) == [0, 0, 0, 0]   # no wait of the tensor-core kernel ran out


def test_pair_bias_full_size_properties(cuda_device):
    """N = 768 (the benchmark's pair size): spot rows against the oracle, and the normalised
    vectors really are normalised (zero mean, unit variance before the affine part)."""
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(5)
    N, H = 768, 4
    pair = torch.randn(N, N, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    ln_w = torch.ones(128, device=dev)
    ln_b = torch.zeros(128, device=dev)
    w = torch.randn(H, 128, generator=g, device=dev) * 0.2
    normed, bias = layernorm_pair_bias(pair, ln_w, ln_b, w)
    again_n, again_b = layernorm_pair_bias(pair, ln_w, ln_b, w)
    assert torch.equal(normed, again_n) and torch.equal(bias, again_b)
    nf = normed.float()
    assert nf.mean(dim=-1).abs().max().item() <= 2e-2
    assert (nf.var(dim=-1, unbiased=False) - 1.0).abs().max().item() <= 3e-2
    rows = [0, 401, 767]
    x_ref, b_ref = O.pair_bias_fp32(pair[rows].cpu(), ln_w.cpu(), ln_b.cpu(), w.cpu())
    assert (bias[:, rows].float().cpu() - b_ref).abs().max().item() <= 3e-2


def test_pair_bias_feeds_attention_in_place(cuda_device):
    """The bias view goes straight into the attention operator: no staging launch."""
    from af3_kernels_b200.dpa import dot_product_attention
    dev = cuda_device
    g = torch.Generator().manual_seed(9)
    N, H, D = 72, 4, 32
    pair = torch.randn(N, N, 128, generator=g).to(torch.bfloat16).to(dev)
    normed, bias = layernorm_pair_bias(pair, torch.ones(128, device=dev), torch.zeros(128, device=dev),
                                       (torch.randn(H, 128, generator=g) * 0.2).to(dev))
    q = torch.randn(N, H, N, D, generator=g).to(torch.bfloat16).to(dev)
    out = dot_product_attention(q, q, q, None, bias, check_status=True)
    assert _capi.load().af3k_last_launch_count() == 1
    ref = O.oracle_fp32(q.cpu(), q.cpu(), q.cpu(), None, bias.cpu())
    st = O.error_stats(out.cpu(), ref)
    assert st["nan"] == 0 and st["max_abs"] <= 2e-2, st


def test_sigmoid_gate_matches_fp32(cuda_device):
    from af3_kernels_b200.fused_ops import sigmoid_gate
    g = torch.Generator().manual_seed(3)
    for shape in ((5, 37, 128), (1, 8), (300, 264)):
        w = (torch.randn(*shape, generator=g) * 2).to(torch.bfloat16).to(cuda_device)
        x = (torch.randn(*shape, generator=g) * 6).to(torch.bfloat16).to(cuda_device)
        x.view(-1)[:4] = torch.tensor([-200.0, 200.0, 0.0, -30.0], dtype=torch.bfloat16)
        out = sigmoid_gate(w, x)
        ref = w.float() * torch.sigmoid(x.float())
        assert out.dtype == torch.bfloat16 and torch.isfinite(out.float()).all()
        assert ((out.float() - ref).abs() <= 2.0 ** -7 * ref.abs() + 1e-6).all()      # one bf16 ulp
    # shapes the kernel does not take go through torch and agree as well
    w = torch.randn(3, 5, device=cuda_device).to(torch.bfloat16)
    assert torch.equal(sigmoid_gate(w, w), w * torch.sigmoid(w))
