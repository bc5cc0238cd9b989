"""Every output row of the two large benchmark configurations at FULL size against the fp32
oracle.

The CPU oracle would need minutes for 768 x 4 x 768 x 768 (and much longer for 2048 x 4 x 2048 x
2048) logits, so the same oracle function (oracle_fp32: plain torch, device-agnostic) is evaluated
in fp32 on the GPU in row chunks with TF32 switched off.  That stand-in is first held to the CPU
evaluation on the golden vectors (1e-5), then used as the reference for every row.
Tolerances: bf16 max-abs <= 2e-2 and mean-abs <= 2e-3; fp8 (de-quantised oracle) max-abs <= 6e-2.
"""
import pytest
import torch

from af3_kernels_b200.dpa import dot_product_attention
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

BF16_MAX_ABS, BF16_MEAN_ABS = 2e-2, 2e-3
FP8_MAX_ABS = 6e-2


@pytest.fixture(autouse=True)
def _exact_fp32_matmul():
    old = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = old


def _gpu_oracle_rows(q, k, v, mask, bias, q_scale, k_scale, lo, hi):
    return O.oracle_fp32(q[lo:hi], k[lo:hi], v[lo:hi], mask[lo:hi] if mask is not None and mask.dim() == 2 else mask,
                         bias, q_scale=q_scale, k_scale=k_scale)


def test_gpu_evaluation_of_the_oracle_equals_the_cpu_one(cuda_device, golden):
    for name, c in golden.items():
        cpu = O.oracle_fp32(c["q"], c["k"], c["v"], c["mask"], c["bias"])
        dev = [t.to(cuda_device) if t is not None else None for t in (c["q"], c["k"], c["v"], c["mask"], c["bias"])]
        gpu = O.oracle_fp32(*dev).cpu()
        assert (gpu - cpu).abs().max().item() <= 1e-5, name
        assert (gpu - c["ref_fp32"]).abs().max().item() <= 1e-5, name


def _full_size_case(dev, name, chunk):
    c = O.CONFIGS[name]
    B1, B2, S, D = c["B1"], c["B2"], c["S"], c["D"]
    g = torch.Generator(device=dev).manual_seed(11)
    qf = torch.randn(B1, B2, S, D, generator=g, device=dev)
    kf = torch.randn(B1, B2, S, D, generator=g, device=dev)
    v = torch.randn(B1, B2, S, D, generator=g, device=dev).to(torch.bfloat16)
    bias = (torch.randn(B2, S, S, generator=g, device=dev) * c["bias_std"]).to(c["bias_dtype"])
    mask = torch.rand(B1, S, generator=g, device=dev) >= 0.05
    if c.get("fp8"):
        q, qs = O.quantize_e4m3_per_head(qf)
        k, ks = O.quantize_e4m3_per_head(kf)
        kw = dict(q_scale=qs, k_scale=ks)
    else:
        q, k, qs, ks, kw = qf.to(torch.bfloat16), kf.to(torch.bfloat16), None, None, {}
    del qf, kf
    out = dot_product_attention(q, k, v, mask, bias, check_status=True, **kw)
    worst, total, nan = 0.0, 0.0, 0
    for lo in range(0, B1, chunk):
        hi = min(B1, lo + chunk)
        ref = _gpu_oracle_rows(q, k, v, mask, bias, qs, ks, lo, hi)
        d = (out[lo:hi].float() - ref).abs()
        nan += int(torch.isnan(out[lo:hi]).sum().item())
        worst = max(worst, d.max().item())
        total += d.sum().item()
        del ref, d
    return worst, total / out.numel(), nan


def test_cfg2_full_size_every_row(cuda_device):
    worst, mean, nan = _full_size_case(cuda_device, "cfg2", chunk=32)
    assert nan == 0 and worst <= BF16_MAX_ABS and mean <= BF16_MEAN_ABS, (worst, mean, nan)


def test_cfg5_fp8_full_size_every_row(cuda_device):
    worst, mean, nan = _full_size_case(cuda_device, "cfg5", chunk=8)
    assert nan == 0 and worst <= FP8_MAX_ABS, (worst, mean, nan)
