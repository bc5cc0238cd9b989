"""The operator's host-tensor path (row blocks pipelined over PCIe): same result as the device
path, through the reference's own call signature."""
import pytest
import torch

import af3_kernels_b200 as A
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pinned", [True, False])
def test_host_tensors_give_the_device_result(cuda_device, pinned):
    g = torch.Generator().manual_seed(31)
    B1, B2, S, D = 13, 2, 200, 32
    q = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16)
    bias = torch.randn(B2, S, S, generator=g)                      # fp32, as the reference's callers pass it
    mask = torch.rand(B1, S, generator=g) >= 0.1
    if pinned:
        q, k, v, bias, mask = (t.pin_memory() for t in (q, k, v, bias, mask))
    out = A.dot_product_attention_cpp(q, k, v, mask, bias)          # host in, host out
    assert not out.is_cuda and out.shape == (B1, B2, S, D) and out.dtype == torch.bfloat16
    dev = cuda_device
    ref_dev = A.dot_product_attention_cpp(q.to(dev), k.to(dev), v.to(dev), mask.to(dev), bias.to(dev))
    assert torch.equal(out, ref_dev.cpu())
    st = O.error_stats(out, O.oracle_fp32(q, k, v, mask, bias))
    assert st["nan"] == 0 and st["max_abs"] <= 2e-2, st
    # uneven row blocks, 1-D mask, preallocated output
    out2 = torch.empty_like(out)
    A.dot_product_attention_host(q, k, v, mask[0], bias, out=out2, chunks=5)
    ref2 = A.dot_product_attention_cpp(q.to(dev), k.to(dev), v.to(dev), mask[0].to(dev), bias.to(dev))
    assert torch.equal(out2, ref2.cpu())


def test_host_path_rejects_cuda_tensors(cuda_device):
    q = torch.zeros(1, 1, 8, 32, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError):
        A.dot_product_attention_host(q, q, q, None, torch.zeros(1, 8, 8))
