"""The allocation-free entry point, called straight through the C ABI.

Some hosts of this library cannot give it scratch memory: all device memory already belongs to
their own arena, or their plug-in boundary only carries inputs and outputs, or they run where
cudaMalloc is off limits.  ``af3k_dot_product_attention_noalloc`` serves them from an array built
into the library.  It must give the same bits as the ordinary entry point, on consecutive calls
that reuse the array with different problem sizes, and must refuse problems that do not fit.

This file sorts last on purpose, so a run that stops at the first failure has already gone
through every other test.
"""
import ctypes

import pytest
import torch

from af3_kernels_b200 import _capi
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def _desc(q, out, bias, mask_stride):
    B1, B2, S, D = q.shape
    d = _capi.AttentionDesc()
    d.B1, d.B2, d.Sq, d.Sk, d.D = B1, B2, S, S, D
    for n, t in (("q_stride", q), ("k_stride", q), ("v_stride", out), ("out_stride", out)):
        getattr(d, n)[:] = [t.stride(0), t.stride(1), t.stride(2)]
    d.bias_stride[:] = [bias.stride(0), bias.stride(1)]
    d.mask_row_stride = mask_stride
    d.qk_dtype = _capi.AF3K_FP8_E4M3 if q.dtype == torch.float8_e4m3fn else _capi.AF3K_BF16
    d.bias_dtype = _capi.AF3K_F32 if bias.dtype == torch.float32 else _capi.AF3K_BF16
    d.softmax_scale = D ** -0.5
    return d


def _problem(dev, B1, B2, S, D, seed, bias_dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16).to(dev)
    bias = torch.randn(B2, S, S, generator=g).to(bias_dtype).to(dev)
    mask = (torch.rand(B1, S, generator=g) >= 0.1).to(dev).view(torch.uint8)
    return q, k, v, bias, mask


def _both_entry_points(dev, q, k, v, bias, mask, q_scale=None, k_scale=None, give_workspace=True):
    """Runs the ordinary entry point (with a torch-allocated workspace, or none) and the
    allocation-free one on the same problem.  Around the allocation-free call the amount of free
    device memory the driver reports must not move: it may not allocate, and neither may anything
    it calls."""
    lib = _capi.load()
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out_ws = torch.empty_like(v)
    out_na = torch.empty_like(v)
    d = _desc(q, out_ws, bias, mask.stride(0))
    need = lib.af3k_dot_product_attention_workspace(ctypes.byref(d), bias.data_ptr())
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
    qs = q_scale.data_ptr() if q_scale is not None else None
    ks = k_scale.data_ptr() if k_scale is not None else None
    rc = lib.af3k_dot_product_attention(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                        bias.data_ptr(), mask.data_ptr(), out_ws.data_ptr(), qs, ks,
                                        ws.data_ptr() if give_workspace else None, need if give_workspace else 0,
                                        status.data_ptr(), stream)
    assert rc == 0, lib.af3k_strerror(rc)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    rc = lib.af3k_dot_product_attention_noalloc(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                bias.data_ptr(), mask.data_ptr(), out_na.data_ptr(), qs,
                                                ks, status.data_ptr(), stream)
    launches = lib.af3k_last_launch_count()
    assert rc == 0, (lib.af3k_strerror(rc), lib.af3k_last_error_detail())
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before, "the allocation-free entry point changed the device's free memory"
    assert status[0].item() == 0
    return out_ws, out_na, need, launches


def _oracle(q, k, v, bias, mask, q_scale=None, k_scale=None):
    return O.oracle_fp32(q.cpu(), k.cpu(), v.cpu(), mask.cpu().view(torch.bool), bias.cpu(),
                         q_scale=None if q_scale is None else q_scale.cpu(),
                         k_scale=None if k_scale is None else k_scale.cpu())


def test_noalloc_matches_workspace_entry_on_consecutive_calls(cuda_device):
    dev = cuda_device
    lib = _capi.load()
    assert lib.af3k_static_scratch_bytes() == 16 << 20
    # first call: fp32 bias, 300 keys -> staging copy with padded pitch in the built-in array
    q, k, v, bias, mask = _problem(dev, 3, 4, 300, 32, seed=11)
    _both_entry_points(dev, q, k, v, bias, mask)      # first call on the device: address look-up
    a_ws, a_na, need_a, _ = _both_entry_points(dev, q, k, v, bias, mask)
    assert need_a > 0
    assert torch.equal(a_ws, a_na)
    st = O.error_stats(a_na.cpu(), _oracle(q, k, v, bias, mask))
    assert st["nan"] == 0 and st["max_abs"] <= 2e-2 and st["mean_abs"] <= 2e-3, st
    # second call, straight after, smaller and differently shaped: whatever the first call left
    # in the array must not leak into it
    q, k, v, bias, mask = _problem(dev, 2, 2, 77, 48, seed=12)
    b_ws, b_na, need_b, _ = _both_entry_points(dev, q, k, v, bias, mask)
    assert 0 < need_b < need_a
    assert torch.equal(b_ws, b_na)
    st = O.error_stats(b_na.cpu(), _oracle(q, k, v, bias, mask))
    assert st["nan"] == 0 and st["max_abs"] <= 2e-2 and st["mean_abs"] <= 2e-3, st
    # and a bias that needs no staging at all leaves the array untouched and still works
    q, k, v, bias, mask = _problem(dev, 2, 2, 128, 32, seed=13, bias_dtype=torch.bfloat16)
    c_ws, c_na, need_c, launches = _both_entry_points(dev, q, k, v, bias, mask)
    assert need_c == 0 and launches == 1 and torch.equal(c_ws, c_na)
    assert torch.isfinite(a_na.float()).all() and torch.isfinite(b_na.float()).all()


def _fp8_problem(dev, B1, B2, S, D, seed):
    g = torch.Generator().manual_seed(seed)
    q, qs = O.quantize_e4m3_per_head(torch.randn(B1, B2, S, D, generator=g))
    k, ks = O.quantize_e4m3_per_head(torch.randn(B1, B2, S, D, generator=g))
    v = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16)
    bias = torch.randn(B2, S, S, generator=g).to(torch.bfloat16)
    mask = (torch.rand(B1, S, generator=g) >= 0.1).view(torch.uint8)
    return [t.to(dev) for t in (q, k, v, bias, mask, qs, ks)]


def test_noalloc_fp8_with_and_without_room_for_the_optional_copy(cuda_device):
    """With fp8 q/k the staging copy (bias divided by the head's logit scale) is optional.  When it
    fits the built-in array both entry points run the same two kernels and give the same bits;
    when it does not fit (here 4 x 1536 x 1536 x 2 bytes = 18.9 MB > 16 MiB) the allocation-free
    entry point leaves it out, launches the one kernel whose softmax threads add the bias, and
    gives the bits of the ordinary entry point called without a workspace."""
    dev = cuda_device
    q, k, v, bias, mask, qs, ks = _fp8_problem(dev, 2, 2, 296, 32, seed=21)
    ws, na, need, launches = _both_entry_points(dev, q, k, v, bias, mask, qs, ks)
    assert 0 < need <= (16 << 20) and launches == 2
    assert torch.equal(ws, na)
    st = O.error_stats(na.cpu(), _oracle(q, k, v, bias, mask, qs, ks))
    assert st["nan"] == 0 and st["max_abs"] <= 6e-2, st

    q, k, v, bias, mask, qs, ks = _fp8_problem(dev, 1, 4, 1536, 32, seed=22)
    ws, na, need, launches = _both_entry_points(dev, q, k, v, bias, mask, qs, ks, give_workspace=False)
    assert need > (16 << 20) and launches == 1
    assert torch.equal(ws, na)
    st = O.error_stats(na.cpu(), _oracle(q, k, v, bias, mask, qs, ks))
    assert st["nan"] == 0 and st["max_abs"] <= 6e-2, st


def test_noalloc_refuses_problems_beyond_the_built_in_array(cuda_device):
    dev = cuda_device
    lib = _capi.load()
    # 16 heads x 1024 x 1024 fp32 bias -> 32 MiB staging copy > 16 MiB
    S = 1024
    q = torch.zeros(1, 16, S, 32, dtype=torch.bfloat16, device=dev)
    bias = torch.zeros(16, S, S, device=dev)
    out = torch.full_like(q, 3.0)
    d = _desc(q, out, bias, 0)
    rc = lib.af3k_dot_product_attention_noalloc(ctypes.byref(d), q.data_ptr(), q.data_ptr(), q.data_ptr(),
                                                bias.data_ptr(), None, out.data_ptr(), None, None, None,
                                                torch.cuda.current_stream().cuda_stream)
    assert rc == 9
    assert b"scratch" in lib.af3k_strerror(rc)
    assert b"built-in" in lib.af3k_last_error_detail()
    torch.cuda.synchronize()
    assert (out == 3.0).all(), "nothing may be launched for a refused call"
