"""CPU-only checks of the boundary: the library loads, exports every symbol the header
declares, validates arguments without a device, and the Python host side keeps the
reference's signatures.  No compute call is made here."""
import ctypes
import inspect
import os
import re

import pytest
import torch

import af3_kernels_b200 as A
from af3_kernels_b200 import _capi
from af3_kernels_b200.dpa import _mask_rows
from af3_kernels_b200.distributed import row_partition

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "af3k.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(af3k_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _capi.load()
    declared = _declared_symbols()
    assert declared, "no declarations found in include/af3k.h"
    for name in declared:
        assert hasattr(lib, name), f"libaf3k.so does not export {name}"
    assert sorted(_capi.EXPORTED_SYMBOLS) == declared


def test_version_and_strerror():
    lib = _capi.load()
    assert lib.af3k_version() >= 1000
    assert lib.af3k_strerror(0) == b"ok"
    for code in range(1, 10):
        assert lib.af3k_strerror(code) not in (b"", b"ok", b"unknown error code")
    assert lib.af3k_strerror(999) == b"unknown error code"


def _desc(B1, B2, S, D, bias_dtype=_capi.AF3K_F32, qk=_capi.AF3K_BF16):
    d = _capi.AttentionDesc()
    d.B1, d.B2, d.Sq, d.Sk, d.D = B1, B2, S, S, D
    for n in ("q_stride", "k_stride", "v_stride", "out_stride"):
        getattr(d, n)[:] = [B2 * S * D, S * D, D]
    d.bias_stride[:] = [S * S, S]
    d.mask_row_stride = S
    d.qk_dtype, d.bias_dtype = qk, bias_dtype
    d.softmax_scale = D ** -0.5
    return d


@pytest.mark.parametrize("shape", [(1, 16, 512, 32), (768, 4, 768, 32), (1, 16, 1536, 24),
                                   (5, 16, 1536, 48), (2048, 4, 2048, 32)])
def test_launch_plan_fits_b200(shape):
    plan = _capi.describe_plan(_desc(*shape))
    assert 1 <= plan["rows_per_item"] <= 8
    assert plan["kv_stages"] >= 2
    assert plan["smem_bytes"] <= 227 * 1024
    assert plan["tmem_cols"] <= 512
    assert 1 <= plan["grid"] <= 148 or not torch.cuda.is_available()
    B1, B2, S, _ = shape
    groups = -(-B1 // plan["rows_per_item"])
    n_qt = -(-S // 128)
    if plan["rows_per_item"] == 1 and n_qt >= 2:    # one pair row per item: two query tiles per item
        n_qt = -(-n_qt // 2)
    assert plan["items"] == groups * B2 * n_qt


def test_max_ctas_caps_the_grid():
    d = _desc(768, 4, 768, 32)
    full = _capi.describe_plan(d)
    d.max_ctas = 140
    capped = _capi.describe_plan(d)
    assert capped["grid"] == min(140, full["grid"]) and capped["items"] == full["items"]
    d.max_ctas = -1
    out = (ctypes.c_int32 * 6)()
    assert _capi.load().af3k_describe_plan(ctypes.byref(d), out) == 2


def test_argument_validation_codes():
    lib = _capi.load()
    out = (ctypes.c_int32 * 6)()
    bad_d = _desc(1, 1, 128, 20)
    assert lib.af3k_describe_plan(ctypes.byref(bad_d), out) == 2      # D not a multiple of 8
    big_d = _desc(1, 1, 128, 128)
    assert lib.af3k_describe_plan(ctypes.byref(big_d), out) == 2      # D > 64
    bad_t = _desc(1, 1, 128, 32, qk=7)
    assert lib.af3k_describe_plan(ctypes.byref(bad_t), out) == 1      # unknown dtype
    bad_s = _desc(1, 1, 128, 32)
    bad_s.q_stride[2] = 33
    assert lib.af3k_describe_plan(ctypes.byref(bad_s), out) == 3      # stride not 16-byte multiple
    assert lib.af3k_describe_plan(None, out) == 6                     # null descriptor
    assert lib.af3k_dot_product_attention(None, *([None] * 9), 0, None, None) == 6


def test_zero_strides_are_rejected_unless_the_extent_is_one():
    # a broadcast view (stride 0) cannot be described to TMA, and a zero output stride would make
    # rows overwrite each other: refused unless the dimension has one entry
    lib = _capi.load()
    out = (ctypes.c_int32 * 6)()
    for field in ("q_stride", "k_stride", "v_stride", "out_stride"):
        for dim in (0, 1):
            d = _desc(4, 2, 128, 32)
            getattr(d, field)[dim] = 0
            assert lib.af3k_describe_plan(ctypes.byref(d), out) == 3, (field, dim)
    d = _desc(4, 2, 128, 32)
    d.bias_stride[0] = 0
    assert lib.af3k_describe_plan(ctypes.byref(d), out) == 3
    ok = _desc(1, 1, 128, 32)                      # extent-1 dimensions may carry any stride
    for field in ("q_stride", "k_stride", "v_stride", "out_stride"):
        getattr(ok, field)[0] = 0
        getattr(ok, field)[1] = 0
    ok.bias_stride[0] = 0
    assert lib.af3k_describe_plan(ctypes.byref(ok), out) == 0


def test_boundary_names_of_the_reference_import():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "src"))
    import af3_kernels as K
    for name in ("Linear", "TriangleMultiplicationCpp", "DistributedTriangleMultiplicationCpp",
                 "GridSelfAttentionCpp", "DistributedGridSelfAttentionCpp"):
        assert hasattr(K, name), name
    lin = K.Linear(8, 4, bias=False)
    assert lin.weight.shape == (4, 8)
    with pytest.raises(NotImplementedError):
        K.TriangleMultiplicationCpp(128)
    with pytest.raises(NotImplementedError):
        K.DistributedTriangleMultiplicationCpp(128)


def test_workspace_size_rules():
    lib = _capi.load()
    f32 = _desc(1, 16, 512, 32, bias_dtype=_capi.AF3K_F32)
    assert lib.af3k_dot_product_attention_workspace(ctypes.byref(f32), None) == 16 * 512 * 512 * 2
    bf = _desc(1, 16, 512, 32, bias_dtype=_capi.AF3K_BF16)
    assert lib.af3k_dot_product_attention_workspace(ctypes.byref(bf), None) == 0
    odd = _desc(1, 2, 37, 32, bias_dtype=_capi.AF3K_BF16)   # 74-byte rows: TMA cannot address
    assert lib.af3k_dot_product_attention_workspace(ctypes.byref(odd), None) == 2 * 37 * 40 * 2


def test_reference_signatures_are_kept():
    sig = inspect.signature(A.dot_product_attention_cpp)
    names = list(sig.parameters)
    assert names[:8] == ["q", "k", "v", "mask", "bias", "use_flash_attention", "BLK_SZ", "FLASH_SZ"]
    assert sig.parameters["use_flash_attention"].default is False
    assert sig.parameters["BLK_SZ"].default == 128 and sig.parameters["FLASH_SZ"].default == 1024
    for extra in ("q_scale", "k_scale"):
        assert sig.parameters[extra].kind is inspect.Parameter.KEYWORD_ONLY
    for name in ("gated_linear_unit_cpp", "_attention_cpp", "self_attention_cpp", "pad_and_align_tensor",
                 "vnni_repack_tensor", "reset_debug_timers", "print_debug_timers",
                 "print_debug_thread_imbalance"):
        assert callable(getattr(A, name))
    with pytest.raises(NotImplementedError):
        A.gated_linear_unit_cpp(None, None)


def test_no_cpu_fallback():
    q = torch.zeros(1, 1, 8, 32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        A.dot_product_attention_cpp(q, q, q, torch.ones(8, dtype=torch.bool), torch.zeros(1, 8, 8))
    with pytest.raises(ValueError):
        A.dot_product_attention_cpp(q, q, q, None, torch.zeros(1, 8, 8), BLK_SZ=0)


def test_mask_forms():
    B1, S = 3, 10
    m1 = torch.ones(S, dtype=torch.bool)
    u, stride = _mask_rows(m1, B1, S)
    assert u.shape == (1, S) and stride == 0 and u.dtype == torch.uint8
    m2 = torch.ones(B1, S, dtype=torch.bool)
    u, stride = _mask_rows(m2, B1, S)
    assert u.shape == (B1, S) and stride == S
    u, stride = _mask_rows(m2[:, None, None, :], B1, S)
    assert u.shape == (B1, S) and stride == S
    u, stride = _mask_rows(torch.tensor([1.0, 0.0] * 5), B1, S)    # non-bool: non-zero = attend
    assert u.tolist() == [[1, 0] * 5]
    assert _mask_rows(None, B1, S) == (None, 0)
    with pytest.raises(ValueError):
        _mask_rows(torch.ones(2, S, dtype=torch.bool), B1, S)
    with pytest.raises(ValueError):
        _mask_rows(torch.ones(S + 1, dtype=torch.bool), B1, S)


def test_row_partition_matches_reference_rule():
    # rank r owns rows [r*ceil(rows/ws), (r+1)*ceil(rows/ws)) clipped to rows
    assert row_partition(2048, 8, 3) == (768, 1024, 256)
    assert row_partition(10, 4, 3) == (9, 10, 3)
    assert row_partition(5, 8, 7) == (5, 5, 1)
    covered = []
    for r in range(3):
        b, e, _ = row_partition(7, 3, r)
        covered += list(range(b, e))
    assert covered == list(range(7))
    with pytest.raises(ValueError):
        row_partition(4, 2, 2)


def test_pad_helpers():
    x = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    assert A.pad_and_align_tensor(x, (2, 3)) is x
    y = A.pad_and_align_tensor(x, (4, 4), True, 1.0)
    assert y.shape == (4, 4) and torch.equal(y[:2, :3], x) and y[3, 3] == 1.0
    z = A.pad_to_size(x, 5, 0)
    assert z.shape == (5, 3) and z[2:].abs().sum() == 0


def test_pair_bias_argument_validation_codes():
    lib = _capi.load()
    one = ctypes.c_void_p(16)
    args = lambda dtype=0, R=4, N=8, C=128, H=4, pitch=8: (one, dtype, R, N, C, H, one, one, one,
                                                           ctypes.c_float(1e-5), one, one, pitch, None)
    assert lib.af3k_pair_bias(*args(dtype=2)) == 1          # fp8 pair
    assert lib.af3k_pair_bias(*args(C=64)) == 2             # only c_pair = 128
    assert lib.af3k_pair_bias(*args(H=17)) == 2
    assert lib.af3k_pair_bias(*args(pitch=7)) == 3          # pitch < N
    assert lib.af3k_pair_bias(*args(N=8, pitch=12)) == 3    # pitch not a multiple of 8
    assert lib.af3k_pair_bias(*args(R=0)) == 0              # empty problem


def test_sigmoid_gate_argument_validation_codes():
    lib = _capi.load()
    one = ctypes.c_void_p(16)
    assert lib.af3k_sigmoid_gate(one, one, one, 12, None) == 2          # not a multiple of 8
    assert lib.af3k_sigmoid_gate(one, one, one, 0, None) == 0           # empty
    assert lib.af3k_sigmoid_gate(None, one, one, 8, None) == 6
    assert lib.af3k_sigmoid_gate(ctypes.c_void_p(8), one, one, 8, None) == 4
