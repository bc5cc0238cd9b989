"""CPU checks of the oracles themselves: O1 against the golden vectors produced by the
reference's own PyTorch function, O2 (C restatement of the reference's bf16 TPP sequence)
against O1 within the error its rounding points imply."""
import pytest
import torch

from oracle import attention_oracle as O

# O1 and the reference function do the same fp32 operations in the same order
O1_TOL = 2e-6
# O2 rounds logits to bf16 three times before the softmax: error grows with |logit| (bias std)
O2_MAX_ABS = 6e-2
O2_MEAN_ABS = 3e-3


def test_o1_matches_reference_golden(golden):
    for name, c in golden.items():
        out = O.oracle_fp32(c["q"], c["k"], c["v"], c["mask"], c["bias"])
        assert out.shape == c["ref_fp32"].shape
        err = (out - c["ref_fp32"]).abs().max().item()
        assert err <= O1_TOL, (name, err)


def test_reference_bf16_run_is_close_to_fp32_golden(golden):
    # what the reference example itself prints as "Diff": bf16 torch vs the operator
    for name, c in golden.items():
        st = O.error_stats(c["ref_bf16"], c["ref_fp32"])
        assert st["max_abs"] <= 8e-2 and st["nan"] == 0, (name, st)


def test_o2_c_restatement_close_to_golden(golden):
    for name, c in golden.items():
        if name.startswith("fully_masked"):
            continue  # semantics differ on purpose, see test below
        out = O.ref_semantics(c["q"], c["k"], c["v"], c["mask"], c["bias"])
        st = O.error_stats(out, c["ref_fp32"])
        assert st["nan"] == 0 and st["max_abs"] <= O2_MAX_ABS and st["mean_abs"] <= O2_MEAN_ABS, (name, st)


def test_o2_float_instantiation_matches_o1(golden):
    for name, c in golden.items():
        if name.startswith("fully_masked"):
            continue
        q, k, v = c["q"].float(), c["k"].float(), c["v"].float()
        out = O.ref_semantics(q, k, v, c["mask"], c["bias"].float(), round_bf16=False)
        ref = O.oracle_fp32(q, k, v, c["mask"], c["bias"].float())
        assert (out - ref).abs().max().item() <= 5e-6, name


def test_o2_flash_branch_agrees_with_plain(golden):
    c = golden["pairformer_s200_d24_mask1d"]
    plain = O.ref_semantics(c["q"], c["k"], c["v"], c["mask"], c["bias"], BLK_SZ=64)
    flash = O.ref_semantics(c["q"], c["k"], c["v"], c["mask"], c["bias"], BLK_SZ=64,
                            use_flash=True, FLASH_SZ=64)
    st = O.error_stats(flash, plain)
    assert st["max_abs"] <= 6e-2 and st["mean_abs"] <= 3e-3, st
    # FLASH_SZ >= padded length falls back to the plain loop (dot_product_attention.cpp:76)
    same = O.ref_semantics(c["q"], c["k"], c["v"], c["mask"], c["bias"], BLK_SZ=64,
                           use_flash=True, FLASH_SZ=1024)
    assert torch.equal(same, plain)


def test_fully_masked_row_semantics(golden):
    c = golden["fully_masked_row_s128_d32"]
    v = c["v"].float()
    # the PyTorch oracle: every key at -1e9 -> uniform average over the S real keys
    ref_row0 = c["ref_fp32"][0]
    uniform = v[0].mean(dim=1, keepdim=True).expand_as(ref_row0)
    assert (ref_row0 - uniform).abs().max().item() <= 1e-5
    # O1 restates exactly that
    out = O.oracle_fp32(c["q"], c["k"], c["v"], c["mask"], c["bias"])
    assert (out[0] - uniform).abs().max().item() <= 1e-5
    # the C++ operator pads keys to BLK_SZ and masks the padding the same way, so with S a
    # multiple of BLK_SZ it is uniform too (up to bf16 rounding of 1/128 * sum)
    o2 = O.ref_semantics(c["q"], c["k"], c["v"], c["mask"], c["bias"])
    assert (o2[0] - uniform).abs().max().item() <= 2e-2


def test_o2_is_deterministic_and_thread_count_independent(golden):
    c = golden["grid_s130_d32_mask2d"]
    a = O.ref_semantics(c["q"], c["k"], c["v"], c["mask"], c["bias"], threads=1)
    b = O.ref_semantics(c["q"], c["k"], c["v"], c["mask"], c["bias"], threads=4)
    assert torch.equal(a, b)


@pytest.mark.parametrize("name", ["cfg1", "cfg3", "cfg4"])
def test_config_generators_shapes(name):
    rows = 1 if name != "cfg4" else 2
    inp = O.make_inputs(name, rows=rows, S=256)
    c = O.CONFIGS[name]
    assert inp["q"].shape == (rows, c["B2"], 256, c["D"])
    assert inp["bias"].dtype == c["bias_dtype"] and inp["bias"].shape == (c["B2"], 256, 256)
    assert inp["mask"].dtype == torch.bool and not inp["mask"][:, -1].any()
    again = O.make_inputs(name, rows=rows, S=256)
    assert torch.equal(inp["q"], again["q"]) and torch.equal(inp["bias"], again["bias"])


def test_fp8_config_quantisation_round_trip():
    inp = O.make_inputs("cfg5", rows=2, S=128)
    assert inp["q"].dtype == torch.float8_e4m3fn and inp["q_scale"].shape == (4,)
    deq = inp["q"].float() * inp["q_scale"].view(1, -1, 1, 1)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 4, 128, 32, generator=g)
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 for normal values
    assert ((deq - q).abs() <= q.abs() * 0.0625 + 2e-2).all()


def test_flop_and_byte_model():
    assert O.attention_flops(768, 4, 768, 768, 32) == pytest.approx(231.93e9, rel=1e-3)
    assert O.attention_bytes(768, 4, 768, 768, 32) == pytest.approx(614.0e6, rel=2e-3)
