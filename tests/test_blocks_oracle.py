"""CPU: the fp32 restatements of the two attention blocks against golden outputs of the
reference's own PyTorch models (tests/golden/make_golden_blocks.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def blocks():
    z = np.load(os.path.join(ROOT, "tests", "golden", "blocks_golden.npz"))
    out = {}
    for key in z.files:
        tag, rest = key.split("/", 1)
        out.setdefault(tag, {})[rest] = torch.from_numpy(z[key].copy())
    return out


def grid_args(c):
    w = {k[2:]: v for k, v in c.items() if k.startswith("w/")}
    return (c["pair"], c["mask"], w["act_norm.weight"], w["act_norm.bias"], w["pair_bias_projection.weight"],
            w["q_projection.weight"], w["k_projection.weight"], w["v_projection.weight"],
            w["gating_query.weight"], w["output_projection.weight"])


def self_args(c):
    w = {k[2:]: v for k, v in c.items() if k.startswith("w/")}
    return (c["x"], c["mask"], c["pair_logits"], w["q_projection.weight"], w["q_projection.bias"],
            w["k_projection.weight"], w["v_projection.weight"], w["gating_query.weight"])


def test_grid_block_restatement_matches_reference_model(blocks):
    for tag, c in blocks.items():
        if not tag.startswith("grid"):
            continue
        N, C, H, T = (int(v) for v in c["meta"])
        out = O.grid_block_fp32(*grid_args(c), H, transpose=bool(T))
        assert out.shape == c["out"].shape
        assert (out - c["out"]).abs().max().item() <= 5e-6, tag


def test_self_block_restatement_matches_reference_model(blocks):
    for tag, c in blocks.items():
        if not tag.startswith("self"):
            continue
        N, C, H = (int(v) for v in c["meta"])
        out = O.self_block_fp32(*self_args(c), H)
        assert out.shape == c["out"].shape
        assert (out - c["out"]).abs().max().item() <= 5e-6, tag
