"""Generates tests/golden/dpa_golden.npz from the reference's own PyTorch comparison function.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py <path of the reference checkout>

The function ``dot_product_attention_torch`` is taken verbatim out of the reference's
``examples/dot_product_attention.py`` at run time (its source text is parsed, the one function
definition is compiled and executed) - the rest of that script needs the reference's compiled
extension, which cannot be built without libxsmm.  The outputs it produces on small seeded
inputs are the golden vectors that pin oracle/attention_oracle.py::oracle_fp32.  Nothing at test
time reads the reference checkout; only the committed ``.npz`` is used.
"""
from __future__ import annotations

import ast
import os
import sys
from typing import Optional

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, B1, B2, S, D, mask form, bias dtype, bias std
CASES = [
    ("single_s64_d32_mask2d", 1, 4, 64, 32, "2d_tail", "float32", 1.0),
    ("grid_s37_d32_mask2d", 5, 2, 37, 32, "2d_rand", "float32", 1.0),
    ("grid_s130_d32_mask2d", 2, 2, 130, 32, "2d_rand", "bfloat16", 1.0),
    ("pairformer_s200_d24_mask1d", 1, 2, 200, 24, "1d_tail", "bfloat16", 2.0),
    ("diffusion_s96_d48_mask2d", 3, 2, 96, 48, "2d_tail", "bfloat16", 1.0),
    ("fully_masked_row_s128_d32", 2, 1, 128, 32, "2d_row0_all_masked", "float32", 1.0),
    ("no_mask_s160_d64", 1, 1, 160, 64, "none", "float32", 1.0),
]


def load_reference_function(ref_root: str):
    path = os.path.join(ref_root, "examples", "dot_product_attention.py")
    tree = ast.parse(open(path).read(), filename=path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef)
              and n.name == "dot_product_attention_torch")
    mod = ast.Module(body=[fn], type_ignores=[])
    ns = {"torch": torch, "Optional": Optional}
    exec(compile(mod, path, "exec"), ns)
    return ns["dot_product_attention_torch"]


def make_case(name, B1, B2, S, D, mask_form, bias_dtype, bias_std, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B1, B2, S, D, generator=g).to(torch.bfloat16)
    bias = (torch.randn(B2, S, S, generator=g) * bias_std).to(getattr(torch, bias_dtype))
    if mask_form == "none":
        mask = None
    elif mask_form == "1d_tail":
        mask = torch.ones(S, dtype=torch.bool)
        mask[S - S // 8:] = False
    elif mask_form == "2d_tail":
        mask = torch.ones(B1, S, dtype=torch.bool)
        mask[:, S - S // 8:] = False
    elif mask_form == "2d_rand":
        mask = torch.rand(B1, S, generator=g) >= 0.05
    elif mask_form == "2d_row0_all_masked":
        mask = torch.rand(B1, S, generator=g) >= 0.05
        mask[0, :] = False
    else:
        raise ValueError(mask_form)
    return q, k, v, bias, mask


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + sys.argv[0] + " <path of the reference checkout>")
    ref_root = sys.argv[1]
    ref_fn = load_reference_function(ref_root)
    out = {}
    for i, (name, B1, B2, S, D, mf, bd, bs) in enumerate(CASES):
        q, k, v, bias, mask = make_case(name, B1, B2, S, D, mf, bd, bs, seed=1896 + i)
        # fp32 run of the reference function on the stored (bf16) inputs: the grading oracle
        ref32 = ref_fn(q.float(), k.float(), v.float(), mask, bias.float())
        # the run the reference example actually performs: every tensor in bf16
        ref16 = ref_fn(q, k, v, mask, bias.to(torch.bfloat16))
        out[f"{name}/q"] = bits(q)
        out[f"{name}/k"] = bits(k)
        out[f"{name}/v"] = bits(v)
        out[f"{name}/bias"] = bits(bias)
        out[f"{name}/bias_is_bf16"] = np.array(bd == "bfloat16")
        if mask is not None:
            out[f"{name}/mask"] = mask.numpy()
        out[f"{name}/ref_fp32"] = ref32.numpy()
        out[f"{name}/ref_bf16"] = bits(ref16)
    np.savez_compressed(os.path.join(HERE, "dpa_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "dpa_golden.npz"), len(CASES), "cases")


if __name__ == "__main__":
    main()
