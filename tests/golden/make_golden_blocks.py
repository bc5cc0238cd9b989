"""Generates tests/golden/blocks_golden.npz from the reference's own PyTorch models of the two
attention blocks.

    python tests/golden/make_golden_blocks.py <path of the reference checkout>

The classes ``AttentionTorch`` of ``examples/grid_self_attention.py`` and
``examples/self_attention.py`` are taken out of the reference's files at run time (source parsed,
the class definition compiled and executed); the rest of those scripts needs the reference's
compiled extension.  Weights, inputs and outputs of small seeded instances are stored; at test
time only the committed ``.npz`` is read.
"""
from __future__ import annotations

import ast
import os
import sys
from typing import Optional

import einops
import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


def load_class(path: str, name: str):
    tree = ast.parse(open(path).read(), filename=path)
    cls = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == name)
    ns = {"torch": torch, "nn": nn, "Optional": Optional, "einops": einops}
    exec(compile(ast.Module(body=[cls], type_ignores=[]), path, "exec"), ns)
    return ns[name]


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + sys.argv[0] + " <path of the reference checkout>")
    ref = sys.argv[1]
    out = {}
    Grid = load_class(os.path.join(ref, "examples", "grid_self_attention.py"), "AttentionTorch")
    for tag, N, c_pair, heads, transpose in (("grid_n24_c64_h2", 24, 64, 2, False),
                                             ("grid_n36_c48_h2_t", 36, 48, 2, True)):
        torch.manual_seed(1896)
        m = Grid(c_pair, heads, transpose).eval()
        with torch.no_grad():
            m.act_norm.weight.uniform_(0.5, 1.5)
            m.act_norm.bias.uniform_(-0.5, 0.5)
            for lin in (m.q_projection, m.k_projection, m.v_projection):
                lin.weight.mul_(4.0)          # logits of a useful size for a parity check
            m.pair_bias_projection.weight.mul_(8.0)
            pair = torch.randn(N, N, c_pair)
            mask = torch.rand(N, N) >= 0.1
            y = m(pair, mask)
        out[f"{tag}/pair"] = pair.numpy()
        out[f"{tag}/mask"] = mask.numpy()
        out[f"{tag}/out"] = y.numpy()
        out[f"{tag}/meta"] = np.array([N, c_pair, heads, int(transpose)])
        for k, v in m.state_dict().items():
            out[f"{tag}/w/{k}"] = v.numpy()
    Self = load_class(os.path.join(ref, "examples", "self_attention.py"), "AttentionTorch")
    for tag, N, c_x, heads in (("self_n90_c96_h2", 90, 96, 2), ("self_n130_c64_h2", 130, 64, 2)):
        torch.manual_seed(1896)
        m = Self(c_x=c_x, num_head=heads).eval()
        with torch.no_grad():
            for lin in (m.q_projection, m.k_projection):
                lin.weight.mul_(4.0)
            x = torch.randn(N, c_x)
            mask = torch.ones(N, dtype=torch.bool)
            mask[N - N // 6:] = False
            logits = torch.randn(heads, N, N)
            y = m(x, mask, logits)
        out[f"{tag}/x"] = x.numpy()
        out[f"{tag}/mask"] = mask.numpy()
        out[f"{tag}/pair_logits"] = logits.numpy()
        out[f"{tag}/out"] = y.numpy()
        out[f"{tag}/meta"] = np.array([N, c_x, heads])
        for k, v in m.state_dict().items():
            out[f"{tag}/w/{k}"] = v.numpy()
    path = os.path.join(HERE, "blocks_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
