"""TEST INFRASTRUCTURE - CPU oracles for biased, key-masked attention.  Not a product path.

Two oracles:

* ``oracle_fp32`` (O1, the grading oracle): an fp32 restatement of the PyTorch comparison
  function the reference's own example measures against
  (examples/dot_product_attention.py:20-43 of HPC-SJTU/af3_kernels): scale q, q k^T, add bias,
  ``masked_fill_(~mask, -1e9)``, softmax, times v.  It is pinned: ``tests/golden`` holds outputs
  of that very function (extracted from the reference's file and executed, see
  tests/golden/make_golden.py) and tests/test_oracle.py checks this restatement against them.

* ``ref_semantics`` (O2): the C restatement in oracle/ref_semantics.c of the reference's C++
  operator with the bf16 rounding points of its TPP sequence
  (src/csrc/dot_product_attention.cpp:88-122, flash branch :148-190).  The reference kernel
  itself cannot be built here (libxsmm is an empty submodule), so O2 is checked against O1 within
  the bf16 error the rounding scheme implies; bit parity with the libxsmm JIT is unpinned.

Also: seeded generators for the five benchmark configurations and the error metrics used by
the tests (max-abs, mean-abs, and the reference example's relative L1,
examples/dot_product_attention.py:129-134).
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Optional

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libaf3k_oracle.so")
_lib = None


# ----------------------------------------------------------------------------- O1
def lift_mask(mask: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """mask -> bool [B|1, 1, 1, S] (True = attend), as examples/dot_product_attention.py:33-37."""
    if mask is None:
        return None
    if mask.dim() == 1:
        return mask[None, None, None, :].to(dtype=torch.bool)
    if mask.dim() == 2:
        return mask[:, None, None, :].to(dtype=torch.bool)
    return mask.to(dtype=torch.bool)


def oracle_fp32(q, k, v, mask, bias, q_scale=None, k_scale=None) -> torch.Tensor:
    """fp32 result on the *stored* inputs: bf16 is widened exactly, fp8 q/k are de-quantised with
    their per-head scales.  Returns fp32 [B1, B2, Sq, D]."""
    qf, kf, vf = q.float(), k.float(), v.float()
    if q_scale is not None:
        qf = qf * q_scale.float().view(1, -1, 1, 1)
        kf = kf * k_scale.float().view(1, -1, 1, 1)
    scaling = q.size(-1) ** -0.5
    logits = torch.matmul(qf * scaling, kf.transpose(-1, -2))
    if bias is not None:
        logits = logits + bias.float().reshape(1, q.shape[1], q.shape[2], k.shape[2])
    m = lift_mask(mask)
    if m is not None:
        logits = logits.masked_fill(~m, -1e9)
    weights = torch.softmax(logits, dim=-1)
    return torch.matmul(weights, vf)


def torch_baseline_bf16(q, k, v, mask, bias) -> torch.Tensor:
    """The same function evaluated in the inputs' own dtype (bf16), as the reference's example
    runs it for its "Torch ms" timing (examples/dot_product_attention.py:20-43, :139-148).  Used
    as a timed CPU baseline only."""
    scaling = q.size(-1) ** -0.5
    logits = torch.matmul(q * scaling, k.transpose(-1, -2))
    logits = logits + bias.to(logits.dtype).reshape(1, q.shape[1], q.shape[2], k.shape[2])
    m = lift_mask(mask)
    if m is not None:
        logits.masked_fill_(~m, -1e9)
    weights = torch.softmax(logits, dim=-1)
    return torch.matmul(weights, v)


# ----------------------------------------------------------------------------- O2
def build_c_oracle(force: bool = False) -> str:
    src = os.path.join(_HERE, "ref_semantics.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(src) > os.path.getmtime(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "-B", "libaf3k_oracle.so"], check=True,
                       capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build_c_oracle()
        lib = ctypes.CDLL(_LIB_PATH)
        f = lib.af3k_oracle_dot_product_attention
        f.restype = ctypes.c_int
        fp = ctypes.c_void_p
        f.argtypes = [fp, fp, fp, fp, fp, ctypes.c_long, fp] + [ctypes.c_int] * 9
        lib.af3k_oracle_num_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def num_threads() -> int:
    return _load().af3k_oracle_num_threads()


def ref_semantics(q, k, v, mask, bias, BLK_SZ: int = 128, use_flash: bool = False,
                  FLASH_SZ: int = 1024, round_bf16: bool = True, threads: int = 0) -> torch.Tensor:
    """Runs the C restatement.  q, k, v [B1, B2, S, D]; bias B2*S*S elements (cast to q.dtype
    first, as src/af3_kernels/__init__.py:48 does); mask 1-D [S], 2-D [B1, S] or None
    (True = attend; a 1-D mask is broadcast over B1).  Returns fp32 (bf16-representable when
    ``round_bf16``)."""
    B1, B2, S, D = q.shape
    cast = (lambda t: t.to(torch.bfloat16).float()) if round_bf16 else (lambda t: t.float())
    qf = cast(q).contiguous().numpy()
    kf = cast(k).contiguous().numpy()
    vf = cast(v).contiguous().numpy()
    bf = cast(bias.reshape(B2, S, S)).contiguous().numpy()
    keep, stride = None, 0
    if mask is not None:
        m = mask.reshape(-1, S) if mask.dim() != 1 else mask[None, :]
        keep = np.ascontiguousarray(m.to(torch.bool).numpy().astype(np.uint8))
        stride = S if keep.shape[0] == B1 and B1 > 1 else (S if B1 == 1 else 0)
    out = np.empty((B1, B2, S, D), dtype=np.float32)
    rc = _load().af3k_oracle_dot_product_attention(
        qf.ctypes.data, kf.ctypes.data, vf.ctypes.data, bf.ctypes.data,
        keep.ctypes.data if keep is not None else None, stride, out.ctypes.data,
        B1, B2, S, D, BLK_SZ, int(use_flash), FLASH_SZ, int(round_bf16), threads)
    if rc != 0:
        raise RuntimeError("C oracle failed")
    return torch.from_numpy(out)


# ----------------------------------------------------------------------------- inputs
CONFIGS = {
    # name: B1, B2, S, D, bias dtype, bias std, mask kind, fp8
    "cfg1": dict(B1=1, B2=16, S=512, D=32, bias_dtype=torch.float32, bias_std=1.0, mask="tail64"),
    "cfg2": dict(B1=768, B2=4, S=768, D=32, bias_dtype=torch.float32, bias_std=1.0, mask="rand05"),
    "cfg3": dict(B1=1, B2=16, S=1536, D=24, bias_dtype=torch.bfloat16, bias_std=2.0, mask="tail128"),
    "cfg4": dict(B1=5, B2=16, S=1536, D=48, bias_dtype=torch.bfloat16, bias_std=1.0, mask="tail96"),
    "cfg5": dict(B1=2048, B2=4, S=2048, D=32, bias_dtype=torch.bfloat16, bias_std=1.0, mask="rand05",
                 fp8=True),
}


def quantize_e4m3_per_head(x: torch.Tensor):
    """x [B1, H, S, D] fp32 -> (float8_e4m3fn tensor, scale [H]) with scale_h = amax_h / 448."""
    amax = x.abs().amax(dim=(0, 2, 3)).clamp_min(1e-12)
    scale = (amax / 448.0).float()
    xq = (x / scale.view(1, -1, 1, 1)).to(torch.float8_e4m3fn)
    return xq, scale


def make_inputs(name: str, rows: Optional[int] = None, seed: int = 0, S: Optional[int] = None):
    """Seeded synthetic inputs of a benchmark configuration (CPU tensors).  Draw order:
    q, k, v, bias, mask.  ``rows`` / ``S`` shrink B1 / the sequence for parity tests."""
    c = dict(CONFIGS[name])
    B1 = rows if rows is not None else c["B1"]
    S = S if S is not None else c["S"]
    B2, D = c["B2"], c["D"]
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B1, B2, S, D, generator=g)
    k = torch.randn(B1, B2, S, D, generator=g)
    v = torch.randn(B1, B2, S, D, generator=g)
    bias = (torch.randn(B2, S, S, generator=g) * c["bias_std"]).to(c["bias_dtype"])
    kind = c["mask"]
    if kind.startswith("tail"):
        n = min(int(kind[4:]), S - 1)
        mask = torch.ones(B1, S, dtype=torch.bool)
        mask[:, S - n:] = False
    else:
        mask = torch.rand(B1, S, generator=g) >= 0.05
    out = dict(v=v.to(torch.bfloat16), bias=bias, mask=mask, q_scale=None, k_scale=None)
    if c.get("fp8"):
        out["q"], out["q_scale"] = quantize_e4m3_per_head(q)
        out["k"], out["k_scale"] = quantize_e4m3_per_head(k)
    else:
        out["q"], out["k"] = q.to(torch.bfloat16), k.to(torch.bfloat16)
    return out


def attention_flops(B1, B2, Sq, Sk, D) -> float:
    return 4.0 * B1 * B2 * Sq * Sk * D


def attention_bytes(B1, B2, Sq, Sk, D, qk_bytes=2, bias_bytes=4, mask_rows=None) -> float:
    """Algorithmic bytes: Q, K, V, O once; bias once; mask one byte per entry."""
    mask_rows = B1 if mask_rows is None else mask_rows
    return (B1 * B2 * (Sq * D * qk_bytes + Sk * D * qk_bytes + Sk * D * 2 + Sq * D * 2)
            + B2 * Sq * Sk * bias_bytes + mask_rows * Sk)


# ----------------------------------------------------------------------------- metrics
def error_stats(out: torch.Tensor, ref: torch.Tensor) -> dict:
    o, r = out.float(), ref.float()
    d = (o - r).abs()
    return {
        "max_abs": d.max().item(),
        "mean_abs": d.mean().item(),
        "rel_l1": (d.sum() / r.abs().sum().clamp_min(1e-30)).item(),
        "nan": int(torch.isnan(o).sum().item()),
    }


# ----------------------------------------------------------------------------- blocks
def pair_bias_fp32(pair, ln_w, ln_b, w_bias, eps=1e-5):
    """fp32 restatement of the two statements in front of the attention core in the reference's
    modules (src/af3_kernels/Attention.py:51-52 and :152-153; the same lines of the PyTorch models
    in examples/grid_self_attention.py): LayerNorm over the channels, then the per-head bias
    projection permuted to [H, R, N].  Returns (normalised pair [R, N, C], bias [H, R, N])."""
    F = torch.nn.functional
    x = F.layer_norm(pair.float(), (pair.shape[-1],), ln_w.float(), ln_b.float(), eps)
    return x, F.linear(x, w_bias.float()).permute(2, 0, 1)


def grid_block_fp32(pair, mask, ln_w, ln_b, w_bias, w_q, w_k, w_v, w_gate, w_out, num_head,
                    transpose=False, eps=1e-5) -> torch.Tensor:
    """fp32 restatement of the reference's PyTorch grid self-attention model
    (examples/grid_self_attention.py:20-96, class AttentionTorch): LayerNorm, pair-bias
    projection, q/k/v projections, biased key-masked attention, sigmoid gate, output projection.
    All weights as ``nn.Linear.weight`` ([out, in]).  pair [N, N, C], mask [N, N] -> [N, N, C]."""
    F = torch.nn.functional
    x, bias = pair_bias_fp32(pair, ln_w, ln_b, w_bias, eps)
    if transpose:
        x = x.permute(1, 0, 2)
    R, N, C = x.shape
    D = C // num_head
    split = lambda t: t.reshape(R, N, num_head, D).permute(0, 2, 1, 3)
    q, k, v = (split(F.linear(x, w.float())) for w in (w_q, w_k, w_v))
    o = oracle_fp32(q, k, v, mask, bias)
    o = o.permute(0, 2, 1, 3).reshape(R, N, C) * torch.sigmoid(F.linear(x, w_gate.float()))
    out = F.linear(o, w_out.float())
    return out.permute(1, 0, 2) if transpose else out


def self_block_fp32(x, mask, pair_logits, w_q, b_q, w_k, w_v, w_gate, num_head) -> torch.Tensor:
    """fp32 restatement of the reference's PyTorch single / diffusion attention model
    (examples/self_attention.py:23-96, class AttentionTorch).  x [N, C], mask [N],
    pair_logits [H, N, N] -> [N, C]."""
    F = torch.nn.functional
    xf = x.float()
    N, C = xf.shape
    D = C // num_head
    split = lambda t: t.reshape(N, num_head, D).permute(1, 0, 2).unsqueeze(0)
    q = split(F.linear(xf, w_q.float(), b_q.float()))
    k = split(F.linear(xf, w_k.float()))
    v = split(F.linear(xf, w_v.float()))
    o = oracle_fp32(q, k, v, mask, pair_logits)
    o = o.squeeze(0).permute(1, 0, 2).reshape(N, C)
    return o * torch.sigmoid(F.linear(xf, w_gate.float()))
