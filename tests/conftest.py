import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected with -m 'not gpu'")


def _from_bits(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.int16:
        return torch.from_numpy(a.copy()).view(torch.bfloat16)
    return torch.from_numpy(a.copy())


@pytest.fixture(scope="session")
def golden():
    """{case name: dict(q, k, v, bias, mask|None, ref_fp32, ref_bf16)} from tests/golden."""
    z = np.load(os.path.join(ROOT, "tests", "golden", "dpa_golden.npz"))
    cases = {}
    for key in z.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = z[key]
    out = {}
    for name, f in cases.items():
        out[name] = dict(
            q=_from_bits(f["q"]), k=_from_bits(f["k"]), v=_from_bits(f["v"]),
            bias=_from_bits(f["bias"]),
            mask=torch.from_numpy(f["mask"].copy()) if "mask" in f else None,
            ref_fp32=torch.from_numpy(f["ref_fp32"].copy()),
            ref_bf16=_from_bits(f["ref_bf16"]),
        )
    return out


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
