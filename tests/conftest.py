import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def load_golden(name: str) -> dict:
    """Loads a fixture written by tests/golden/make_golden.py; fp8 / bf16
    arrays come back as torch tensors of the right dtype."""
    z = np.load(os.path.join(GOLDEN, name))
    out = {}
    for k in z.files:
        a = z[k]
        if a.dtype == np.uint8:
            out[k] = torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)
        elif a.dtype == np.uint16:
            out[k] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        elif a.ndim == 0:
            out[k] = float(a)
        else:
            out[k] = torch.from_numpy(a.copy())
    return out


def load_golden16(name: str, dtype: torch.dtype):
    """A gemm_alpha_beta fixture whose a, b, c and out are all stored as raw 16-bit patterns of `dtype`
    (float16 or bfloat16): returns (a, b, c, out, alpha, beta)."""
    z = np.load(os.path.join(GOLDEN, name))
    t = [torch.from_numpy(z[k].view(np.int16).copy()).view(dtype) for k in ("a", "b", "c", "out")]
    return (*t, float(z["alpha"]), float(z["beta"]))


@pytest.fixture(scope="session")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
