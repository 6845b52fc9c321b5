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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """npz fixture -> {case: {key: np.ndarray}}"""
    z = np.load(os.path.join(GOLDEN, name))
    out = {}
    for k in z.files:
        case, key = k.split("/")
        out.setdefault(case, {})[key] = z[k]
    return out


def as_fp8(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)


def as_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


DT = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}


def golden_tensor(a: np.ndarray, code: int) -> torch.Tensor:
    if code == 0:
        return as_bf16(a)
    return torch.from_numpy(a.copy())


def make_activation(M, K, seed, dtype=torch.bfloat16, outliers=True):
    """N(0,1) activations with 1% outlier channels scaled x20 (CPU, seeded)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    if outliers and K >= 100:
        idx = torch.randperm(K, generator=g)[: (K + 99) // 100]
        x[:, idx] *= 20
    return x.to(dtype)


def make_weight(N, K, seed):
    """N(0, 0.02^2) weight, block-quantised 128x128 by the oracle's weight quantiser."""
    import oracle as O

    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    return O.block_quant_weight_fp8(w, (128, 128))
