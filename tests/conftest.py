"""Shared fixtures: marker registration, golden-fixture loading, oracle access."""
import os
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def from_f16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.float16))


def load_packed(z, prefix: str):
    """Rebuild a PackedTensor-shaped object from a fixture written by make_golden.py."""
    meta = [int(v) for v in z[f"{prefix}.meta"]]
    return SimpleNamespace(
        packed=torch.from_numpy(z[f"{prefix}.packed"]), scale=from_f16(z[f"{prefix}.scale"]),
        mins=from_f16(z[f"{prefix}.mins"]), bits=meta[0], axis=meta[1], group_size=meta[2],
        axis_len=meta[3], orig_shape=tuple(meta[4:]))


@pytest.fixture(scope="session")
def golden():
    def _load(name):
        return np.load(os.path.join(GOLDEN, name))
    return _load


@pytest.fixture(scope="session")
def oracle():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import pkv_oracle
    return pkv_oracle


def attention_close(out: torch.Tensor, ref: torch.Tensor, atol=2e-3, rel=1e-2):
    """The parity bar of the decode path: max-abs <= 2e-3 and max-abs / max|ref| <= 1e-2."""
    d = (out.float().cpu() - ref.float().cpu()).abs().max().item()
    scale = ref.float().abs().max().item()
    assert d <= atol, f"max-abs {d:.3e} > {atol}"
    assert d <= rel * max(scale, 1e-12), f"max-abs {d:.3e} > {rel} * max|ref| {scale:.3e}"
    return d
