"""Shared fixtures: golden-vector loader and the `gpu` marker."""

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
GOLDEN_CASES = ["d128_fp32_k3v2", "d128_bf16_k3v2", "d256_bf16_k3v2", "d128_bf16_k4v4", "d128_fp16_k3v2"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """One golden case as torch tensors (bf16 restored from its uint16 bits)."""

    def __init__(self, name: str):
        z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
        self.name = name
        (self.D, self.H, self.Qh, self.T, self.ring, self.key_bits, self.value_bits,
         self.layer, self.seed) = [int(v) for v in z["meta"]]
        self.dtype = getattr(torch, str(z["dtype"]))
        self.raw = {}
        for k in z.files:
            a = z[k]
            if k.endswith("_bf16"):
                self.raw[k[:-5]] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
            elif a.dtype.kind in "fiu" and a.ndim > 0 and k not in ("meta",):
                self.raw[k] = torch.from_numpy(a.copy())
        self.memory_bytes = int(z["memory_bytes"])

    def __getattr__(self, k):
        try:
            return self.__dict__["raw"][k]
        except KeyError:
            raise AttributeError(k)

    @property
    def mse_bits(self):
        return self.key_bits - 1


@pytest.fixture(params=GOLDEN_CASES)
def golden(request):
    return Golden(request.param)


def load_golden(name: str) -> Golden:
    return Golden(name)
