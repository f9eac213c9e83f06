"""Shared test setup: import paths, the `gpu` marker, fixtures for the golden vectors."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "sageattention-rdna4_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


GOLDEN = os.path.join(ROOT, "tests", "golden", "quant_golden.npz")
GOLDEN_CASES = ["f16_n1", "f16_n65", "f16_n136", "f16_n70_nosmooth", "bf16_n40", "bf16_n136"]


def _from_bits(arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if dtype in (torch.float16, torch.bfloat16):
        return t.view(dtype)
    if dtype == torch.float8_e4m3fn:
        return t.view(dtype)
    return t


class GoldenCase:
    """One stored case: inputs, the reference checkers' vectors, the oracle's vectors."""

    def __init__(self, z, name):
        self.name = name
        b, h, n, is_bf16, causal, smooth = (int(x) for x in z[name + "/meta"])
        self.B, self.H, self.N = b, h, n
        self.dtype = torch.bfloat16 if is_bf16 else torch.float16
        self.causal, self.smooth = bool(causal), bool(smooth)
        self.int8 = not is_bf16
        code = torch.int8 if self.int8 else torch.float8_e4m3fn
        g = lambda key: z[name + "/" + key]
        self.q = _from_bits(g("q"), self.dtype)
        self.k = _from_bits(g("k"), self.dtype)
        self.v = _from_bits(g("v"), self.dtype)
        self.ref_k8 = _from_bits(g("ref_k8"), code)
        self.ref_sk = _from_bits(g("ref_sk"), torch.float32)
        self.ref_v8 = _from_bits(g("ref_v8"), torch.float8_e4m3fn)
        self.ref_sv = _from_bits(g("ref_sv"), torch.float32)
        self.ref_S = _from_bits(g("ref_S"), torch.float32)               # the reference's fold_v_scale
        self.ref_svfold = _from_bits(g("ref_svfold"), torch.float32)     # (B*H, N_pad), sv / S
        self.ora = {}
        for key, dt in (("q8", code), ("sq", torch.float32), ("k8", code), ("sk", torch.float32),
                        ("v8", torch.float8_e4m3fn), ("sv", torch.float32), ("svp", torch.float32),
                        ("S", torch.float32)):
            self.ora[key] = _from_bits(g("ora_" + key), dt)
        self.ora["mean"] = _from_bits(g("ora_mean"), torch.float32) if self.smooth else None
        self.out128 = _from_bits(g("ora_out128"), self.dtype)
        self.out64 = _from_bits(g("ora_out64"), self.dtype)


@pytest.fixture(scope="session")
def golden_file():
    return np.load(GOLDEN)


@pytest.fixture(params=GOLDEN_CASES)
def golden(request, golden_file):
    return GoldenCase(golden_file, request.param)


def bytes_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bit-for-bit comparison that also works for fp8 tensors."""
    a, b = a.contiguous().cpu(), b.contiguous().cpu()
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return torch.equal(a.view(torch.uint8), b.view(torch.uint8))
