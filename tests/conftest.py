import json
import os
import struct
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_cuda() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle module (C library built on demand)."""
    from oracle import shrew_oracle
    shrew_oracle.build()
    return shrew_oracle


def load_golden():
    with open(os.path.join(ROOT, "tests", "golden", "quantize_golden.json")) as f:
        cases = json.load(f)["cases"]
    out = []
    for c in cases:
        data = np.array([struct.unpack("<f", struct.pack("<I", b))[0] for b in c["data_f32_bits"]],
                        dtype=np.float32).reshape(c["shape"])
        scales = np.array([struct.unpack("<d", struct.pack("<Q", b))[0] for b in c["scales_f64_bits"]],
                          dtype=np.float64)
        codes = np.array(c["codes"], dtype=np.int8).reshape(c["shape"])
        out.append(dict(name=c["name"], data=data, scales=scales, codes=codes,
                        granularity=1 if c["granularity"] == "per_channel" else 0, shape=c["shape"]))
    return out


GOLDEN = load_golden()


@pytest.fixture(scope="session")
def golden_cases():
    return GOLDEN
