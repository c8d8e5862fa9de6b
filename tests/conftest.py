import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # GPU tests are selected with `-m gpu`; without a device they are skipped, never silently passed.
    try:
        import torch
        has_cuda = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def reference_vectors():
    """The two known-answer vectors of the reference test-suite, as fp16 numpy arrays."""
    with open(os.path.join(GOLDEN_DIR, "reference_test_vectors.json")) as f:
        doc = json.load(f)
    cases = []
    for c in doc["cases"]:
        cases.append({
            "name": c["name"],
            "dense": np.array(c["dense"], dtype=np.float16),
            "values": np.array(c["values"], dtype=np.float16),
            "deltas": np.array(c["deltas"], dtype=np.uint8),
            "row_indices": np.array(c["row_indices"], dtype=np.int32),
            "rows": c["rows"],
            "cols": c["cols"],
        })
    return cases


@pytest.fixture(scope="session")
def reference_cases():
    """Fixtures produced by the compiled reference compressor (tests/golden/make_golden.py)."""
    z = np.load(os.path.join(GOLDEN_DIR, "reference_cases.npz"))
    names = sorted({k.split("/")[0] for k in z.files})
    return [
        {
            "name": n,
            "dense": z[f"{n}/dense"],
            "values": z[f"{n}/values"],
            "deltas": z[f"{n}/deltas"],
            "row_indices": z[f"{n}/row_indices"],
        }
        for n in names
    ]


@pytest.fixture(scope="session")
def reference_cases_int8():
    """Fixtures produced by the compiled reference int8 encoder (tests/golden/make_golden.py)."""
    z = np.load(os.path.join(GOLDEN_DIR, "reference_cases_int8.npz"))
    names = sorted({k.split("/")[0] for k in z.files})
    return [
        {
            "name": n,
            "dense": z[f"{n}/dense"],
            "values": z[f"{n}/values"],
            "deltas": z[f"{n}/deltas"],
            "row_indices": z[f"{n}/row_indices"],
        }
        for n in names
    ]
