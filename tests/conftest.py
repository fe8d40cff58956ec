import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_rows():
    import json
    import numpy as np
    with open(os.path.join(ROOT, "tests", "golden", "quant_rows.json")) as f:
        doc = json.load(f)
    rows = []
    for r in doc["rows"]:
        rows.append({
            "encoding": r["encoding"],
            "name": r["name"],
            "bytes": np.frombuffer(bytes.fromhex(r["bytes_hex"]), dtype=np.uint8).copy(),
            "values": np.frombuffer(bytes.fromhex(r["values_f32le_hex"]), dtype="<f4").copy(),
        })
    return rows
