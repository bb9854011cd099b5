import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qwen3-triton_b200"
for p in (str(PKG), str(ROOT), str(ROOT / "tests" / "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_ops():
    import numpy as np
    data = np.load(ROOT / "tests" / "golden" / "ops.npz")
    return {k: torch.from_numpy(data[k]) for k in data.files}


@pytest.fixture(scope="session")
def golden_tiny():
    import numpy as np
    data = np.load(ROOT / "tests" / "golden" / "tiny_model.npz")
    return {k: torch.from_numpy(data[k]) for k in data.files}


@pytest.fixture(autouse=True)
def _l2_log(request):
    """With Q3_TEST_L2_LOG=<file>, append the largest relative L2 distance each test measured through helpers.close."""
    import helpers
    helpers.l2_seen.clear()
    yield
    path = helpers.l2_log_path()
    if path and helpers.l2_seen:
        what, worst = max(helpers.l2_seen, key=lambda t: t[1])
        over = [w for w, _ in helpers.l2_seen if " OVER " in w]
        with open(path, "a") as fh:
            fh.write(f"{worst:.3e}\t{request.node.nodeid}\t{what}\t{';'.join(over)}\n")


@pytest.fixture(autouse=True)
def _status_clean():
    """After every GPU test the device status word must be clean (no out-of-range id, no timed-out wait)."""
    yield
    if torch.cuda.is_available():
        from qwen3_triton import _abi
        if _abi._status:
            assert _abi.read_status() == 0
