import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def golden_block_mask():
    import json
    return json.loads((ROOT / "tests" / "golden" / "block_mask_known_answers.json").read_text())


MASKS = {
    "causal": lambda b, h, q, k: q >= k,
    "mod3": lambda b, h, q, k: (q + k) % 3 == 0,
    "parity": lambda b, h, q, k: (q + k) % 2 == 0,
    "block_band2": lambda b, h, q, k: (k // 2 >= q // 2) & (k // 2 <= q // 2 + 1),
}


@pytest.fixture(scope="session")
def named_masks():
    return MASKS


@pytest.fixture(autouse=True)
def _device_status_is_clean(request):
    """After every GPU test: no kernel may have given up a bounded wait (the status word the kernels
    write instead of hanging).  A test that provokes a time-out on purpose reads the word itself."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from jaxmodules_b200 import attention as A
    code = A.device_status()          # the current device: the one the single-process tests run on
    assert code == 0, f"a kernel reported status {code} during {request.node.name}"
