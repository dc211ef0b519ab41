import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def bi():
    import mlx_batch_invariant_b200 as m

    return m


@pytest.fixture(scope="session", autouse=True)
def _final_device_status():
    """After the whole session: no kernel may have given up a bounded wait."""
    yield
    import torch

    if torch.cuda.is_available():
        import mlx_batch_invariant_b200 as m

        m.check_device_status()
