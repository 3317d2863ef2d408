import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
for entry in (REPO, REPO / "trinity-be_b200"):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def golden():
    import torch
    return torch.load(REPO / "tests" / "golden" / "reference_eval.pt")
