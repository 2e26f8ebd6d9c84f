import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# device status word is checked after every decode call in the tests
os.environ.setdefault("INFER_B200_CHECK", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import json
    with open(ROOT / "tests" / "golden" / "golden.json") as f:
        return json.load(f)
