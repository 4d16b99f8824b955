import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device; run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np

    z = np.load(ROOT / "tests" / "golden" / "reference_vectors.npz")
    cases = json.loads(bytes(z["cases_json"]).decode())
    return z, cases


@pytest.fixture(scope="session")
def ctx():
    """One decxb context on cuda:0 for the whole GPU session; fails loudly without the library."""
    import backup_1_b200 as b

    c = b.Context(0)
    c.set_wait_limit_ms(1000)
    yield c
    c.close()
