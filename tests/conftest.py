import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")

# Parity tolerances stated by the benchmark contract: bf16 output max-abs error and LSE
# relative error against the fp32 oracle.
OUT_ATOL = 2e-2
LSE_RTOL = 1e-3


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN_DIR
