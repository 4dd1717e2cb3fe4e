import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden" / "packages"
PACKAGES = ["cfg1_bf16_mtp", "tiny_int4_mtp", "tiny_int4_mtp_v16", "tiny_fp8_mtp", "tiny_moe_fp8_mtp"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
