import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle binding (builds liboracle.so on first use)."""
    from oracle import binding
    binding.build()
    return binding


@pytest.fixture(scope="session")
def kats():
    import json
    return json.loads((ROOT / "tests" / "golden" / "reference_kats.json").read_text())


@pytest.fixture(scope="session")
def backend():
    """The device backend through the C ABI. Fails loudly (no skip) when the library cannot run."""
    from vibe_compiler_b200.backend import B200TargetModelBackend
    return B200TargetModelBackend(int(os.environ.get("LOCAL_RANK", "0")))
