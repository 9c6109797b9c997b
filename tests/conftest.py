import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "ins-conv_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_sessionstart(session):
    """Builds the native parts when they are missing or older than their sources (a no-op otherwise), so that a fresh
    checkout can run the suite; a failed build is reported by the tests that load the library."""
    try:
        import importlib.util
        spec = importlib.util.spec_from_file_location("insconv_build", os.path.join(ROOT, "ins-conv_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_all()
    except Exception as e:  # noqa: BLE001
        sys.stderr.write("native build skipped: %s\n" % (e,))


def pytest_collection_modifyitems(config, items):
    # files named test_zz_* run last
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz_"),))


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device; the library has no CPU fallback")
    return torch.device("cuda:0")
