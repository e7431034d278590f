import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
# children started with the "spawn" method import the test modules by name
os.environ["PYTHONPATH"] = ROOT + os.pathsep + os.path.join(ROOT, "tests") + os.pathsep + os.environ.get("PYTHONPATH", "")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs at least one CUDA device (run on a B200 box)")


@pytest.fixture(autouse=True)
def _restore_config():
    import jaxdecomp_b200 as jd

    snap = {k: getattr(jd.config, k) for k in ("transpose_axis_contiguous", "backend", "reference_compat_halo_grad")}
    yield
    for k, v in snap.items():
        setattr(jd.config, k, v)
