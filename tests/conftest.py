import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    import __graft_entry__ as ge
    return ge.load_oracle()


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="session")
def ops(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    from distributed_xfold_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="session")
def golden():
    import torch
    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.pt"), weights_only=False)
