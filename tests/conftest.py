import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as g
    g.build()
    return g.load_package()


@pytest.fixture(scope="session")
def synth(pkg):
    from llama2_jl_b200 import synth as s
    return s


@pytest.fixture(scope="session")
def orc(pkg):
    import oracle_binding
    return oracle_binding
