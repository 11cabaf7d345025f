import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    orc.lib()
    return orc


@pytest.fixture(scope="session")
def ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import hesper_b200
    c = hesper_b200.Context(0)
    yield c
    c.check()
    c.close()


@pytest.fixture(scope="session")
def ctx_mv():
    """A context that sends every one-token k-quant matvec that fits to the mma.sync kernel
    (HB200_MV=2 is read when the context is created), so its prologue / epilogue variants are
    covered at small shapes too."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import hesper_b200
    old = os.environ.get("HB200_MV")
    os.environ["HB200_MV"] = "2"
    try:
        c = hesper_b200.Context(0)
    finally:
        if old is None:
            del os.environ["HB200_MV"]
        else:
            os.environ["HB200_MV"] = old
    yield c
    c.check()
    c.close()
