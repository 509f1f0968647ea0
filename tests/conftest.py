import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


import __graft_entry__ as _ge  # noqa: E402

_ge.package()  # registers the hyphen-named package directory as `fish_audio_cpp_b200`


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as ge

    if not (ge.PKG_DIR / "lib" / "libw8a8.so").exists():
        ge.build()
    return ge.package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o

    o.build()
    return o


@pytest.fixture(scope="session")
def ctx(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    torch.cuda.set_device(0)
    c = pkg.Context(0, 0)
    yield c
    c.close()
