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


def pytest_terminal_summary(terminalreporter):
    """How many fp16 outputs passed only through the re-ordering clause of tests/test_gpu_parity.py
    (neither within 2 ulp nor within 2e-3 relative of the oracle, but within what re-associating the same
    fp32 sum can move them): per case label, elements compared and elements that needed the clause."""
    mod = sys.modules.get("test_gpu_parity") or sys.modules.get("tests.test_gpu_parity")
    stats = getattr(mod, "REORDER_STATS", None) if mod else None
    if not stats:
        return
    total = sum(v[0] for v in stats.values())
    third = sum(v[1] for v in stats.values())
    terminalreporter.write_line(f"re-ordering clause: {third} of {total} fp16 outputs needed it "
                                f"({third / max(total, 1):.2e}); cases that did:")
    for k, (n, t) in sorted(stats.items()):
        if t:
            terminalreporter.write_line(f"  {k}: {t} of {n}")
