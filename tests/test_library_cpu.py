"""Host-side checks that need no GPU: the library loads, exports what the header declares, and
fails loudly (never falls back) when no device is present."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols(header: Path):
    text = header.read_text()
    return sorted(set(re.findall(r"W8A8_API\s+[\w\s\*]+?\b(w8a8_\w+)\s*\(", text)))


def test_header_symbols_are_exported(pkg):
    lib = pkg.load_library()
    names = declared_symbols(ROOT / "include" / "w8a8.h")
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/w8a8.h but not exported"
    from fish_audio_cpp_b200 import capi

    assert set(capi.EXPORTS) <= set(names)
    host = declared_symbols(ROOT / "include" / "w8a8_container.h")
    assert len(host) == 8 and set(capi.CONTAINER_EXPORTS) == set(host)
    for n in host:
        assert hasattr(lib, n), f"{n} declared in include/w8a8_container.h but not exported"


def test_shim_exports_reference_signatures(pkg):
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", str(pkg.library_path())], capture_output=True,
                         text=True, check=True).stdout
    for sig in ["fish::kernels::int8_dequant_gemm_fp16(signed char const*, __half const*, int, __half const*, "
                "__half const*, __half const*, __half*, int, int, int, cublasContext*, CUstream_st*)",
                "fish::kernels::rms_norm(__half const*, __half const*, __half*, int, int, float, CUstream_st*)",
                "fish::kernels::silu_forward(__half*, int, CUstream_st*)",
                "fish::kernels::mul_forward(__half*, __half const*, int, CUstream_st*)",
                "fish::kernels::residual_add(__half*, __half const*, int, CUstream_st*)"]:
        assert sig in out, sig


def test_status_strings_and_workspace_arithmetic(pkg):
    lib = pkg.load_library()
    assert lib.w8a8_status_string(0) == b"ok"
    assert b"workspace" in lib.w8a8_status_string(5)
    # codes M*K (256-aligned) + scales M*G*4 (256-aligned)
    assert lib.w8a8_workspace_bytes(100, 64, 512, 64) == 51200 + 3328
    assert lib.w8a8_workspace_bytes(0, 64, 512, 64) == 0
    assert pkg.num_groups(2560, 256) == 10 and pkg.num_groups(2560, 0) == 1 and pkg.num_groups(100, 64) == 2


def test_no_silent_fallback_without_a_device(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(pkg.W8A8Error) as e:
        pkg.Context(0, 1 << 20)
    assert e.value.status == 3  # W8A8_ERR_CUDA


def test_null_context_is_rejected(pkg):
    lib = pkg.load_library()
    assert lib.w8a8_linear(None, None, None, 64, None, None, None, None, 1, 8, 64, None, None) == 1
    assert b"context" in lib.w8a8_last_error()
    assert lib.w8a8_destroy(None) == 0


def test_product_never_touches_the_oracle():
    """Nothing under the package may import, link or read oracle/ (checker only)."""
    pat = re.compile(r"(^|\s)(import|from)\s+oracle\b|oracle/|w8a8o_|libw8a8_oracle|fishref")
    for p in list((ROOT / "fish-audio-cpp_b200").rglob("*")) + list((ROOT / "include").glob("*.h")):
        if p.suffix in {".py", ".cu", ".h", ".cuh"}:
            assert not pat.search(p.read_text()), p
