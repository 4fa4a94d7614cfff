"""The C-ABI library loads and exports every symbol include/krn_b200.h declares; entry points refuse bad
arguments and, without a GPU, fail loudly instead of computing anything. CPU only."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from krn_b200.hw import Libraries, LibraryNotFound, LoadedLibrary
from krn_b200.hw.libraries import KERNEL_LIBRARY
from krn_b200.runtime import native

ROOT = Path(__file__).resolve().parent.parent


def declared() -> list[str]:
    text = (ROOT / "include" / "krn_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(krn_b200_\w+)\s*\(", text)


def test_header_symbols_are_all_exported_and_bound() -> None:
    names = declared()
    assert len(names) >= 9 and len(set(names)) == len(names)
    handle = Libraries.load(KERNEL_LIBRARY).handle
    for name in names:
        assert getattr(handle, name) is not None, name
    assert set(native.PROTOTYPES) == set(names)


def test_version_and_error_text() -> None:
    handle = native.library()
    assert handle.krn_b200_version() == native.ABI_VERSION
    status = handle.krn_b200_gemm_tn(native.BF16, native.BF16, None, None, None, 128, 128, 128, 128, 128, 128, None)
    assert status == native.ERR_INVALID_ARGUMENT
    assert "null" in native.last_error()
    status = handle.krn_b200_gemm_tn(native.E4M3, native.BF16, 16, 16, 16, 128, 128, 128, 128, 128, 128, None)
    assert status == native.ERR_UNSUPPORTED
    with pytest.raises(Exception) as error:
        native.check(status, "tile matrix product")
    assert "is not available on sm_100a" in str(error.value) and "Instead:" in str(error.value)


def test_no_cpu_fallback() -> None:
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    handle = native.library()
    status = handle.krn_b200_gemm_tn(native.BF16, native.BF16, 16, 16, 16, 128, 128, 128, 128, 128, 128, None)
    assert status == native.ERR_CUDA
    with pytest.raises(Exception, match="KRN_B200_ERR_CUDA"):
        native.check(status, "tile matrix product")


def test_libraries_loader_contract(tmp_path: Path) -> None:
    """Absolute paths are tried as given and nowhere else; failures are cached until clear_cache
    (src/krn/hw/libraries.py:324-377, tests/hw/test_libraries.py)."""
    loaded = Libraries.load(KERNEL_LIBRARY)
    assert isinstance(loaded, LoadedLibrary) and loaded.path.is_absolute() and isinstance(loaded.handle, ctypes.CDLL)
    assert Libraries.load(KERNEL_LIBRARY) is loaded
    assert Libraries.find(KERNEL_LIBRARY) == loaded.path and Libraries.available(KERNEL_LIBRARY)
    missing = str(tmp_path / "libnothing.so")
    with pytest.raises(LibraryNotFound) as error:
        Libraries.load(missing)
    assert error.value.names == (missing,) and missing in str(error.value) and "Fix:" in str(error.value)
    assert not Libraries.available(missing) and Libraries.find(missing) is None
    (tmp_path / "libnothing.so").write_bytes(Path(loaded.path).read_bytes())
    assert not Libraries.available(missing)  # the failure is cached
    Libraries.clear_cache()
    assert Libraries.available(missing)
    Libraries.clear_cache()


def test_ctypes_cdll_is_called_in_one_place_only() -> None:
    """All native loads are centralised in hw/libraries.py (tests/hw/test_libraries.py:238-242)."""
    offenders = [path for path in (ROOT / "krn_b200").rglob("*.py")
                 if "CDLL(" in path.read_text() and path.name != "libraries.py"]
    assert offenders == []
