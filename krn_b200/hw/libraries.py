"""Cached native library loading: the one place in the package where `ctypes.CDLL` is called.

Mirrors the reference's loader (src/krn/hw/libraries.py:32-45,324-377): `Libraries.load(name)` returns a
frozen `LoadedLibrary(name, path, handle, source)`, an absolute path is tried as given and nowhere else,
results — failures included — are cached until `clear_cache()`, and a failure is a `LibraryNotFound` that
lists every name and place tried together with a fix. The registry here knows one logical name,
`"krn_b200"`: the prebuilt sm_100a kernel library, looked for at `$KRN_B200_LIB` and then beside the package.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from functools import cache
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent.parent
KERNEL_LIBRARY = "krn_b200"
KERNEL_LIBRARY_FILE = "libkrn_b200.so"


class HardwareError(RuntimeError):
    """A hardware-layer failure with the step that fixes it (src/krn/hw/exceptions.py)."""

    def __init__(self, message: str, fix: str) -> None:
        self.fix = fix
        super().__init__(f"{message}. Fix: {fix}")


@dataclass(frozen=True, kw_only=True)
class LoadedLibrary:
    name: str
    path: Path
    handle: ctypes.CDLL
    source: str


class LibraryNotFound(HardwareError):
    """All attempted names and search locations, including loader errors."""

    def __init__(self, name: str, names: tuple[str, ...], places: tuple[str, ...], fix: str) -> None:
        self.name, self.names, self.places = name, names, places
        super().__init__(f"Library {name!r} unavailable; names: {', '.join(names)}; tried: {'; '.join(places)}", fix)


def _candidates(name: str) -> tuple[tuple[str, ...], str, str]:
    """(paths or sonames to try in order, source label, fix text)."""
    if Path(name).is_absolute():
        return (name,), "soname", "Check the path; build the kernel library with `python -m krn_b200.csrc.build`"
    if name == KERNEL_LIBRARY:
        places = []
        if os.environ.get("KRN_B200_LIB"):
            places.append(os.environ["KRN_B200_LIB"])
        places.append(str(PACKAGE_DIR / KERNEL_LIBRARY_FILE))
        return tuple(places), "package", "Build it with `python -m krn_b200.csrc.build` (needs nvcc), or set KRN_B200_LIB"
    return (name,), "soname", "Install the system runtime that provides it"


class Libraries:
    """Process-wide flyweights; failures persist until clear_cache is called."""

    @staticmethod
    @cache
    def _result(name: str) -> LoadedLibrary | LibraryNotFound:
        candidates, source, fix = _candidates(name)
        tried = []
        for candidate in candidates:
            try:
                handle = ctypes.CDLL(candidate)
            except OSError as error:
                tried.append(f"{candidate}: {error}")
                continue
            return LoadedLibrary(name=name, path=Path(candidate), handle=handle, source=source)
        return LibraryNotFound(name, candidates, tuple(tried), fix)

    @staticmethod
    def load(name: str) -> LoadedLibrary:
        result = Libraries._result(name)
        if isinstance(result, LibraryNotFound):
            raise result
        return result

    @staticmethod
    @cache
    def _find(name: str) -> Path | None:
        candidates, _, _ = _candidates(name)
        return next((Path(p) for p in candidates if Path(p).is_absolute() and Path(p).is_file()), None)

    @staticmethod
    def find(name: str) -> Path | None:
        """Locate without executing native code."""
        return Libraries._find(name)

    @staticmethod
    def available(name: str) -> bool:
        return isinstance(Libraries._result(name), LoadedLibrary)

    @staticmethod
    def clear_cache() -> None:
        Libraries._result.cache_clear()
        Libraries._find.cache_clear()
