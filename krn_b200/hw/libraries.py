"""The one module of the package that opens shared libraries (`ctypes.CDLL` is called here and nowhere else).

The public surface is the reference loader's (src/krn/hw/libraries.py:32-45,324-377), because host code and tests
are written against it:

* `Libraries.load(name)` gives a `LoadedLibrary(name, path, handle, source)` or raises `LibraryNotFound`;
  the same object comes back on every later call, and a failure is remembered too, until `clear_cache()`.
* An absolute path is opened exactly as given and nothing else is searched.
* `Libraries.find(name)` only looks at the file system; `Libraries.available(name)` actually loads.
* `LibraryNotFound` carries `name`, `names` (what was asked of the loader) and `places` (each attempt with the
  loader's complaint), and its text ends in a `Fix:` sentence.

This package knows one logical name, `"krn_b200"`: the prebuilt sm_100a kernel library. It is looked for at
`$KRN_B200_LIB` when that is set, then next to the package directory. Any other relative name is handed to the
system loader unchanged.
"""

from __future__ import annotations

import ctypes
import os
import threading
from dataclasses import dataclass
from pathlib import Path
from typing import NamedTuple

PACKAGE_DIR = Path(__file__).resolve().parents[1]
KERNEL_LIBRARY = "krn_b200"
KERNEL_LIBRARY_FILE = "libkrn_b200.so"


class HardwareError(RuntimeError):
    """Something at the hardware boundary failed; `fix` says what the user can do about it
    (src/krn/hw/exceptions.py)."""

    def __init__(self, message: str, fix: str) -> None:
        super().__init__(f"{message}. Fix: {fix}")
        self.fix = fix


@dataclass(frozen=True, kw_only=True)
class LoadedLibrary:
    """An opened shared library: the name it was asked for by, the file it came from, the ctypes handle and which
    search rule found it (`"package"` for the kernel library, `"soname"` for everything else)."""

    name: str
    path: Path
    handle: ctypes.CDLL
    source: str


class LibraryNotFound(HardwareError):
    """No attempt to open the library succeeded. `names` lists what was tried, `places` pairs each try with the
    dynamic loader's message."""

    def __init__(self, name: str, names: tuple[str, ...], places: tuple[str, ...], fix: str) -> None:
        listing = f"names: {', '.join(names)}; tried: {'; '.join(places)}"
        super().__init__(f"Library {name!r} unavailable; {listing}", fix)
        self.name = name
        self.names = names
        self.places = places


class _Search(NamedTuple):
    """How one name is resolved: the strings handed to the loader in order, the label recorded on success and the
    advice attached to a failure."""

    attempts: tuple[str, ...]
    source: str
    fix: str


def _search_for(name: str) -> _Search:
    if os.path.isabs(name):
        return _Search((name,), "soname", "Check the path; build the kernel library with `python -m krn_b200.csrc.build`")
    if name != KERNEL_LIBRARY:
        return _Search((name,), "soname", "Install the system runtime that provides it")
    override = os.environ.get("KRN_B200_LIB")
    beside_package = str(PACKAGE_DIR / KERNEL_LIBRARY_FILE)
    attempts = (override, beside_package) if override else (beside_package,)
    return _Search(attempts, "package", "Build it with `python -m krn_b200.csrc.build` (needs nvcc), or set KRN_B200_LIB")


class Libraries:
    """Process-wide registry of opened libraries. Successes and failures are both kept, so a missing library is
    diagnosed once and every later caller gets the same answer until `clear_cache()`."""

    _lock = threading.Lock()
    _outcomes: dict[str, LoadedLibrary | LibraryNotFound] = {}
    _locations: dict[str, Path | None] = {}

    @classmethod
    def _open(cls, name: str) -> LoadedLibrary | LibraryNotFound:
        search = _search_for(name)
        complaints: list[str] = []
        for attempt in search.attempts:
            try:
                return LoadedLibrary(name=name, path=Path(attempt), handle=ctypes.CDLL(attempt), source=search.source)
            except OSError as error:
                complaints.append(f"{attempt}: {error}")
        return LibraryNotFound(name, search.attempts, tuple(complaints), search.fix)

    @classmethod
    def _outcome(cls, name: str) -> LoadedLibrary | LibraryNotFound:
        with cls._lock:
            if name not in cls._outcomes:
                cls._outcomes[name] = cls._open(name)
            return cls._outcomes[name]

    @classmethod
    def load(cls, name: str) -> LoadedLibrary:
        """Open `name` (once) and return its record; raises the remembered `LibraryNotFound` otherwise."""
        outcome = cls._outcome(name)
        if isinstance(outcome, LibraryNotFound):
            raise outcome
        return outcome

    @classmethod
    def find(cls, name: str) -> Path | None:
        """Where the library's file is, judged from the file system alone: no native code runs."""
        with cls._lock:
            if name not in cls._locations:
                files = (Path(p) for p in _search_for(name).attempts if os.path.isabs(p))
                cls._locations[name] = next((f for f in files if f.is_file()), None)
            return cls._locations[name]

    @classmethod
    def available(cls, name: str) -> bool:
        """True when `load(name)` would succeed (this loads the library)."""
        return isinstance(cls._outcome(name), LoadedLibrary)

    @classmethod
    def clear_cache(cls) -> None:
        """Forget every remembered success, failure and location."""
        with cls._lock:
            cls._outcomes.clear()
            cls._locations.clear()
