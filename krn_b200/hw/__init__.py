"""Hardware-facing helpers of the B200 path: the native library loader."""

from krn_b200.hw.libraries import Libraries, LibraryNotFound, LoadedLibrary

__all__ = ["Libraries", "LibraryNotFound", "LoadedLibrary"]
