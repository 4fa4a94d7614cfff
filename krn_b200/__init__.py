"""B200-native implementation of the dense-contraction path of the krn kernel language.

The public names are krn's (src/krn/__init__.py:15-242) for the part of the language the tile matrix product and
the flash-attention pattern are written in; `import krn_b200 as krn` lets such a kernel file run unchanged:

    from krn_b200 import Const, Matrix, block, bf16, f32, host, kernel, pipelined, struct, zeros

Kernels are captured from source, matched against the contractions the prebuilt sm_100a library implements
(`krn_b200/csrc`, reached through `krn_b200.hw.Libraries` and ctypes) and launched on `host.Device.current()`.
"""

from krn_b200 import errors, formats, host, hw, targets
from krn_b200.errors import CaptureError, CUDAError, LaunchError, PerformanceWarning, PrecisionWarning, TargetError
from krn_b200.frontend.device_functions import (UNIFORM, PingPong, Space, Uniform, WarpSpecialized, arange, block, chunks,
                                                full, maximum, minimum, pipelined, where, zeros)
from krn_b200.frontend.geometry import Blocks, Items, Tiles
from krn_b200.frontend.kernel import Kernel, kernel
from krn_b200.frontend.variants import AmbiguousVariant, Family, family
from krn_b200.frontend.records import AUTO, Const, struct
from krn_b200.frontend.types import (QMatrix, QTile, T, Matrix, Tensor, Tile, Vector, bf16, f8e4m3fn, f8e5m2, f16, f32,
                                     f64, i32, i64, u8, u32)
from krn_b200.runtime.settings import config, configure
from krn_b200.targets import Feature

__all__ = [
    "AUTO", "AmbiguousVariant", "Blocks", "CUDAError", "CaptureError", "Const", "Family", "Feature", "Items", "Kernel",
    "LaunchError", "Matrix",
    "PerformanceWarning", "PingPong", "PrecisionWarning", "QMatrix", "QTile", "Space", "T", "TargetError", "Tensor",
    "Tile", "Tiles", "UNIFORM", "Uniform", "Vector", "WarpSpecialized", "arange", "bf16", "block", "chunks", "config",
    "configure", "errors", "f16", "family", "f32", "f64", "f8e4m3fn", "f8e5m2", "formats", "full", "host", "hw", "i32", "i64",
    "kernel", "maximum", "minimum", "pipelined", "struct", "targets", "u32", "u8", "where", "zeros",
]
