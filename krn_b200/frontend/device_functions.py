"""Signature-only device functions of tile kernels. Kernel bodies are read, never run
(src/krn/compiler/source.py), so calling one of these on the host is a mistake and says so."""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

from krn_b200.frontend.records import AUTO, Auto


def _device_only(name: str):
    raise RuntimeError(f"{name} is a device function: it has a meaning only inside a @kernel body")


class Space(str, Enum):
    """Where a tile lives (src/krn/frontend/memory.py:272-278)."""

    REGISTERS = "registers"
    SHARED = "shared"
    TENSOR_MEMORY = "tensor_memory"


@dataclass(frozen=True)
class Uniform:
    """Every warp loads and computes."""


@dataclass(frozen=True)
class WarpSpecialized:
    """Producer warps move tiles, consumer warps multiply: TMA with barriers on sm_100a."""

    producers: int = 1
    consumers: int = 2


@dataclass(frozen=True)
class PingPong:
    groups: int = 2


UNIFORM = Uniform()


class block:
    """The block: `block.tile(bm, bn)` is the tile of the output this block owns (rows from y, columns from x);
    `block.index()` its coordinates in the grid (src/krn/frontend/groups/block.py:12-43)."""

    @staticmethod
    def tile(*sizes: int):
        _device_only("block.tile")

    @staticmethod
    def index():
        _device_only("block.index")


def zeros(dtype, *extent: int, space: Space = Space.REGISTERS):
    _device_only("zeros")


def full(dtype, value: float, *extent: int):
    _device_only("full")


def where(condition, x, y):
    _device_only("where")


def arange(extent: int, axis: int = 0, *, rank: int = 1, start=0):
    _device_only("arange")


def maximum(a, b):
    _device_only("maximum")


def minimum(a, b):
    _device_only("minimum")


def pipelined(extent: int, tile: int, *, stages: int | Auto = AUTO, schedule=AUTO):
    _device_only("pipelined")


def chunks(extent: int, tile: int):
    _device_only("chunks")
