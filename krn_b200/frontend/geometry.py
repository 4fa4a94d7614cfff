"""The three ways a call can state its launch size with `launch=` instead of having it inferred from the kernel
body. Field names and the `Tiles.blocks` axis order are those of src/krn/frontend/geometry.py:8-41."""

from __future__ import annotations

from dataclasses import dataclass


def ceildiv(a: int, b: int) -> int:
    return -(-a // b)


@dataclass(frozen=True)
class Items:
    """`count` independent work items, one thread each; how they are grouped into blocks is the device's choice."""

    count: int


@dataclass(frozen=True)
class Blocks:
    """A grid given outright: `x`, `y`, `z` blocks, optionally with the number of threads per block."""

    x: int
    y: int = 1
    z: int = 1
    threads: int | None = None


@dataclass(frozen=True)
class Tiles:
    """A grid derived from an output: enough `tile`-sized blocks to cover `shape`, rounding up on every axis, e.g.
    `Tiles(c.shape, (bm, bn))`.

    Grid axes are assigned from the back — columns become x, rows y — which is the order `block.tile(bm, bn)` uses
    inside the kernel, so each block lands on the tile it computes."""

    shape: tuple[int, ...]
    tile: tuple[int, ...]

    @property
    def blocks(self) -> Blocks:
        if len(self.shape) != len(self.tile):
            raise ValueError(f"Tiles: shape {self.shape} and tile {self.tile} differ in rank")
        counts = [ceildiv(extent, size) for extent, size in zip(self.shape, self.tile)]
        return Blocks(*reversed(counts))


Geometry = Items | Blocks | Tiles
