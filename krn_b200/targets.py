"""Target facts of the one target this build has (src/krn/facts/targets.py:22-37,177-210 for sm_100a)."""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class Feature(str, Enum):
    """What a kernel may need from a target, with the reference's names (src/krn/facts/targets.py:22-37)."""

    SHARED_MEMORY = "shared_memory"
    WARP_SHUFFLE = "warp_shuffle"
    WARP_VOTE = "warp_vote"
    ATOMICS_64 = "atomics_64"
    FLOAT64 = "float64"
    TENSOR_CORE = "tensor_core"        # some native matrix unit exists
    ASYNC_COPY = "async_copy"          # cp.async
    BULK_COPY = "bulk_copy"            # TMA
    ASYNC_MMA = "async_mma"            # a product issued by one thread, reading shared memory (tcgen05)
    GRID_SYNC = "grid_sync"
    TENSOR_MEMORY = "tensor_memory"    # tcgen05 accumulators
    CLUSTERS = "clusters"
    BLOCK_SCALED_MMA = "block_scaled_mma"


@dataclass(frozen=True)
class Target:
    arch: str
    shared_bytes: int
    tensor_memory_columns: int
    features: frozenset
    mma_native_types: frozenset

    @classmethod
    def of(cls, arch: str) -> "Target":
        if arch != "sm_100a":
            from krn_b200.errors import TargetError

            raise TargetError(f"target {arch}", "this build", "only sm_100a kernels are built", "use sm_100a")
        return Nvidia(arch, 227 * 1024, 512, frozenset(Feature),
                      frozenset({"f16", "bf16", "tf32", "f8e4m3fn", "f8e5m2", "f6", "f4"}))

    def has(self, feature: Feature) -> bool:
        return feature in self.features

    def mma_native(self, dtype) -> bool:
        """Whether the tensor cores multiply this element type directly; a coarse fp32 scale per block is applied to
        the partial sums outside the unit (src/krn/facts/targets.py:127-138)."""
        return getattr(dtype, "name", str(dtype)) in self.mma_native_types


class Nvidia(Target):
    """The vendor classes exist so that a family's rules can name them (`@gemm.variant(targets.Nvidia, ...)`,
    examples/04_libraries/03_gemm_variants.py:53); only an sm_100a `Nvidia` target can be the device here."""


class AMD(Target):
    pass


class Apple(Target):
    pass


class CPU(Target):
    pass


def described(vendor: type, arch: str, features: frozenset) -> Target:
    """A target this build cannot run on but a family can be audited against: arch and features, no resources."""
    return vendor(arch, 0, 0, frozenset(features), frozenset())
