"""Target facts of the one target this build has (src/krn/facts/targets.py:22-37,177-210 for sm_100a)."""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class Feature(str, Enum):
    TENSOR_CORES = "tensor_cores"
    BULK_COPY = "bulk_copy"            # TMA
    TENSOR_MEMORY = "tensor_memory"    # tcgen05 accumulators
    BLOCK_SCALED_MMA = "block_scaled_mma"
    CLUSTERS = "clusters"


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
        return cls(arch, 227 * 1024, 512, frozenset(Feature),
                   frozenset({"f16", "bf16", "tf32", "f8e4m3fn", "f8e5m2", "f6", "f4"}))

    def has(self, feature: Feature) -> bool:
        return feature in self.features

    def mma_native(self, dtype) -> bool:
        """Whether the tensor cores multiply this element type directly; a coarse fp32 scale per block is applied to
        the partial sums outside the unit (src/krn/facts/targets.py:127-138)."""
        return getattr(dtype, "name", str(dtype)) in self.mma_native_types
