"""Kernel families: a portable kernel plus variants that say where they apply, chosen per target.

The behaviour of the reference's families (src/krn/frontend/variants.py:1-130; the example is
examples/04_libraries/03_gemm_variants.py): `@family` wraps the portable kernel; `@gemm.variant(targets.Nvidia,
arch={...}, requires={Feature...})` registers another kernel of the same signature under a rule; `select(target)`
takes the matching rule that is most specific — a pinned architecture outranks any number of required features, more
required features outrank fewer, naming a vendor outranks not naming one — and two winners of equal rank raise
`AmbiguousVariant`; `audit(targets)` runs the selection over a list of targets; `run.variants` pins a family to one
variant (or to "portable"). Calling the family, or indexing it with a configuration, launches the selected kernel on
the current device — here always the sm_100a device, where a `requires={Feature.TENSOR_MEMORY}` variant is the one
that survives."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Iterable

from krn_b200.frontend.kernel import Kernel
from krn_b200.runtime.settings import Settings, current_settings
from krn_b200.targets import Feature, Target


class AmbiguousVariant(LookupError):
    """Two variants of one family match a target with the same specificity."""


@dataclass(frozen=True)
class Rule:
    """Where a variant applies; an empty field does not restrict."""

    vendors: tuple[type, ...] = ()
    archs: frozenset = frozenset()
    requires: frozenset = frozenset()

    def matches(self, target: Target) -> bool:
        if self.vendors and not isinstance(target, self.vendors):
            return False
        if self.archs and target.arch not in self.archs:
            return False
        return self.requires <= target.features

    @property
    def specificity(self) -> tuple[int, int, int]:
        return (1 if self.archs else 0, len(self.requires), 1 if self.vendors else 0)


@dataclass(frozen=True)
class Selection:
    """The kernel chosen for a target, its name and why."""

    kernel: Kernel
    name: str
    reason: str


@dataclass
class Family:
    name: str
    portable: Kernel
    variants: dict[str, tuple[Rule, Kernel]] = field(default_factory=dict)

    def variant(self, *vendors: type, arch: Iterable[str] = (), requires: Iterable[Feature] = ()) -> Callable[[Callable[..., None]], Kernel]:
        """Decorator registering a specialised kernel; its signature must be the portable kernel's."""
        rule = Rule(tuple(vendors), frozenset(arch), frozenset(requires))

        def register(fn: Callable[..., None]) -> Kernel:
            made = Kernel(fn)
            self.variants[made.name] = (rule, made)
            return made

        return register

    def select(self, target: Target, settings: Settings | None = None) -> Selection:
        pinned = dict((settings or current_settings()).run.variants).get(self.name)
        if pinned is not None:
            if pinned == "portable":
                return Selection(self.portable, pinned, "pinned by run.variants")
            if pinned not in self.variants:
                raise LookupError(f"run.variants pins {self.name} to `{pinned}`, which is not one of "
                                  f"{', '.join(['portable', *self.variants])}")
            return Selection(self.variants[pinned][1], pinned, "pinned by run.variants")
        ranked = sorted(((rule.specificity, name) for name, (rule, _) in self.variants.items() if rule.matches(target)),
                        reverse=True)
        if not ranked:
            return Selection(self.portable, "portable", f"no variant applies to {target.arch}")
        tied = [name for rank, name in ranked if rank == ranked[0][0]]
        if len(tied) > 1:
            raise AmbiguousVariant(f"{self.name} on {target.arch}: {', '.join(sorted(tied))} tie")
        return Selection(self.variants[tied[0]][1], tied[0], f"most specific rule for {target.arch}")

    def audit(self, targets: Iterable[Target], settings: Settings | None = None) -> dict[str, str]:
        """arch -> chosen variant for every target; raises on an ambiguous one."""
        return {target.arch: self.select(target, settings).name for target in targets}

    def _selected(self) -> Kernel:
        from krn_b200.runtime.device import default_device

        return self.select(default_device().target).kernel

    def __call__(self, *args: Any, launch: Any = None) -> None:
        self._selected()(*args, launch=launch)

    def __getitem__(self, configuration: Any):
        return self._selected()[configuration]

    def explain(self, *args: Any, launch: Any = None):
        return self._selected().explain(*args, launch=launch)


def family(fn: Callable[..., None]) -> Family:
    """Declare a family from its portable kernel."""
    portable = Kernel(fn)
    return Family(portable.name, portable)
