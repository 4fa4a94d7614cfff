"""Kernel objects: `@kernel` marks a device function; capture decides its role from how it is used.

A host call infers the geometry from the body: `gemm(a, b, c)`. Brackets carry only a configuration,
`gemm[Tiling(bm=64)](a, b, c)`, and `launch=` overrides the inferred geometry. A configured kernel, whose first
parameter is a `@struct` with `Const` fields, uses the defaults of that struct when the call omits it
(src/krn/frontend/kernel.py:22-117)."""

from __future__ import annotations

import inspect
from typing import Any, Callable

from krn_b200.frontend.geometry import Geometry, Tiles
from krn_b200.frontend.records import is_configuration
from krn_b200.runtime.api import Configured, Device, Launcher
from krn_b200.runtime.settings import current_settings


class Kernel:
    __slots__ = ("_shape", "fn", "name")

    def __init__(self, fn: Callable[..., None]) -> None:
        self.fn = fn
        self.name = getattr(fn, "__name__", type(fn).__name__)
        self._shape: tuple[int, type | None] | None = None

    def _inspect(self) -> tuple[int, type | None]:
        """The parameter count and the configuration struct of the first parameter, if it has one. Read on the first
        launch: annotations may name what follows the kernel in its file."""
        if self._shape is None:
            parameters = tuple(inspect.signature(self.fn).parameters.values())
            first = parameters[0].annotation if parameters else None
            if isinstance(first, str):
                first = eval(first, self.fn.__globals__)  # noqa: S307 - the user's own annotation text
            self._shape = (len(parameters), first if is_configuration(first) else None)
        return self._shape

    @property
    def configuration(self) -> type | None:
        return self._inspect()[1]

    def __call__(self, *args: Any, launch: Geometry | None = None) -> None:
        """Launch on the current device, evaluating the body's iteration space on these arguments."""
        device = Device.current()
        launcher: Launcher = device.launcher(self, launch.blocks if isinstance(launch, Tiles) else launch)
        arity, configuration = self._inspect()
        if configuration is not None and len(args) == arity - 1:
            try:
                config = current_settings().configuration(self.name, configuration)
            except TypeError:
                raise TypeError(f"{self.name}: configuration needs arguments; write {self.name}[Config(...)](...)") from None
            launcher = Configured(launcher, config)
        launcher(*args)

    def explain(self, *args: Any, launch: Geometry | None = None):
        device = Device.current()
        launcher = device.launcher(self, launch.blocks if isinstance(launch, Tiles) else launch)
        arity, configuration = self._inspect()
        if configuration is not None and len(args) == arity - 1:
            args = (current_settings().configuration(self.name, configuration), *args)
        return launcher.explain(*args)

    def __getitem__(self, configuration: Any) -> Launcher:
        """Specialise on a configuration; launch geometry belongs in `launch=`."""
        _, kind = self._inspect()
        if kind is None or not isinstance(configuration, kind):
            raise TypeError(f"{self.name}: brackets take a configuration; pass geometry with launch=")
        return Configured(Device.current().launcher(self), configuration)


def kernel(fn: Callable[..., None]) -> Kernel:
    """The one decorator of device code."""
    return Kernel(fn)
