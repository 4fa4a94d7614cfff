"""The runtime surface kernels launch through: `Device`, `Stream`, `Event`, `Launcher`, `Bound`, `Configured`,
`Graph` — names, argument meaning and error behaviour of the reference's abstract classes
(src/krn/runtime/api.py:54-318), implemented once, for the B200 device (`krn_b200.runtime.device`).

Launches are enqueued on the current stream and return at once; completion is an `Event` that can be waited on with a
timeout (`event.wait(60)`) or awaited; asynchronous device failures (an expired bounded wait inside a kernel) surface
at the next event, as the reference's sticky stream errors do (src/krn/runtime/runtime.py:392-399)."""

from __future__ import annotations

import asyncio
from abc import ABC, abstractmethod
from contextvars import ContextVar
from dataclasses import dataclass
from typing import Any, Callable


@dataclass(frozen=True)
class Explanation:
    """What a launch would do, without launching: the recognised pattern, geometry and the kernel that runs it."""

    kernel: str
    plan: str
    geometry: object
    entry: str
    notes: tuple[str, ...] = ()

    def __str__(self) -> str:
        lines = [f"{self.kernel}: {self.plan}", f"  geometry: {self.geometry}", f"  runs: {self.entry}"]
        return "\n".join([*lines, *(f"  note: {n}" for n in self.notes)])


class Event(ABC):
    """A point in a stream's order. `done()` never blocks; awaiting suspends the awaiting task only."""

    @abstractmethod
    def done(self) -> bool: ...

    @property
    @abstractmethod
    def error(self) -> BaseException | None: ...

    @abstractmethod
    def wait(self, timeout: float | None = None) -> None:
        """Block the host until completion; `TimeoutError` after `timeout` seconds."""

    @abstractmethod
    def elapsed_since(self, earlier: "Event") -> float:
        """Milliseconds between two events of one device, measured by the device clock."""

    def __await__(self):
        return self._await().__await__()

    async def _await(self) -> None:
        while not self.done():
            await asyncio.sleep(0.0005)
        if self.error is not None:
            raise self.error


current_stream: ContextVar["Stream | None"] = ContextVar("krn_b200_current_stream", default=None)


class Stream(ABC):
    """An in-order queue of device work. `with stream:` makes it the current stream of the thread or task."""

    device: "Device"

    @abstractmethod
    def record(self) -> Event: ...

    @abstractmethod
    def wait(self, event: Event) -> None:
        """Make later work on this stream wait for an event of another stream, without blocking the host."""

    def __enter__(self) -> "Stream":
        self._tokens = getattr(self, "_tokens", [])
        self._tokens.append(current_stream.set(self))
        return self

    def __exit__(self, *exc) -> None:
        current_stream.reset(self._tokens.pop())


class Launcher(ABC):
    """A kernel bound to a launch geometry. Calling it enqueues on the current stream and returns at once."""

    @abstractmethod
    def __call__(self, *args: Any) -> None: ...

    @abstractmethod
    def explain(self, *args: Any) -> Explanation: ...

    @abstractmethod
    def submit(self, *args: Any) -> Event: ...

    @abstractmethod
    def bind(self, *args: Any) -> "Bound": ...


class Bound(ABC):
    """A launch whose arguments are already encoded: the fast path for loops that repeat a launch."""

    @abstractmethod
    def __call__(self) -> None: ...

    @abstractmethod
    def submit(self) -> Event: ...

    @abstractmethod
    def rebind(self, *args: Any) -> None: ...


class ConfiguredBound(Bound):
    def __init__(self, inner: Bound, config: Any) -> None:
        self.inner, self.config = inner, config

    def __call__(self) -> None:
        self.inner()

    def submit(self) -> Event:
        return self.inner.submit()

    def rebind(self, *args: Any) -> None:
        self.inner.rebind(self.config, *args)


class Configured(Launcher):
    """The launcher of a configured kernel: the configuration chosen in the brackets is passed as the first argument
    (src/krn/runtime/api.py:206-222)."""

    def __init__(self, inner: Launcher, config: Any) -> None:
        self.inner, self.config = inner, config

    def __call__(self, *args: Any) -> None:
        self.inner(self.config, *args)

    def explain(self, *args: Any) -> Explanation:
        return self.inner.explain(self.config, *args)

    def submit(self, *args: Any) -> Event:
        return self.inner.submit(self.config, *args)

    def bind(self, *args: Any) -> Bound:
        return ConfiguredBound(self.inner.bind(self.config, *args), self.config)


class Graph(ABC):
    """Recorded launches that replay with one call. CUDA graphs require the recorded arguments; tensor CONTENTS may
    change between replays (src/krn/runtime/api.py:225-243)."""

    @abstractmethod
    def __call__(self, *args: Any) -> None: ...

    @abstractmethod
    def submit(self, *args: Any) -> Event: ...


class Device(ABC):
    """One GPU with the target facts the path needs."""

    target: Any

    @classmethod
    def current(cls) -> "Device":
        """The device kernels launch on. The first call detects the system and builds the device; `KRN_TARGET` names
        another target (src/krn/runtime/api.py:321-354). There is one device family here, sm_100a."""
        from krn_b200.runtime.device import default_device

        return default_device()

    @property
    @abstractmethod
    def default_stream(self) -> Stream: ...

    @abstractmethod
    def stream(self) -> Stream: ...

    @abstractmethod
    def to_device(self, array: Any) -> Any: ...

    @abstractmethod
    def empty(self, dtype: Any, *shape: int) -> Any: ...

    @abstractmethod
    def launcher(self, kernel: Any, launch: Any = None) -> Launcher: ...

    @abstractmethod
    def graph(self, fn: Callable[..., None], *args: Any) -> Graph: ...

    @abstractmethod
    async def synchronize(self) -> None: ...
