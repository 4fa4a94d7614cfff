"""The settings the path reads, with the reference's spelling: `configure("run.target", ...)` /
`configure(**{"run.target": ...})`, `config.run.target = ...`, scoped `with configure(...)`, and the `KRN_TARGET`
environment seed (src/krn/runtime/settings.py:279-515). Only the `run` group has fields here; `cache.dir` is accepted
and ignored because nothing is compiled at run time."""

from __future__ import annotations

import os
from contextvars import ContextVar
from dataclasses import dataclass, field, replace
from typing import Any

from krn_b200.errors import SettingError

TARGETS = ("sm_100a",)


@dataclass(frozen=True)
class Run:
    target: str = "sm_100a"
    graphs: bool = True
    variants: tuple[tuple[str, str], ...] = ()  # family name -> pinned variant ("portable" for the portable kernel)


@dataclass(frozen=True)
class Cache:
    dir: str = ""


@dataclass(frozen=True)
class Settings:
    run: Run = field(default_factory=Run)
    cache: Cache = field(default_factory=Cache)
    configurations: tuple[tuple[str, Any], ...] = ()

    def key(self) -> tuple:
        return (self.run.target,)

    def configuration(self, kernel_name: str, kind: type) -> Any:
        """The default configuration of a kernel: one pinned with `configure(**{"run.config": {...}})`, else the
        struct's own defaults (src/krn/runtime/settings.py:314-336)."""
        for name, value in self.configurations:
            if name == kernel_name and isinstance(value, kind):
                return value
        return kind()


def _from_environment() -> Settings:
    target = os.environ.get("KRN_TARGET", "sm_100a")
    return Settings(run=Run(target=_check_target("KRN_TARGET", target)))


def _check_target(variable: str, value: str) -> str:
    if value not in TARGETS:
        raise SettingError(variable, value, f"one of {', '.join(TARGETS)} (this build has no other back end and no "
                                            f"CPU fallback)")
    return value


_current: ContextVar[Settings | None] = ContextVar("krn_b200_settings", default=None)


def current_settings() -> Settings:
    settings = _current.get()
    if settings is None:
        settings = _from_environment()
        _current.set(settings)
    return settings


def _apply(settings: Settings, dotted: str, value: Any) -> Settings:
    group, _, name = dotted.partition(".")
    if group == "run" and name == "target":
        return replace(settings, run=replace(settings.run, target=_check_target(dotted, value)))
    if group == "run" and name == "graphs":
        if not isinstance(value, bool):
            raise SettingError(dotted, str(value), "a bool")
        return replace(settings, run=replace(settings.run, graphs=value))
    if group == "run" and name == "variants":
        if not isinstance(value, dict) or not all(isinstance(k, str) and isinstance(v, str) for k, v in value.items()):
            raise SettingError(dotted, str(value), "a mapping of family name to variant name")
        return replace(settings, run=replace(settings.run, variants=tuple(value.items())))
    if group == "run" and name == "config":
        if not isinstance(value, dict):
            raise SettingError(dotted, str(value), "a mapping of kernel name to configuration")
        return replace(settings, configurations=tuple(value.items()))
    if group == "cache" and name == "dir":
        return replace(settings, cache=Cache(str(value)))
    raise SettingError(dotted, str(value), "a setting this path reads (run.target, run.graphs, run.config, run.variants, cache.dir)")


class configure:
    """Apply overrides now; used as a context manager, restore the previous snapshot on exit."""

    def __init__(self, *pairs: Any, **dotted: Any) -> None:
        settings = current_settings()
        if len(pairs) % 2:
            raise TypeError("configure takes name, value pairs")
        for name, value in zip(pairs[::2], pairs[1::2]):
            settings = _apply(settings, name, value)
        for name, value in dotted.items():
            settings = _apply(settings, name.replace("__", "."), value)
        self._token = _current.set(settings)

    def __enter__(self) -> Settings:
        return current_settings()

    def __exit__(self, *exc) -> None:
        _current.reset(self._token)


class _Group:
    def __init__(self, name: str) -> None:
        object.__setattr__(self, "_name", name)

    def __getattr__(self, field_name: str) -> Any:
        return getattr(getattr(current_settings(), self._name), field_name)

    def __setattr__(self, field_name: str, value: Any) -> None:
        _current.set(_apply(current_settings(), f"{self._name}.{field_name}", value))


class _Config:
    run = _Group("run")
    cache = _Group("cache")


config = _Config()
