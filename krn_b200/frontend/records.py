"""Records passed to kernels by value, and compile-time fields (src/krn/frontend/records.py:7-28).

`@struct` makes a frozen dataclass; fields annotated `Const[X]` are compile-time values: they join the
specialisation key and are not marshalled (src/krn/runtime/runtime.py:110-148)."""

from __future__ import annotations

import typing
from dataclasses import dataclass, fields, is_dataclass


def struct(cls):
    """A record passed to kernels by value: a frozen dataclass on the host, hashable as a cache key."""
    return dataclass(frozen=True)(cls)


class _ConstMeta(type):
    def __getitem__(cls, item):
        return typing.Annotated[item, "krn.Const"]


class Const(metaclass=_ConstMeta):
    """`Const[int]`: a field whose value is a capture-time constant of the kernel specialisation."""


def is_const(annotation) -> bool:
    if isinstance(annotation, str):
        return annotation.replace(" ", "").startswith("Const[")
    return typing.get_origin(annotation) is typing.Annotated and "krn.Const" in getattr(annotation, "__metadata__", ())


def is_configuration(cls) -> bool:
    """A dataclass with at least one `Const` field: the kind of struct a kernel's first parameter may be."""
    if not (isinstance(cls, type) and is_dataclass(cls)):
        return False
    hints = getattr(cls, "__annotations__", {})
    return any(is_const(hints.get(f.name, f.type)) for f in fields(cls))


@dataclass(frozen=True, slots=True, eq=False, repr=False)
class Auto:
    """The type of AUTO; choices compare by identity."""

    def __repr__(self) -> str:
        return "AUTO"


AUTO = Auto()  # "let the compiler decide from the target": `pipelined(..., stages=AUTO)`
