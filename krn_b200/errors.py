"""Error conventions of the path, kept as the reference spells them.

* `CaptureError(span, message)` prints `file:line:col: error: message` with the source line and a caret;
  `TargetError(feature, target, reason, instead)` is the four-part refusal "`{feature} is not available on
  {target}: {reason}. Instead: {instead}.`" (src/krn/compiler/errors.py:41-62).
* `LaunchError(ValueError)`: the launch geometry cannot be inferred (src/krn/compiler/space.py:82-86).
* `SettingError(ValueError)` (src/krn/compiler/errors.py:65-69).
* `CUDAError(RuntimeError)`: "NAME: message" for a failed device call (src/krn/runtime/cuda_backend.py:97-105).
"""

from __future__ import annotations

import ast
import linecache
from dataclasses import dataclass


class PrecisionWarning(UserWarning):
    """Numeric precision is reduced because the call site asked for it."""


class PerformanceWarning(UserWarning):
    """A computed fact about a kernel that costs performance."""


@dataclass(frozen=True, slots=True)
class Span:
    """A position in the user's file; `col` is 1-based like a compiler's."""

    file: str
    line: int
    col: int

    @classmethod
    def of(cls, file: str, node: ast.AST) -> "Span":
        return cls(file, getattr(node, "lineno", 0), getattr(node, "col_offset", 0) + 1)

    def __str__(self) -> str:
        return f"{self.file}:{self.line}:{self.col}"


class CaptureError(Exception):
    """A compiler-style diagnostic: `file:line:col: error: message`, then the source line and a caret."""

    def __init__(self, span: Span | None, message: str) -> None:
        super().__init__(f"{span}: error: {message}" if span else f"error: {message}")
        self.span = span
        self.message = message

    def __str__(self) -> str:
        if self.span is None:
            return self.args[0]
        source = linecache.getline(self.span.file, self.span.line).rstrip()
        return f"{self.args[0]}\n    {source}\n    {' ' * (self.span.col - 1)}^" if source else self.args[0]


class TargetError(CaptureError):
    """An unavailable target feature, with an actionable alternative and an optional source location."""

    def __init__(self, feature: str, target: str, reason: str, instead: str, *, span: Span | None = None) -> None:
        self.feature, self.target, self.reason, self.instead = feature, target, reason, instead
        message = f"{feature} is not available on {target}: {reason.rstrip('.')}. Instead: {instead.rstrip('.')}."
        super().__init__(span, message)


class SettingError(ValueError):
    """An override cannot be interpreted as the setting it names."""

    def __init__(self, variable: str, value: str, expected: str) -> None:
        super().__init__(f"{variable}={value!r}: expected {expected}")


FIXES = (
    "write the loop as `for i in items(n)`, or slice the tensors with `block.tile`, so the body says how big the work "
    "is; or pass `launch=Items(n)` or `launch=Blocks(...)` to the call"
)


class LaunchError(ValueError):
    """The launch geometry of a kernel cannot be read from its body and its arguments."""

    def __init__(self, kernel_name: str, reason: str) -> None:
        super().__init__(f"{kernel_name}: the launch geometry cannot be inferred, {reason}; {FIXES}")


class CUDAError(RuntimeError):
    """A device-side call returned a status other than success."""
