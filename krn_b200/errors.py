"""Exceptions of the path. Names, constructor arguments and message layouts are the reference's, because callers
match on them; the code behind them is this package's own.

Message layouts that are contract:

* `CaptureError(span, message)` → ``file:line:col: error: message`` and, when the source line can be read, that
  line and a caret under column `col` (src/krn/compiler/errors.py:41-52).
* `TargetError(feature, target, reason, instead)` → ``{feature} is not available on {target}: {reason}. Instead:
  {instead}.`` (src/krn/compiler/errors.py:55-62).
* `SettingError(variable, value, expected)` → ``VARIABLE='value': expected …`` (src/krn/compiler/errors.py:65-69).
* `LaunchError(kernel, reason)` → ``kernel: the launch geometry cannot be inferred, reason; <how to fix>``
  (src/krn/compiler/space.py:82-86).
* `CUDAError` → ``NAME: message`` of a failed device call (src/krn/runtime/cuda_backend.py:97-105).
"""

from __future__ import annotations

import ast
import linecache
from typing import NamedTuple


class PrecisionWarning(UserWarning):
    """Emitted when a call site chose a narrower number format than the data had."""


class PerformanceWarning(UserWarning):
    """Emitted when something known about a kernel at capture time will make it slow."""


class Span(NamedTuple):
    """Where in the user's source a diagnostic points: file, 1-based line, 1-based column."""

    file: str
    line: int
    col: int

    @classmethod
    def of(cls, file: str, node: ast.AST) -> "Span":
        """The span of an `ast` node (ast columns are 0-based, diagnostics 1-based)."""
        line = getattr(node, "lineno", 0)
        column = getattr(node, "col_offset", 0)
        return cls(file, line, column + 1)

    def __str__(self) -> str:
        return ":".join((self.file, str(self.line), str(self.col)))


def _excerpt(span: Span) -> str | None:
    """The source line a span points at plus a caret line, indented by four; None when the file cannot be read."""
    text = linecache.getline(span.file, span.line).rstrip()
    if not text:
        return None
    pointer = " " * (span.col - 1) + "^"
    return f"    {text}\n    {pointer}"


class CaptureError(Exception):
    """The kernel source cannot be captured; rendered the way a compiler prints a diagnostic."""

    def __init__(self, span: Span | None, message: str) -> None:
        self.span = span
        self.message = message
        head = f"error: {message}" if span is None else f"{span}: error: {message}"
        super().__init__(head)

    def __str__(self) -> str:
        head = self.args[0]
        excerpt = _excerpt(self.span) if self.span is not None else None
        return head if excerpt is None else f"{head}\n{excerpt}"


class TargetError(CaptureError):
    """The target lacks `feature`: says why and what to write instead, optionally with a source span."""

    def __init__(self, feature: str, target: str, reason: str, instead: str, *, span: Span | None = None) -> None:
        self.feature = feature
        self.target = target
        self.reason = reason
        self.instead = instead
        why, fix = reason.rstrip("."), instead.rstrip(".")
        super().__init__(span, f"{feature} is not available on {target}: {why}. Instead: {fix}.")


class SettingError(ValueError):
    """A configuration override whose text does not parse as the setting it is meant for."""

    def __init__(self, variable: str, value: str, expected: str) -> None:
        super().__init__(f"{variable}={value!r}: expected {expected}")


FIXES = (
    "write the loop as `for i in items(n)`, or slice the tensors with `block.tile`, so the body says how big the work "
    "is; or pass `launch=Items(n)` or `launch=Blocks(...)` to the call"
)


class LaunchError(ValueError):
    """Neither the kernel body nor the call's arguments determine how many blocks to launch."""

    def __init__(self, kernel_name: str, reason: str) -> None:
        super().__init__(f"{kernel_name}: the launch geometry cannot be inferred, {reason}; {FIXES}")


class CUDAError(RuntimeError):
    """A CUDA call or a kernel-library entry point reported failure; the text is ``NAME: message``."""
