"""`lib.matmul` for the B200 device: the plain-function caller of the tile product, with the fused epilogues.

Mirrors the reference's library layer for this one operation (src/krn/lib/lib.py): the same call
`matmul(a, b, *, precision, epilogue, bias, out, options)` with `a` (m, k) and row-major `b` (k, n), the same
`Epilogue` / `Compute` vocabulary, and the same candidate protocol — a `MatmulCandidate` says who it is
(`name`, `op`, `origin`), what it refuses (`refusal(problem, target)` returns the reason or None) and `run`s without
synchronising; `CANDIDATES` lists them and a call whose every candidate refuses raises `NoCandidate` with each reason
(src/krn/lib/lib.py:201-235,247-262,580-615). The reference's own candidate launches its `matmul_epilogue` tile kernel
(src/krn/lib/lib_ours.py:58-75); the one here passes the same statements to the prebuilt sm_100a kernel, whose
epilogue applies bias and activation to the f32 accumulator in registers before the single rounding.

There is one candidate and no tuner, vendor adapter or stored winners: those parts of the reference's library layer
are outside the path this package rebuilds."""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from enum import StrEnum, auto
from typing import Any, ClassVar

from krn_b200.errors import TargetError
from krn_b200.frontend.types import Dtype, bf16, f16, f32
from krn_b200.runtime import calls
from krn_b200.runtime.device import DeviceTensor, _element_of, _raw, default_device

TARGET = "sm_100a"


class Op(StrEnum):
    MATMUL = auto()


class Origin(StrEnum):
    VENDOR = auto()
    OURS = auto()
    HOST = auto()


class Epilogue(StrEnum):
    """Fused after the multiply (src/krn/lib/lib.py:82-91)."""

    NONE = auto()
    BIAS = auto()
    RELU = auto()
    GELU = auto()
    BIAS_RELU = auto()
    BIAS_GELU = auto()
    SILU = auto()


class Compute(StrEnum):
    """STRICT is the accumulator the dtypes name; the others are explicit operation choices, never defaults
    (src/krn/lib/lib.py:99-102)."""

    STRICT = auto()
    TF32 = auto()
    EMULATED = auto()


# C-ABI flags (include/krn_b200.h KRN_B200_EPILOGUE_*) of each epilogue: bit 0 bias, bits 1-2 activation
FLAGS = {Epilogue.NONE: 0, Epilogue.BIAS: 1, Epilogue.RELU: 2, Epilogue.GELU: 4, Epilogue.BIAS_RELU: 3,
         Epilogue.BIAS_GELU: 5, Epilogue.SILU: 6}


@dataclass(frozen=True, slots=True, kw_only=True)
class LibOptions:
    """Plan-time options. Only the fields this candidate could honour are kept: `sm_count` (0 = all SMs; any other
    value is refused, the persistent kernel sizes its own grid) and `workspace_bytes` (unused: no workspace)."""

    workspace_bytes: int = 0
    sm_count: int = 0


@dataclass(frozen=True, slots=True)
class Problem:
    """shape is (m, n, k); dtypes are those of a, b and the result."""

    op: Op
    dtypes: tuple[Dtype, ...]
    shape: tuple[int, ...]
    options: LibOptions
    epilogue: Epilogue = Epilogue.NONE
    precision: Compute = Compute.STRICT


@dataclass(frozen=True, slots=True)
class Operands:
    """The tensors of a multiply by role: `a` (m, k), `b` (k, n), the result `out` (m, n), the optional `bias` (n),
    which has the type of the result (src/krn/lib/lib.py:155-163)."""

    a: Any
    b: Any
    out: Any = field()
    bias: Any | None = None


class NoCandidate(LookupError):
    """Every candidate refused. The message lists each refusal."""


class Candidate(ABC):
    name: ClassVar[str]
    op: ClassVar[Op]
    origin: ClassVar[Origin]
    precisions: ClassVar[frozenset[Compute]] = frozenset({Compute.STRICT})

    def unavailable(self, target: str) -> str | None:
        """Why this implementation cannot run on the machine at all, or None if available."""
        return None

    @abstractmethod
    def refusal(self, problem: Problem, target: str) -> str | None:
        """Why this candidate cannot run the problem (dtype, layout, epilogue, architecture), or None if it can."""


class MatmulCandidate(Candidate):
    @abstractmethod
    def run(self, problem: Problem, operands: Operands, stream: Any) -> None: ...


class TensorMemoryMatmul(MatmulCandidate):
    """The tcgen05 tile product of libkrn_b200.so (`krn_b200_matmul`)."""

    name, op, origin = "b200", Op.MATMUL, Origin.OURS

    def unavailable(self, target: str) -> str | None:
        from krn_b200.hw.libraries import LibraryNotFound
        from krn_b200.runtime import native

        try:
            native.library()
        except LibraryNotFound as error:
            return str(error)
        return None

    def refusal(self, problem: Problem, target: str) -> str | None:
        a, b, out = problem.dtypes
        if problem.precision is not Compute.STRICT:
            return f"the tensor-memory product accumulates in f32 as the dtypes name; {problem.precision} is not offered"
        if a != b or a not in (bf16, f16):
            return f"the tensor-memory product multiplies two bf16 or two f16 matrices, got {a} @ {b}"
        if out not in (bf16, f16, f32):
            return f"the result type must be bf16, f16 or f32, got {out}"
        if problem.options.sm_count:
            return "the persistent kernel sizes its own grid; sm_count must stay 0"
        return None

    def run(self, problem: Problem, operands: Operands, stream: Any) -> None:
        bias = None if operands.bias is None else _raw(operands.bias)
        calls.matmul(_raw(operands.a), _raw(operands.b), _raw(operands.out), b_kn=True, epilogue=FLAGS[problem.epilogue],
                     bias=bias, stream=getattr(stream, "raw", stream))


CANDIDATES: list[MatmulCandidate] = [TensorMemoryMatmul()]


def product_type(a: Dtype, b: Dtype) -> Dtype:
    """The type that holds both inputs: the type itself for two equal ones, f32 otherwise."""
    return a if a == b else f32


def matmul(a: Any, b: Any, *, precision: Compute = Compute.STRICT, epilogue: Epilogue = Epilogue.NONE,
           bias: Any | None = None, out: Any | None = None, options: LibOptions | None = None, stream: Any = None) -> Any:
    """a @ b with an optional fused epilogue, enqueued on `stream` (the device's default stream when None). Allocates
    `out` when it is not given, in the type that holds both inputs. An epilogue that names a bias needs `bias` (a
    vector of n elements of the result type); a bias without such an epilogue is an error rather than ignored."""
    device = default_device()
    epilogue = Epilogue(epilogue)
    raw_a, raw_b = _raw(a), _raw(b)
    if len(raw_a.shape) != 2 or len(raw_b.shape) != 2 or raw_a.shape[1] != raw_b.shape[0]:
        raise ValueError(f"shapes do not compose: a {tuple(raw_a.shape)} @ b {tuple(raw_b.shape)}")
    type_a, type_b = _element_of(raw_a), _element_of(raw_b)
    result = out if out is not None else device.empty(product_type(type_a, type_b), raw_a.shape[0], raw_b.shape[1])
    raw_out = _raw(result)
    wants_bias = bool(FLAGS[epilogue] & 1)
    if wants_bias != (bias is not None):
        raise ValueError(f"epilogue {epilogue} " + ("needs a bias vector" if wants_bias else "takes no bias"))
    if bias is not None:
        raw_bias = _raw(bias)
        if tuple(raw_bias.shape) != (raw_b.shape[1],) or _element_of(raw_bias) != _element_of(raw_out):
            raise ValueError(f"the bias must be a vector of {raw_b.shape[1]} {_element_of(raw_out)} elements, got "
                             f"{tuple(raw_bias.shape)} {_element_of(raw_bias)}")
    problem = Problem(Op.MATMUL, (type_a, type_b, _element_of(raw_out)),
                      (raw_a.shape[0], raw_b.shape[1], raw_a.shape[1]), options or LibOptions(), epilogue, precision)
    refusals = []
    for candidate in CANDIDATES:
        reason = candidate.unavailable(TARGET) or candidate.refusal(problem, TARGET)
        if reason is None:
            candidate.run(problem, Operands(a, b, result, bias), stream or device.default_stream)
            return result
        refusals.append(f"{candidate.name}: {reason}")
    if precision is not Compute.STRICT:
        raise TargetError(f"matmul precision {precision}", TARGET, "; ".join(refusals), "use Compute.STRICT")
    raise NoCandidate(f"{problem.op}: " + "; ".join(refusals))


__all__ = ["CANDIDATES", "Candidate", "Compute", "DeviceTensor", "Epilogue", "LibOptions", "MatmulCandidate", "NoCandidate",
           "Op", "Operands", "Origin", "Problem", "TensorMemoryMatmul", "matmul", "product_type"]
