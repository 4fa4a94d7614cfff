"""Generate the golden fixtures in this folder by RUNNING the reference's own Python arithmetic.

Run from the repository root in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference package cannot be imported on Python 3.12 (its package `__init__` pulls in 3.14-only modules), but
the files that hold the arithmetic of this path parse fine. This script loads `src/krn/data/formats.py` as a
standalone module and lifts single functions out of `src/krn/emulator/emulate.py` (`fused`, `accumulate`,
`any_valid`, `_bfloat16`) and `src/krn/compiler/narrow.py` (`_levels`, `maximum_code`, `nan_code`,
`reference_encode`, `reference_decode`) with `ast`, executing them unmodified — nothing is copied into this
repository; only their OUTPUTS on seeded inputs are saved:

    gemm_emulator.npz   `accumulate` (k-ordered exact fma) on the shapes/seeds of the reference's tensor-core
                        tests, f32 / f16 / bf16 operands, plus `_bfloat16` roundings
    e4m3.npz            E4M3FN decode table, `reference_encode` of seeded values and edge cases

The tests compare the C oracle with these bit for bit; they never read the reference checkout.
"""

from __future__ import annotations

import ast
import importlib.util
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def lift(path: Path, names: tuple[str, ...], namespace: dict) -> dict:
    """Execute the named top-level function definitions of `path`, unmodified, in `namespace`."""
    tree = ast.parse(path.read_text())
    wanted = [node for node in tree.body if isinstance(node, ast.FunctionDef) and node.name in names]
    assert {node.name for node in wanted} == set(names), f"missing in {path}"
    for node in wanted:
        node.decorator_list = [d for d in node.decorator_list if not (isinstance(d, ast.Name) and d.id == "cache")]
    module = ast.Module(body=wanted, type_ignores=[])
    exec(compile(module, str(path), "exec"), namespace)  # noqa: S102 - the reference's own functions
    return namespace


def main(reference: Path) -> None:
    spec = importlib.util.spec_from_file_location("krn_formats", reference / "src/krn/data/formats.py")
    formats = importlib.util.module_from_spec(spec)
    sys.modules["krn_formats"] = formats
    spec.loader.exec_module(formats)

    emulator = lift(reference / "src/krn/emulator/emulate.py", ("fused", "accumulate", "any_valid", "_bfloat16"),
                    {"np": np})
    narrow = lift(reference / "src/krn/compiler/narrow.py",
                  ("_levels", "maximum_code", "nan_code", "reference_encode", "reference_decode"),
                  {"np": np, "math": __import__("math"), "FloatFormat": formats.FloatFormat, "ArrayLike": object})

    # ---- tile product through the emulator's accumulate -------------------------------------------------
    out: dict[str, np.ndarray] = {}
    shapes = [(50, 38, 70), (16, 8, 8), (33, 17, 56), (64, 64, 64), (130, 70, 100)]
    for index, (m, n, k) in enumerate(shapes):
        for dtype in ("f32", "f16", "bf16"):
            rng = np.random.default_rng(index if dtype == "f32" else index + 100)
            a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
            b = rng.uniform(-1, 1, (n, k)).astype(np.float32)  # b is (N, K): the product is a @ b^T
            if dtype == "f16":
                a, b = (x.astype(np.float16).astype(np.float32) for x in (a, b))
            elif dtype == "bf16":
                a, b = (emulator["_bfloat16"](x) for x in (a, b))
            acc = np.zeros((m, n), np.float32)
            emulator["accumulate"](acc, a, np.ascontiguousarray(b.T), None, None, None)
            key = f"{dtype}_{m}x{n}x{k}"
            out[f"{key}_a"], out[f"{key}_b"], out[f"{key}_c"] = a, b, acc
            out[f"{key}_c_bf16"] = emulator["_bfloat16"](acc)
    # the accumulator is re-read between k tiles: two chained calls equal one
    rng = np.random.default_rng(7)
    a, b = rng.standard_normal((24, 40), np.float32), rng.standard_normal((40, 16), np.float32)
    acc = np.zeros((24, 16), np.float32)
    emulator["accumulate"](acc, a[:, :24], b[:24], None, None, None)
    emulator["accumulate"](acc, a[:, 24:], b[24:], None, None, None)
    out["chained_a"], out["chained_b"], out["chained_c"] = a, b, acc
    specials = np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.0e38, -3.0e38, 1e-40, np.inf, -np.inf, np.nan,
                         65504.0, 0.1, -0.1], np.float32)
    out["bf16_in"], out["bf16_out"] = specials, emulator["_bfloat16"](specials)
    np.savez_compressed(HERE / "gemm_emulator.npz", **out)

    # ---- e4m3fn ----------------------------------------------------------------------------------------------
    fmt = formats.E4M3FN
    rng = np.random.default_rng(11)
    values = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * 64,
        rng.uniform(-500, 500, 2048).astype(np.float32),
        rng.standard_normal(1024).astype(np.float32) * 0.01,
        np.array([0.0, -0.0, 448.0, 449.0, 464.0, 480.0, 1e9, -1e9, np.inf, -np.inf, np.nan, 2.0**-9, 2.0**-10,
                  1.5 * 2.0**-9, 2.5 * 2.0**-9, 0.0009765625, 17.0, 18.0, 19.0, 20.0, 22.0, 26.0, 30.0], np.float32),
    ])
    np.savez_compressed(
        HERE / "e4m3.npz",
        table=np.asarray(fmt.table, np.float64),
        decode=narrow["reference_decode"](fmt, np.arange(256)),
        values=values,
        codes=narrow["reference_encode"](fmt, values),
        max=np.float64(fmt.max),
    )
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    main(Path(sys.argv[1]))
