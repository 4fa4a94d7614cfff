"""Host logic of the kernel-language surface, without a GPU: capture of the tile subset, launch-geometry inference
(src/krn/compiler/space.py semantics, tests/frontend/test_launch_inference.py cases), the pattern recogniser and
the refusal conventions."""

from __future__ import annotations

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import Blocks, CaptureError, LaunchError, TargetError, Tiles
from krn_b200.compiler import ir
from krn_b200.compiler.capture import capture
from krn_b200.compiler.recognise import AttentionPlan, GemmPlan, recognise
from krn_b200.compiler.space import geometry
from tests.kernels import tile_kernels as K


def test_public_surface_names() -> None:
    """The names a tile-kernel file imports from krn (src/krn/__init__.py:15-242)."""
    for name in ("kernel", "struct", "Const", "AUTO", "T", "Matrix", "Tensor", "Tile", "QMatrix", "Tiles", "Blocks",
                 "Items", "block", "pipelined", "zeros", "where", "arange", "maximum", "host", "configure", "config",
                 "hw", "targets", "formats", "errors", "bf16", "f8e4m3fn", "f32"):
        assert hasattr(krn, name), name
    assert krn.T.bf16 is krn.bf16 and krn.T.f32(2.5).value == 2.5
    assert krn.Matrix[krn.bf16].rank == 2 and krn.Tensor[krn.T.f16, int, int, int].rank == 3
    target = krn.targets.Target.of("sm_100a")
    assert target.has(krn.targets.Feature.TENSOR_MEMORY) and target.mma_native(krn.f8e4m3fn)
    assert krn.formats.FP8FN().block == (1, 128) and krn.formats.E4M3FN.max == 448.0


@pytest.mark.parametrize("shape,tile,want", [((50, 38), (16, 16), Blocks(3, 4)), ((1, 1), (8, 16), Blocks(1, 1)),
                                             ((9, 17), (8, 16), Blocks(2, 2)), ((2, 200), (1, 16), Blocks(13, 2))])
def test_tiles_blocks(shape, tile, want) -> None:
    """`Tiles(shape, tile).blocks`: ceiling division, last axis along x (src/krn/frontend/geometry.py:28-41)."""
    assert Tiles(shape, tile).blocks == want


def test_gemm_capture_ir_and_inferred_geometry() -> None:
    captured = capture(K.matmul_nt.fn, K.Tiling(bm=64, bn=32, bk=16))
    loop = captured.body[1]
    assert isinstance(loop, ir.For) and loop.pipelined and loop.step == 16 and loop.stop == ir.Dim("a", 1)
    step = loop.body[0]
    assert isinstance(step, ir.Accumulate) and isinstance(step.rhs, ir.Transpose) and step.rhs.shape == (16, 32)
    axes = {axis.grid: axis for axis in captured.space}
    assert {g: a.tile for g, a in axes.items()} == {"y": 64, "x": 32}
    assert axes["y"].extents == (ir.Dim("c", 0),) and axes["x"].extents == (ir.Dim("c", 1),)  # stored extents win
    args = [K.Tiling(), np.zeros((50, 70)), np.zeros((38, 70)), np.zeros((50, 38))]
    assert geometry(captured, args) == Tiles((50, 38), (64, 32)).blocks
    args[3] = np.zeros((1, 1))
    assert geometry(captured, args) == Blocks(1, 1)  # a launch always has one block at least


def test_recognise_gemm_forms() -> None:
    plan = recognise(capture(K.matmul_nt.fn, K.Tiling()))
    assert plan == GemmPlan("a", "b", "c", krn.bf16, krn.bf16, (128, 128, 32))
    plan = recognise(capture(K.matmul_nt_f16_f32.fn))
    assert plan == GemmPlan("a", "b", "c", krn.f16, krn.f32, (32, 64, 16))
    # the reference example's own form, b stored (K, N)
    plan = recognise(capture(K.matmul_nn.fn, K.Tiling()))
    assert plan == GemmPlan("a", "b", "c", krn.f16, krn.f16, (128, 128, 32), transposed_b=False)
    with pytest.raises(TargetError) as error:
        recognise(capture(K.matmul_mixed.fn, K.Tiling()))
    text = str(error.value)
    assert "is not available on sm_100a" in text and "Instead:" in text and "convert one operand" in text
    assert "tile_kernels.py" in text and "^" in text  # compiler-style location with a caret


def test_recognise_fp8_pairs() -> None:
    """fp8 pairs that are direct tile loads are a product of their own, each operand in its own format
    (src/krn/compiler/capture.py:3185-3192)."""
    plan = recognise(capture(K.fp8_pair_kn.fn))
    assert isinstance(plan, GemmPlan) and not plan.transposed_b
    assert (plan.operand.name, plan.operand_b.name, plan.output.name) == ("f8e4m3fn", "f8e5m2", "f32")
    plan = recognise(capture(K.fp8_pair_nt.fn))
    assert plan.transposed_b and (plan.operand.name, plan.operand_b.name, plan.output.name) == ("f8e4m3fn", "f8e4m3fn", "bf16")


@pytest.mark.parametrize("near_miss", ["attention_old_maximum_in_exponent", "attention_sum_starts_at_one",
                                       "attention_correction_swapped"])
def test_near_misses_of_the_attention_pattern_are_refused(near_miss) -> None:
    """A body that differs from the example's online softmax in one operand is not standard attention: it must be refused
    with the four-part message, never run as the prebuilt kernel ("never ignore it silently")."""
    with pytest.raises(TargetError) as error:
        recognise(capture(getattr(K, near_miss).fn, K.Heads()))
    assert "is not available on sm_100a" in str(error.value) and "Instead:" in str(error.value)


def test_recognise_library_epilogues() -> None:
    """The reference's `matmul_epilogue` kernel (src/krn/lib/lib_kernels.py:30-48) under each flag set."""
    tile = (64, 64, 32)
    plan = recognise(capture(K.matmul_epilogue.fn, K.MatmulTiling()))
    assert plan == GemmPlan("a", "b", "out", krn.f16, krn.f16, tile, False)
    plan = recognise(capture(K.matmul_epilogue.fn, K.MatmulTiling(bias=True, gelu=True)))
    assert plan == GemmPlan("a", "b", "out", krn.f16, krn.f16, tile, False, "bias", "gelu")
    assert recognise(capture(K.matmul_epilogue.fn, K.MatmulTiling(silu=True))).activation == "silu"
    with pytest.raises(TargetError, match="relu followed by gelu"):
        recognise(capture(K.matmul_epilogue.fn, K.MatmulTiling(relu=True, gelu=True)))


def test_family_selection_audit_and_pinning() -> None:
    """Most specific matching rule wins, ties raise, `run.variants` pins (the reference's family rules,
    src/krn/frontend/variants.py:47-112, on the family of examples/04_libraries/03_gemm_variants.py)."""
    from krn_b200 import AmbiguousVariant, Feature, targets

    F = Feature
    b200 = targets.Target.of("sm_100a")
    hopper = targets.described(targets.Nvidia, "sm_90a", {F.TENSOR_CORE, F.ASYNC_COPY, F.BULK_COPY, F.ASYNC_MMA, F.CLUSTERS})
    ampere = targets.described(targets.Nvidia, "sm_80", {F.TENSOR_CORE, F.ASYNC_COPY})
    mi300 = targets.described(targets.AMD, "gfx942", {F.TENSOR_CORE, F.ASYNC_COPY})
    cpu = targets.described(targets.CPU, "x86_64", set())
    assert K.gemm.audit([b200, hopper, ampere, mi300, cpu]) == {
        "sm_100a": "gemm_tensor_memory", "sm_90a": "gemm_hopper", "sm_80": "portable", "gfx942": "gemm_amd",
        "x86_64": "portable"}
    selection = K.gemm.select(b200)
    assert selection.kernel is K.gemm_tensor_memory and "most specific" in selection.reason
    assert K.gemm.select(cpu).reason == "no variant applies to x86_64"
    # the selected variant is the tile product with row-major b, its space= and schedule= intents accepted
    plan = recognise(capture(selection.kernel.fn, K.FamilyTiling()))
    assert plan == GemmPlan("a", "b", "c", krn.f16, krn.f32, (128, 128, 64), False)
    with krn.configure(**{"run.variants": {"gemm": "portable"}}):
        assert K.gemm.select(b200).name == "portable" and K.gemm.select(b200).reason == "pinned by run.variants"
    with krn.configure(**{"run.variants": {"gemm": "gemm_hopper"}}):
        assert K.gemm.select(b200).kernel is K.gemm_hopper
    with krn.configure(**{"run.variants": {"gemm": "nonesuch"}}), pytest.raises(LookupError, match="nonesuch"):
        K.gemm.select(b200)

    @K.gemm.variant(targets.Nvidia, requires={F.BLOCK_SCALED_MMA})
    def gemm_rival(t: K.FamilyTiling, a, b, c) -> None: ...

    try:
        with pytest.raises(AmbiguousVariant, match="gemm on sm_100a: gemm_rival, gemm_tensor_memory tie"):
            K.gemm.select(b200)
        assert K.gemm.select(hopper).name == "gemm_hopper"  # the tie only exists where both rules match
    finally:
        del K.gemm.variants["gemm_rival"]


def test_library_candidate_protocol() -> None:
    """Names, refusals and flags of the one matmul candidate (protocol of src/krn/lib/lib.py:201-235)."""
    from krn_b200 import lib

    candidate = lib.CANDIDATES[0]
    assert (candidate.name, candidate.op, candidate.origin) == ("b200", lib.Op.MATMUL, lib.Origin.OURS)
    assert [e.value for e in lib.Epilogue] == ["none", "bias", "relu", "gelu", "bias_relu", "bias_gelu", "silu"]
    assert lib.FLAGS[lib.Epilogue.BIAS_GELU] == 1 | 4 and lib.FLAGS[lib.Epilogue.SILU] == 6
    problem = lib.Problem(lib.Op.MATMUL, (krn.bf16, krn.bf16, krn.f32), (8, 8, 8), lib.LibOptions())
    assert candidate.refusal(problem, "sm_100a") is None
    mixed = lib.Problem(lib.Op.MATMUL, (krn.bf16, krn.f16, krn.f32), (8, 8, 8), lib.LibOptions())
    assert "got bf16 @ f16" in candidate.refusal(mixed, "sm_100a")
    carved = lib.Problem(lib.Op.MATMUL, (krn.f16, krn.f16, krn.f16), (8, 8, 8), lib.LibOptions(sm_count=64))
    assert "sm_count" in candidate.refusal(carved, "sm_100a")
    relaxed = lib.Problem(lib.Op.MATMUL, (krn.f16, krn.f16, krn.f16), (8, 8, 8), lib.LibOptions(), precision=lib.Compute.TF32)
    assert "tf32" in candidate.refusal(relaxed, "sm_100a")
    assert lib.product_type(krn.f16, krn.f16) == krn.f16 and lib.product_type(krn.f16, krn.bf16) == krn.f32


@pytest.mark.parametrize("causal", [False, True])
def test_recognise_flash_attention_example(causal) -> None:
    captured = capture(K.flash_attention.fn, K.Heads(causal=causal, d=128))
    plan = recognise(captured)
    assert plan == AttentionPlan("q", "k", "v", "o", ("scale",), krn.T.f16, 128, causal, False, 1, (16, 16))
    # rows come from x only; the head is a scalar index, so y needs launch= as in the example
    assert [(a.grid, a.tile) for a in captured.space] == [("x", 16)]
    shapes = [K.Heads(), *(np.zeros((2, 200, 128)) for _ in range(4)), 1.0]
    assert geometry(captured, shapes) == Blocks(13)


def test_recognise_grouped_batched_attention() -> None:
    plan = recognise(capture(K.grouped_causal_attention.fn, K.Grouped()))
    assert isinstance(plan, AttentionPlan) and plan.batched and plan.group == 4 and plan.causal and plan.d == 128


def test_refusals_follow_the_reference_conventions() -> None:
    with pytest.raises(TargetError) as error:
        recognise(capture(K.row_scale.fn))
    assert error.value.feature == "kernel `row_scale`" and error.value.target == "sm_100a"
    assert "no code generator" in error.value.reason
    with pytest.raises(CaptureError, match="capture-time constant"):
        capture(K.data_dependent_branch.fn)
    with pytest.raises(CaptureError, match="loaded directly"):
        capture(K.fp8_needs_direct_loads.fn)
    with pytest.raises(TypeError, match="brackets take a configuration"):
        K.matmul_nt[Tiles((4, 4), (2, 2))]
    with pytest.raises(RuntimeError, match="device function"):
        krn.zeros(krn.f32, 4, 4)


def test_launch_errors() -> None:
    captured = capture(K.mismatched_extents.fn)
    with pytest.raises(LaunchError) as error:
        geometry(captured, [np.zeros((37, 8)), np.zeros((9, 8)), np.zeros((37, 8)), np.zeros((9, 8))])
    assert "mismatched_extents" in str(error.value) and "launch=" in str(error.value) and "[9, 37]" in str(error.value)
    assert geometry(captured, [np.zeros((9, 8))] * 4) == Blocks(1, 2)  # and recovers once the shapes agree
    with pytest.raises(LaunchError, match="more than one size"):
        geometry(capture(K.conflicting_tiles.fn), [np.zeros((16, 4)), np.zeros((16, 4))])


def test_settings_and_no_cpu_fallback(monkeypatch) -> None:
    from krn_b200.errors import SettingError
    from krn_b200.runtime import settings

    assert krn.config.run.target == "sm_100a"
    with pytest.raises(SettingError, match="no CPU fallback"):
        krn.configure("run.target", "avx512")
    with krn.configure("run.graphs", False):
        assert krn.config.run.graphs is False
    assert krn.config.run.graphs is True
    pinned = K.Tiling(bm=64)
    with krn.configure(**{"run__config": {"matmul_nt": pinned}}):
        assert settings.current_settings().configuration("matmul_nt", K.Tiling) is pinned
    assert settings.current_settings().configuration("matmul_nt", K.Tiling) == K.Tiling()
    import torch

    if not torch.cuda.is_available():
        with pytest.raises(TargetError, match="no CPU fallback"):
            krn.host.Device.current()


def test_streaming_panels_cover_the_extent_on_tile_boundaries() -> None:
    """Panel ranges of the host-operand streaming: contiguous, covering, boundaries on the requested multiple."""
    from krn_b200.streaming import _panels

    for extent, count, multiple in ((8192, 16, 256), (3584, 8, 256), (1024, 8, 256), (1100, 3, 256), (300, 16, 256), (8, 8, 1),
                                    (28672, 16, 256)):
        ranges = _panels(extent, count, multiple)
        assert ranges[0][0] == 0 and ranges[-1][1] == extent and len(ranges) <= count
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:])) and all(hi > lo for lo, hi in ranges)
        assert all(lo % multiple == 0 for lo, _ in ranges)
