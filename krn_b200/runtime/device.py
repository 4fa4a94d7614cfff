"""The B200 device: device memory, streams and events through torch (plumbing only), launches through the C ABI.

What the reference's CUDA device does with NVRTC and `cuLaunchKernel` (src/krn/runtime/cuda_backend.py:297-483,
675-747) happens here without a compiler: the launcher captures the kernel once per signature
(src/krn/runtime/runtime.py:523-582), the recogniser names the prebuilt kernel, and a call is one ctypes call that
enqueues on the current stream. There is no other device and no CPU fallback: without a compute-capability 10.x GPU
`Device.current()` raises."""

from __future__ import annotations

import math
import threading
import time
from typing import Any, Callable

import numpy as np

from krn_b200.compiler import ir
from krn_b200.compiler.capture import capture
from krn_b200.compiler.recognise import AttentionPlan, GemmPlan, recognise
from krn_b200.compiler.space import geometry as infer_geometry
from krn_b200.errors import CUDAError, LaunchError, TargetError
from krn_b200.frontend.geometry import Blocks, Items, Tiles, ceildiv
from krn_b200.frontend.types import BY_NAME, Dtype, Scalar, bf16, f8e4m3fn
from krn_b200.runtime import api, calls, native
from krn_b200.runtime.settings import current_settings

_TORCH_NAMES = {"f32": "float32", "f16": "float16", "bf16": "bfloat16", "f64": "float64", "i32": "int32", "i64": "int64",
                "i16": "int16", "i8": "int8", "u8": "uint8", "bool": "bool", "f8e4m3fn": "float8_e4m3fn",
                "f8e5m2": "float8_e5m2", "u16": "uint16", "u32": "uint32", "u64": "uint64"}


def _torch():
    import torch

    return torch


def _element_of(tensor) -> Dtype:
    name = str(tensor.dtype).replace("torch.", "")
    for ours, theirs in _TORCH_NAMES.items():
        if theirs == name:
            return BY_NAME[ours]
    raise TypeError(f"no element type for torch.{name}")


class DeviceTensor:
    """C-contiguous (or strided-view) device memory with the reference's tensor attributes: `pointer`, `shape`,
    `strides` (in elements), `nbytes`, `element`, `__cuda_array_interface__`, `to_host()`
    (src/krn/runtime/cuda_backend.py:205-248)."""

    def __init__(self, data, element: Dtype | None = None) -> None:
        self.data = data
        self.element = element or _element_of(data)

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.data.shape)

    @property
    def strides(self) -> tuple[int, ...]:
        return tuple(self.data.stride())

    @property
    def pointer(self) -> int:
        return int(self.data.data_ptr())

    @property
    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    @property
    def __cuda_array_interface__(self) -> dict:
        return self.data.__cuda_array_interface__

    def to_host(self) -> np.ndarray:
        """A host copy. bf16 and fp8 come back as `ml_dtypes` arrays when that package is present, else as their
        storage words (uint16 / uint8), as the reference's tests handle bf16 (tests/compiler/test_tensor_cores.py:4)."""
        torch = _torch()
        data = self.data.detach().contiguous().cpu()
        if self.element == bf16 or self.element.name in ("f8e4m3fn", "f8e5m2"):
            words = data.view(torch.int16 if self.element == bf16 else torch.uint8).numpy()
            words = words.view(np.uint16) if self.element == bf16 else words
            try:
                import ml_dtypes

                return words.view({"bf16": ml_dtypes.bfloat16, "f8e4m3fn": ml_dtypes.float8_e4m3fn,
                                   "f8e5m2": ml_dtypes.float8_e5m2}[self.element.name])
            except ImportError:
                return words
        return data.numpy()

    def __getitem__(self, item) -> "DeviceTensor":
        return DeviceTensor(self.data[item], self.element)

    def __repr__(self) -> str:
        return f"DeviceTensor({self.element}, {list(self.shape)})"


def _raw(value: Any):
    """The torch tensor behind a DeviceTensor (torch tensors pass through)."""
    return value.data if isinstance(value, DeviceTensor) else value


class B200Event(api.Event):
    def __init__(self, stream: "B200Stream") -> None:
        torch = _torch()
        self._event = torch.cuda.Event(enable_timing=True)
        self._event.record(stream.raw)
        self._error: BaseException | None = None
        self._checked = False

    def done(self) -> bool:
        finished = bool(self._event.query())
        if finished and not self._checked:
            self._checked = True
            code, site, block = native.device_status()
            if code != native.OK:
                self._error = CUDAError(f"KRN_B200_ERR_DEVICE_TIMEOUT: a bounded device-side wait expired at site "
                                        f"{site} in block {block}")
        return finished

    @property
    def error(self) -> BaseException | None:
        return self._error

    def wait(self, timeout: float | None = None) -> None:
        deadline = None if timeout is None else time.monotonic() + timeout
        while not self.done():
            if deadline is not None and time.monotonic() > deadline:
                raise TimeoutError(f"event not complete after {timeout} s")
            time.sleep(0.0002)
        if self._error is not None:
            raise self._error

    def elapsed_since(self, earlier: api.Event) -> float:
        assert isinstance(earlier, B200Event)
        return float(earlier._event.elapsed_time(self._event))


class B200Stream(api.Stream):
    def __init__(self, device: "B200Device", raw) -> None:
        self.device, self.raw = device, raw

    def record(self) -> B200Event:
        return B200Event(self)

    def wait(self, event: api.Event) -> None:
        assert isinstance(event, B200Event)
        self.raw.wait_event(event._event)

    def __cuda_stream__(self) -> tuple[int, int]:
        return (0, int(self.raw.cuda_stream))

    @property
    def handle(self) -> int:
        return int(self.raw.cuda_stream)


class Call:
    """One validated launch: a closure over the C-ABI call and what `explain` prints."""

    def __init__(self, run: Callable[[B200Stream], None], explanation: api.Explanation) -> None:
        self.run, self.explanation = run, explanation


class B200Launcher(api.Launcher):
    def __init__(self, device: "B200Device", kernel, launch) -> None:
        self.device, self.kernel, self.launch = device, kernel, launch
        self._plans = device._plans.setdefault(id(kernel), {})  # shared by every launcher of this kernel
        self._lock = device._plan_lock

    # ---- specialisation --------------------------------------------------------------------------------------------

    def _signature(self, args: tuple) -> tuple:
        key = [current_settings().key()]
        for value in args:
            raw = _raw(value)
            if hasattr(raw, "shape") and hasattr(raw, "dtype"):
                key.append((str(raw.dtype), len(raw.shape)))
            elif isinstance(value, (int, float, Scalar)):
                key.append(type(value).__name__)
            else:
                key.append(value)  # a configuration struct: its Const values are the specialisation
        return tuple(key)

    def _plan(self, args: tuple) -> tuple[ir.Kernel, Any]:
        key = self._signature(args)
        with self._lock:
            if key not in self._plans:
                config = args[0] if self.kernel.configuration is not None and args else None
                captured = capture(self.kernel.fn, config)
                self._plans[key] = (captured, recognise(captured))
            return self._plans[key]

    # ---- encoding ------------------------------------------------------------------------------------------------------

    def _encode(self, args: tuple) -> Call:
        captured, plan = self._plan(args)
        if len(args) != len(captured.params):
            raise TypeError(f"{captured.name} takes {len(captured.params)} arguments, got {len(args)}")
        named = dict(zip((name for name, _ in captured.params), args))
        for name, kind in captured.params:
            if isinstance(kind, ir.TensorParam):
                raw = _raw(named[name])
                if not hasattr(raw, "data_ptr"):
                    raise TypeError(f"{captured.name}: `{name}` must be a device tensor (device.to_device(array))")
                if len(raw.shape) != kind.rank or _element_of(raw) != kind.dtype:
                    raise TypeError(f"{captured.name}: `{name}` is declared {kind.dtype} rank {kind.rank}, got "
                                    f"{_element_of(raw)} rank {len(raw.shape)}")
        shapes = [np.empty(_raw(v).shape, np.uint8) if hasattr(_raw(v), "data_ptr") else v for v in args]
        launch = self.launch.blocks if isinstance(self.launch, Tiles) else self.launch
        if isinstance(plan, GemmPlan):
            return self._gemm(captured, plan, named, shapes, launch)
        return self._attention(captured, plan, named, shapes, launch)

    def _gemm(self, captured, plan: GemmPlan, named, shapes, launch) -> Call:
        a, b, c = (_raw(named[n]) for n in (plan.a, plan.b, plan.c))
        needed = infer_geometry(captured, shapes)
        self._check_cover(captured, launch, needed)
        b_k, b_n = (b.shape[1], b.shape[0]) if plan.transposed_b else (b.shape[0], b.shape[1])
        if a.shape[1] != b_k or tuple(c.shape) != (a.shape[0], b_n):
            raise ValueError(f"{captured.name}: shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, "
                             f"c {tuple(c.shape)}")
        fp8 = plan.operand.name in ("f8e4m3fn", "f8e5m2")
        operands = f"{plan.operand} @ {plan.operand_b}" if fp8 else f"{plan.operand} operands"
        entry = ("krn_b200_gemm_fp8" if fp8 else "krn_b200_matmul" if plan.bias or plan.activation else
                 f"krn_b200_gemm_{'tn' if plan.transposed_b else 'nn'}")
        explanation = api.Explanation(
            captured.name, f"tile matrix product c = a @ b{'^T' if plan.transposed_b else ''}, {operands}, "
            f"{plan.output} output, declared tile {plan.tile}", launch or needed,
            entry + " (tcgen05, 256x256 CTA-pair tiles)",
            ("the library chooses its own CTA tiling; the declared tile only shapes the inferred geometry",))
        if fp8:
            return Call(lambda stream: calls.gemm_fp8(a, b, c, b_kn=not plan.transposed_b, stream=stream.raw), explanation)
        if plan.bias is None and plan.activation is None:
            product = calls.gemm_tn if plan.transposed_b else calls.gemm_nn
            return Call(lambda stream: product(a, b, c, stream.raw), explanation)
        bias = _raw(named[plan.bias]) if plan.bias is not None else None
        flags = (1 if bias is not None else 0) | {None: 0, "relu": 2, "gelu": 4, "silu": 6}[plan.activation]
        if bias is not None and tuple(bias.shape) != (c.shape[1],):
            raise ValueError(f"{captured.name}: the bias has {tuple(bias.shape)} elements for {c.shape[1]} columns")
        return Call(lambda stream: calls.matmul(a, b, c, b_kn=not plan.transposed_b, epilogue=flags, bias=bias,
                                                stream=stream.raw), explanation)

    def _attention(self, captured, plan: AttentionPlan, named, shapes, launch) -> Call:
        q, k, v, o = (_raw(named[n]) for n in (plan.q, plan.k, plan.v, plan.o))
        scale = named[plan.scale[0]]
        scale = float(scale.value) if isinstance(scale, Scalar) else float(scale)
        if not plan.batched:
            q, k, v, o = (t.unsqueeze(0) for t in (q, k, v, o))
        batch, hq, seq, d = q.shape
        if d != plan.d or k.shape[3] != d or k.shape[1] * plan.group != hq or tuple(v.shape) != tuple(k.shape) \
                or tuple(o.shape) != tuple(q.shape) or k.shape[0] != batch:
            raise ValueError(f"{captured.name}: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)} do not fit "
                             f"d = {plan.d} and {plan.group} q heads per kv head")
        if plan.causal and k.shape[2] != seq:
            raise ValueError(f"{captured.name}: the causal mask compares positions of equally long sequences")
        needed = Blocks(ceildiv(seq, plan.tile[0]), hq, batch)
        self._check_cover(captured, launch, needed)
        explanation = api.Explanation(
            captured.name, f"flash attention forward, {plan.dtype}, d = {plan.d}, causal = {plan.causal}, "
            f"{plan.group} q head(s) per kv head", launch or needed,
            "krn_b200_attn_fwd (tcgen05, S/P/O in tensor memory)",
            ("the library tiles queries by 2 x 128 rows and keys by 128; the declared tile only shapes the geometry",))
        return Call(lambda stream: calls.attention_forward(q, k, v, o, scale, plan.causal, stream.raw), explanation)

    @staticmethod
    def _check_cover(captured, launch, needed) -> None:
        if launch is None or isinstance(needed, Items):
            return
        if isinstance(launch, Items):
            raise LaunchError(captured.name, "a tile kernel is launched in blocks, not items")
        if (launch.x, launch.y, launch.z) != (needed.x, needed.y, needed.z):
            raise TargetError(f"launch={launch}", "sm_100a", f"the prebuilt kernel computes the whole output, which "
                              f"takes {needed}", "omit `launch=` or pass the geometry that covers the output")

    # ---- Launcher ------------------------------------------------------------------------------------------------------

    def __call__(self, *args: Any) -> None:
        self._encode(args).run(self.device.current_stream())

    def submit(self, *args: Any) -> api.Event:
        stream = self.device.current_stream()
        self._encode(args).run(stream)
        return stream.record()

    def explain(self, *args: Any) -> api.Explanation:
        return self._encode(args).explanation

    def bind(self, *args: Any) -> "B200Bound":
        return B200Bound(self, args)


class B200Bound(api.Bound):
    def __init__(self, launcher: B200Launcher, args: tuple) -> None:
        self.launcher = launcher
        self.call = launcher._encode(args)

    def __call__(self) -> None:
        self.call.run(self.launcher.device.current_stream())

    def submit(self) -> api.Event:
        stream = self.launcher.device.current_stream()
        self.call.run(stream)
        return stream.record()

    def rebind(self, *args: Any) -> None:
        self.call = self.launcher._encode(args)


class B200Graph(api.Graph):
    """Stream capture of everything `fn(*args)` launches; replay is one `cudaGraphLaunch`. The function runs once
    uncaptured first, so one-time set-up of the kernel library (function attributes, the status word) happens outside
    the capture (src/krn/runtime/cuda_backend.py:486-545 records by stream capture too)."""

    def __init__(self, device: "B200Device", fn: Callable[..., None], args: tuple) -> None:
        torch = _torch()
        self.device, self.args = device, args
        side = B200Stream(device, torch.cuda.Stream())
        side.raw.wait_stream(torch.cuda.current_stream())
        with side, torch.cuda.stream(side.raw):
            fn(*args)
        side.raw.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with side, torch.cuda.graph(self.graph, stream=side.raw):
            fn(*args)

    def __call__(self, *args: Any) -> None:
        if args and any(a is not b for a, b in zip(args, self.args)):
            raise TargetError("replaying a graph with new arguments", "sm_100a",
                              "a CUDA graph holds the recorded addresses", "record a new graph for new arguments")
        torch = _torch()
        with torch.cuda.stream(self.device.current_stream().raw):
            self.graph.replay()

    def submit(self, *args: Any) -> api.Event:
        self(*args)
        return self.device.current_stream().record()


class B200Device(api.Device):
    def __init__(self, ordinal: int = 0) -> None:
        torch = _torch()
        from krn_b200.targets import Target

        self.ordinal = ordinal
        self.target = Target.of("sm_100a")
        self._default = B200Stream(self, torch.cuda.default_stream(ordinal))
        self._plans: dict[int, dict[tuple, tuple[ir.Kernel, Any]]] = {}
        self._plan_lock = threading.Lock()
        self._launchers: dict[tuple, B200Launcher] = {}
        native.library()  # LibraryNotFound here if the kernel library is not built: there is no fallback

    @property
    def default_stream(self) -> B200Stream:
        return self._default

    def current_stream(self) -> B200Stream:
        stream = api.current_stream.get()
        return stream if isinstance(stream, B200Stream) else self._default

    def stream(self) -> B200Stream:
        return B200Stream(self, _torch().cuda.Stream(self.ordinal))

    def empty(self, dtype: Dtype, *shape: int) -> DeviceTensor:
        torch = _torch()
        if not isinstance(dtype, Dtype) or dtype.name not in _TORCH_NAMES:
            raise TypeError(f"device.empty takes an element type, got {dtype!r}")
        return DeviceTensor(torch.empty(shape, device=f"cuda:{self.ordinal}", dtype=getattr(torch, _TORCH_NAMES[dtype.name])),
                            dtype)

    def to_device(self, array: Any, element: Dtype | None = None) -> DeviceTensor:
        """A device copy of a host array with the element type of the array. `ml_dtypes` bfloat16 / float8_e4m3fn
        arrays keep their type; `element=` reinterprets storage words (uint16 as bf16, uint8 as e4m3)."""
        torch = _torch()
        array = np.ascontiguousarray(array)
        name = array.dtype.name
        if name == "bfloat16":
            array, element = array.view(np.uint16), bf16
        elif name == "float8_e4m3fn":
            array, element = array.view(np.uint8), f8e4m3fn
        elif name == "float8_e5m2":
            array, element = array.view(np.uint8), BY_NAME["f8e5m2"]
        if array.dtype == np.uint16:
            tensor = torch.from_numpy(array.view(np.int16)).to(f"cuda:{self.ordinal}", non_blocking=True)
            tensor = tensor.view(torch.bfloat16) if element == bf16 else tensor.view(torch.uint16)
        else:
            tensor = torch.from_numpy(array).to(f"cuda:{self.ordinal}", non_blocking=True)
            if element == f8e4m3fn:
                tensor = tensor.view(torch.float8_e4m3fn)
            elif element is not None and element.name == "f8e5m2":
                tensor = tensor.view(torch.float8_e5m2)
        return DeviceTensor(tensor, element)

    def launcher(self, kernel, launch=None) -> B200Launcher:
        """Capture on first use and cache by specialisation; with no launch, geometry is inferred on every call."""
        key = (id(kernel), launch)
        if key not in self._launchers:
            self._launchers[key] = B200Launcher(self, kernel, launch)
        return self._launchers[key]

    def graph(self, fn: Callable[..., None], *args: Any) -> api.Graph:
        if not current_settings().run.graphs:
            class Plain(api.Graph):  # run.graphs=False selects plain launches (src/krn/runtime/api.py:225-231)
                def __call__(inner, *a: Any) -> None:
                    fn(*(a or args))

                def submit(inner, *a: Any) -> api.Event:
                    fn(*(a or args))
                    return self.current_stream().record()

            return Plain()
        return B200Graph(self, fn, args)

    async def synchronize(self) -> None:
        await self._default.record()
        _torch().cuda.synchronize(self.ordinal)
        native.raise_device_status()


_DEVICE: B200Device | None = None
_DEVICE_LOCK = threading.Lock()


def default_device() -> B200Device:
    global _DEVICE
    with _DEVICE_LOCK:
        if _DEVICE is None:
            target = current_settings().run.target
            torch = _torch()
            if not torch.cuda.is_available():
                raise TargetError(f"a {target} device", "this machine", "no CUDA device is visible and this build has "
                                  "no CPU fallback for the tile path", "run on a B200")
            major, minor = torch.cuda.get_device_capability(0)
            if major != 10:
                raise TargetError("the prebuilt tcgen05 kernels", f"sm_{major}{minor}", "the kernel library holds "
                                  "sm_100a code only", "run on a B200 (compute capability 10.x)")
            _DEVICE = B200Device(0)
        return _DEVICE
