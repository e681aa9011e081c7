"""Host-side mirror of Tempest's `Library` plugin protocol for the B200 kernels.

Tempest offers a kernel package its work through `Tempest.Compiler.Implement`
(src/Compiler/Implement/library.jl:9-105): a `Library` lists `templates`, the
cover matches groups to them and hands `supports` / `build` a `Binding` whose
arrays are `Strided` views (offset, sizes and strides in ELEMENTS of a device
buffer, column-major axes first-fastest); `build` returns `(launch,
description)`, `launch()` takes no arguments and only enqueues work on the
calling task's stream, and `repoint!(launch, value, buffer)` moves one
operand to another buffer (the pattern of ext/cuDNNExt.jl:145-218 and
ext/cuBLASExt.jl:247-268).

This module keeps those names, argument meanings and error behaviour
(`supports` answers False, `build` raises, nothing falls back to the CPU) so
that a Julia shim is a transliteration: each launch is one call into
libtempest_b200.so with `pointer(buffer) + offset * sizeof(eltype)`.

Buffers are anything with `data_ptr()` (a torch tensor) or a plain int device
address.  The stream is taken from `current_stream` (torch's current stream by
default), as a Tempest launch takes the task's.
"""
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Tuple

from . import lib

ELTYPES = {"Float32": (lib.F32, 4), "BFloat16": (lib.BF16, 2)}


def _torch_stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


current_stream: Callable[[], int] = _torch_stream


@dataclass(frozen=True)
class Template:
    """A function the library computes: its name, the Julia spelling Tempest
    would trace, and the named axes of each input (library.jl:21-42)."""
    name: str
    spelling: str
    inputs: Dict[str, Tuple[str, ...]]
    outputs: Tuple[str, ...]


@dataclass
class Strided:
    """An array of a binding (library.jl:44-59): `size`/`strides` in elements,
    first axis fastest; `buffer` None while only `supports` is asked."""
    eltype: str
    offset: int
    size: Tuple[int, ...]
    strides: Tuple[int, ...]
    buffer: Any = None
    value: int = 0

    def pointer(self) -> int:
        base = self.buffer if isinstance(self.buffer, int) else self.buffer.data_ptr()
        return base + self.offset * ELTYPES[self.eltype][1]


@dataclass
class Binding:
    """A group matched to one template (library.jl:61-72)."""
    template: str
    extents: Dict[str, int]
    arrays: Dict[str, Strided]


@dataclass
class Work:
    """The cost statement of one launch (src/Compiler/Implement/Implement.jl:61-82)."""
    bytes: int
    flops: float = 0.0
    blocks: int = 0
    launches: int = 1


@dataclass
class Target:
    """What of `CUDATarget` the kernels look at (src/Compiler/runtime/target.jl:71-75)."""
    device: int = 0
    online: bool = True
    deterministic: bool = True


def dense_columns(buffer, eltype, n, rows, value=0, offset=0, ld=None):
    """A Julia (n, rows) matrix stored densely (or with leading dimension ld)."""
    ld = n if ld is None else ld
    return Strided(eltype, offset, (n, rows), (1, ld), buffer, value)


def dense_vector(buffer, eltype, n, value=0, offset=0):
    return Strided(eltype, offset, (n,), (1,), buffer, value)


SOFTMAX = Template(
    "softmax_columns", "x -> exp.(x .- Tempest.logsumexp(x; dims = 1))",
    {"x": ("n", "rows")}, ("y",))
SOFTMAX_LSE = Template(
    "softmax_columns_lse", "x -> (l = Tempest.logsumexp(x; dims = 1); (exp.(x .- l), l))",
    {"x": ("n", "rows")}, ("y", "lse"))
SOFTMAX_PULLBACK = Template(
    "softmax_columns_pullback", "(y, g) -> (t = g .* y; t .- y .* sum(t; dims = 1))",
    {"y": ("n", "rows"), "g": ("n", "rows")}, ("dx",))
SOFTMAX_PULLBACK_RECOMPUTED = Template(
    "softmax_columns_pullback_recomputed",
    "(x, lse, g) -> (y = exp.(x .- lse); t = g .* y; t .- y .* sum(t; dims = 1))",
    {"x": ("n", "rows"), "lse": ("one", "rows"), "g": ("n", "rows")}, ("dx",))
LAYERNORM = Template(
    "layernorm",
    "(x, w) -> (m = sum(x; dims = 1) ./ size(x, 1); v = sum(abs2, x .- m; dims = 1) ./ size(x, 1); "
    "(x .- m) ./ sqrt.(v .+ eps) .* w)",
    {"x": ("n", "rows"), "w": ("n",)}, ("y",))
LAYERNORM_BIAS = Template(
    "layernorm_bias", "(x, w, b) -> layernorm(x, w) .+ b",
    {"x": ("n", "rows"), "w": ("n",), "b": ("n",)}, ("y",))
LAYERNORM_PULLBACK = Template(
    "layernorm_pullback", "(x, w, g) -> the tape's derivative of layernorm by x, w and b",
    {"x": ("n", "rows"), "w": ("n",), "g": ("n", "rows")}, ("dx", "dw", "db"))

ROW_TEMPLATES = (SOFTMAX, SOFTMAX_LSE, SOFTMAX_PULLBACK, SOFTMAX_PULLBACK_RECOMPUTED, LAYERNORM, LAYERNORM_BIAS,
                 LAYERNORM_PULLBACK)

_ROWOP = {
    "softmax_columns": lib.SOFTMAX_FWD, "softmax_columns_lse": lib.SOFTMAX_FWD,
    "softmax_columns_pullback": lib.SOFTMAX_BWD, "softmax_columns_pullback_recomputed": lib.SOFTMAX_BWD,
    "layernorm": lib.LAYERNORM_FWD, "layernorm_bias": lib.LAYERNORM_FWD, "layernorm_pullback": lib.LAYERNORM_BWD,
}
_STREAMS = {  # row-sized arrays read + written: the algorithmic traffic
    lib.SOFTMAX_FWD: 2, lib.SOFTMAX_BWD: 3, lib.LAYERNORM_FWD: 2, lib.LAYERNORM_BWD: 3,
}


class Resources:
    """Per-executable scratch (Implement.jl:141): one workspace, grown to the
    largest request while building, used by one launch at a time."""

    def __init__(self, allocate=None):
        self._allocate = allocate or _torch_allocate
        self.buffer = None
        self.bytes = 0

    def workspace(self, nbytes):
        if nbytes > self.bytes:
            self.buffer = self._allocate(nbytes)
            self.bytes = nbytes
        return self.buffer


def _torch_allocate(nbytes):
    import torch
    return torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")


class RowLaunch:
    """One fused row kernel on fixed operands.  Calling it enqueues the kernel;
    `repoint` replaces the buffer of one value (ext/cuDNNExt.jl:207-218)."""

    def __init__(self, binding: Binding, eps: float, workspace, workspace_bytes: int):
        self.binding = binding
        self.eps = eps
        self.workspace = workspace
        self.workspace_bytes = workspace_bytes
        first = next(iter(binding.arrays.values()))
        self.dtype = ELTYPES[first.eltype][0]
        self.n, self.rows = binding.extents["n"], binding.extents["rows"]

    def repoints(self) -> bool:
        return True

    def repoint(self, value: int, buffer) -> "RowLaunch":
        for s in self.binding.arrays.values():
            if s.value == value:
                s.buffer = buffer
        return self

    def _ptr(self, name) -> int:
        s = self.binding.arrays.get(name)
        return s.pointer() if s is not None else 0

    def _ld(self, name) -> int:
        s = self.binding.arrays[name]
        return s.strides[1] if len(s.strides) > 1 and s.size[1] > 1 else s.size[0]

    def __call__(self):
        a, t = self.binding.arrays, self.binding.template
        ws = self.workspace.data_ptr() if self.workspace is not None and self.workspace_bytes else 0
        stream = current_stream()
        if t in ("softmax_columns", "softmax_columns_lse"):
            stat = ELTYPES[a["lse"].eltype][0] if "lse" in a else lib.F32
            lib.softmax_fwd(self._ptr("x"), self._ptr("y"), self._ptr("lse"), self.n, self.rows, self._ld("x"),
                            self.dtype, stat, ws, self.workspace_bytes, stream)
        elif t == "softmax_columns_pullback":
            lib.softmax_bwd(self._ptr("y"), 0, self._ptr("g"), self._ptr("dx"), self.n, self.rows, self._ld("y"),
                            self.dtype, lib.F32, ws, self.workspace_bytes, stream)
        elif t == "softmax_columns_pullback_recomputed":
            stat = ELTYPES[a["lse"].eltype][0]
            lib.softmax_bwd(self._ptr("x"), self._ptr("lse"), self._ptr("g"), self._ptr("dx"), self.n, self.rows,
                            self._ld("x"), self.dtype, stat, ws, self.workspace_bytes, stream)
        elif t in ("layernorm", "layernorm_bias"):
            lib.layernorm_fwd(self._ptr("x"), self._ptr("w"), self._ptr("b"), self._ptr("y"), self._ptr("mean"),
                              self._ptr("rstd"), self.eps, self.n, self.rows, self._ld("x"), self.dtype, ws,
                              self.workspace_bytes, stream)
        elif t == "layernorm_pullback":
            lib.layernorm_bwd(self._ptr("x"), self._ptr("w"), self._ptr("g"), self._ptr("mean"), self._ptr("rstd"),
                              self._ptr("dx"), self._ptr("dw"), self._ptr("db"), self.eps, self.n, self.rows,
                              self._ld("x"), self.dtype, ws, self.workspace_bytes, stream)
        else:  # pragma: no cover - build() refuses unknown templates
            raise ValueError(t)


class B200Kernels:
    """The library (`<: Library`): which templates it computes, whether it takes
    a binding, what a launch costs, and the launch itself."""

    def __init__(self, eps: float = 1.0e-5):
        self.eps = eps

    def templates(self, target: Target):
        # the row kernels fold each statistic in one pass, which a target that
        # forbids the online rewrites does not permit (ext/cuDNNExt.jl:60-62)
        return ROW_TEMPLATES if target.online else ()

    def resources(self, target: Target) -> Resources:
        return Resources()

    def supports(self, target: Target, b: Binding) -> bool:
        if b.template not in _ROWOP:
            return False
        n, rows = b.extents.get("n", 0), b.extents.get("rows", 0)
        if n < 0 or rows < 0 or n > 1 << 30:
            return False
        eltype = None
        for name, s in b.arrays.items():
            if name in ("mean", "rstd"):
                if s.eltype != "Float32":
                    return False
                continue
            if s.eltype not in ELTYPES:
                return False
            if name != "lse":
                if eltype not in (None, s.eltype):
                    return False
                eltype = s.eltype
            if s.strides and s.strides[0] != 1 and s.size[0] > 1:
                return False  # the folded axis must be contiguous
        lds = {s.strides[1] for name, s in b.arrays.items() if len(s.size) == 2 and s.size[0] == n and s.size[1] > 1}
        if len(lds) > 1:
            return False  # one leading dimension for all row-shaped operands
        if _ROWOP[b.template] == lib.LAYERNORM_BWD and n > 8192:
            return False
        return True

    def estimate(self, target: Target, b: Binding):
        first = next(iter(b.arrays.values()))
        size = ELTYPES[first.eltype][1]
        n, rows = b.extents["n"], b.extents["rows"]
        op = _ROWOP[b.template]
        launches = 2 if (op == lib.LAYERNORM_BWD or n > 16384) else 1
        return [Work(bytes=_STREAMS[op] * n * rows * size, blocks=rows, launches=launches)]

    def build(self, target: Target, b: Binding, resources: Optional[Resources] = None):
        if not self.supports(target, b):
            raise ValueError(f"B200Kernels does not compute this binding of {b.template}")
        for s in b.arrays.values():
            if s.buffer is None:
                raise ValueError("build needs every array's buffer")
        first = next(iter(b.arrays.values()))
        dtype = ELTYPES[first.eltype][0]
        n, rows = b.extents["n"], b.extents["rows"]
        need = lib.rowop_workspace_bytes(_ROWOP[b.template], n, rows, dtype)
        resources = resources if resources is not None else Resources()
        ws = resources.workspace(need) if need else None
        launch = RowLaunch(b, self.eps, ws, need)
        schedule = "split" if n > 16384 else "resident"
        return launch, f"B200 {b.template}, {rows} rows of {n} {first.eltype}, {schedule}"
