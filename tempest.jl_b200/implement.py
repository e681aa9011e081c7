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

from . import groups, lib

ELTYPES = {"Float32": (lib.F32, 4), "BFloat16": (lib.BF16, 2)}
_BYTES = {"Float32": 4, "BFloat16": 2, "Int32": 4}   # of every element type an array of a binding may have (masks: Int32)


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
        return base + self.offset * _BYTES[self.eltype]


@dataclass
class Binding:
    """A group matched to one template (library.jl:61-72)."""
    template: str
    extents: Dict[str, int]
    arrays: Dict[str, Strided]


@dataclass
class Work:
    """The cost statement of a claim (src/Compiler/Implement/Implement.jl:30-82).  The reference states one `Work`
    per launch; the mirror states a claim's launches together (`launches`) with the fields the reference prices:
    what is moved, what is read again, what passes between the claim's launches, the products' flops and factor
    type, the flops of folds recomputed inside them, the blocks and whether they split sums, the steps a block
    takes one after another."""
    bytes: int
    flops: float = 0.0
    blocks: int = 0
    launches: int = 1
    applied: int = 0     # function applications per element the launch pays for beyond its bytes
    reread: int = 0      # bytes read again, beyond the first time (operand tiles fetched by several blocks)
    passed: int = 0      # bytes passed between the claim's launches through a workspace (partial sums, dq in Float32)
    recomputed: float = 0.0   # flops of folds recomputed inside the products (attention's scores)
    factor: str = "Float32"   # the products' factor type
    split: bool = False  # the blocks split sums among them
    steps: int = 0       # steps a block takes one after another, each waiting for what it loads


@dataclass
class Target:
    """What of `CUDATarget` the kernels look at (src/Compiler/runtime/target.jl:71-75)."""
    device: int = 0
    online: bool = True
    deterministic: bool = False   # the reference's default (src/Compiler/runtime/target.jl:31)


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


# Products: y = act.(w * x .+ b) with a Julia w::(m, k) (memory [k][m]) and x::(k, n) (memory [n][k]).
LINEAR_SPELLINGS = {
    "linear": ("(w, x) -> w * x", lib.EPI_NONE),
    "linear_bias": ("(w, x, b) -> w * x .+ b", lib.EPI_BIAS),
    "linear_bias_gelu": ("(w, x, b) -> gelu.(w * x .+ b)", lib.EPI_BIAS_GELU),
    "linear_bias_tanh": ("(w, x, b) -> tanh.(w * x .+ b)", lib.EPI_BIAS_TANH),
}
LINEAR_TEMPLATES = tuple(
    Template(name, spelling, {"w": ("m", "k"), "x": ("k", "n"), **({"b": ("m",)} if "bias" in name else {})}, ("y",))
    for name, (spelling, _) in LINEAR_SPELLINGS.items())

# Attention as the reference spells it (test/fixtures/operations.jl:21-76, ext/cuDNNExt.jl:38-57):
# q (d, h, m, b), k and v (d, hk, n, b); with the log-sum-exp (1, h, m, b) beside the output or not.
ATTENTION_TEMPLATES = tuple(
    Template(f"attention{'_causal' if causal else ''}{'_lse' if stats else ''}",
             f"(q, k, v) -> Ops.attention_forward(q, k, v; causal = {str(causal).lower()}, scale)" +
             (".o" if not stats else ""),
             {"q": ("d", "h", "m", "b"), "k": ("d", "hk", "n", "b"), "v": ("d", "hk", "n", "b")},
             ("o", "lse") if stats else ("o",))
    for stats in (False, True) for causal in (False, True))
# With masks the device holds (test/cuda/attention.jl:217-275): `start` (m, b) Int32, the first key each query sees
# (0-based) under the causal mask -- packed documents; `lengths` (b,) Int32, keys at and beyond a sequence's length
# hidden -- decode over a cache.
_MASK_INPUTS = {"documents": {"start": ("m", "b")}, "lengths": {"lengths": ("b",)}}
ATTENTION_MASKED = tuple(
    Template(f"attention_{kind}{'_lse' if stats else ''}",
             f"(q, k, v, {list(extra)[0]}) -> attention with the mask read from the device" + (".o" if not stats else ""),
             {"q": ("d", "h", "m", "b"), "k": ("d", "hk", "n", "b"), "v": ("d", "hk", "n", "b"), **extra},
             ("o", "lse") if stats else ("o",))
    for kind, extra in (("causal_documents", _MASK_INPUTS["documents"]), ("lengths", _MASK_INPUTS["lengths"]))
    for stats in (False, True)) + tuple(
    Template(f"attention_{kind}_pullback", "(q, k, v, mask, o, lse, g) -> the tape's derivative by q, k and v",
             {"q": ("d", "h", "m", "b"), "k": ("d", "hk", "n", "b"), "v": ("d", "hk", "n", "b"), **extra,
              "o": ("d", "h", "m", "b"), "lse": ("one", "h", "m", "b"), "g": ("d", "h", "m", "b")},
             ("dq", "dk", "dv"))
    for kind, extra in (("causal_documents", _MASK_INPUTS["documents"]), ("lengths", _MASK_INPUTS["lengths"])))
ATTENTION_PULLBACKS = tuple(
    Template(f"attention{'_causal' if causal else ''}_pullback",
             "(q, k, v, o, lse, g) -> the tape's derivative of attention by q, k and v",
             {"q": ("d", "h", "m", "b"), "k": ("d", "hk", "n", "b"), "v": ("d", "hk", "n", "b"),
              "o": ("d", "h", "m", "b"), "lse": ("one", "h", "m", "b"), "g": ("d", "h", "m", "b")},
             ("dq", "dk", "dv"))
    for causal in (False, True))


# Scans as Julia spells them (test/cuda/scans.jl:12-22): along the first axis (dims = 1, the contiguous one) or the
# second (dims = 2) of a (n, rows) matrix; the recurrence takes its pairs from two arrays.
SCAN_SPELLINGS = {
    "cumsum": ("x -> cumsum(x; dims)", lib.SCAN_SUM), "cumprod": ("x -> cumprod(x; dims)", lib.SCAN_PROD),
    "cummax": ("x -> accumulate(max, x; dims)", lib.SCAN_MAX), "cummin": ("x -> accumulate(min, x; dims)", lib.SCAN_MIN),
    "recurrence": ("(a, b) -> accumulate(RECURRENCE, tuple.(a, b); dims)", lib.SCAN_AFFINE),
    "running_variance": ("x -> accumulate(VARIANCE, x; dims)", lib.SCAN_VARIANCE),
}
SCAN_TEMPLATES = tuple(
    Template(f"{name}_dims{dims}{'_reverse' if rev else ''}", spelling.replace("dims", f"dims = {dims}") +
             (" from the last element back" if rev else ""),
             {"x": ("n", "rows"), **({"x2": ("n", "rows")} if name == "recurrence" else {})}, ("y",))
    for name, (spelling, _) in SCAN_SPELLINGS.items() for dims in (1, 2) for rev in (False, True))


def _scan_parts(template):
    """(op, across, reverse) of a scan template's name, or None."""
    base, _, rest = template.partition("_dims")
    if base not in SCAN_SPELLINGS or not rest or rest[0] not in "12":
        return None
    return SCAN_SPELLINGS[base][1], rest[0] == "2", rest.endswith("_reverse")


class ScanLaunch:
    """One scan on fixed operands (tb200_scan)."""

    def __init__(self, binding: "Binding", resources=None):
        self.binding = binding
        self.op, self.across, self.reverse = _scan_parts(binding.template)
        # a scan across many rows of few columns is cut into runs of rows when it is given scratch for their totals
        self.workspace, self.workspace_bytes = None, 0
        if self.across:
            e, a = binding.extents, binding.arrays
            need = lib.scan_workspace_bytes(lib.scan_desc(e["n"], e["rows"], self.op, across=True, reverse=self.reverse,
                                                          dtype=ELTYPES[a["x"].eltype][0]))
            if need:
                resources = resources if resources is not None else Resources()
                self.workspace, self.workspace_bytes = resources.workspace(need), need

    def repoints(self) -> bool:
        return True

    def repoint(self, value: int, buffer) -> "ScanLaunch":
        for s in self.binding.arrays.values():
            if s.value == value:
                s.buffer = buffer
        return self

    def __call__(self):
        a, e = self.binding.arrays, self.binding.extents
        ld = lambda s: s.strides[1] if len(s.strides) > 1 and s.size[1] > 1 else s.size[0]   # noqa: E731
        lib.scan(a["x"].pointer(), a["y"].pointer(), e["n"], e["rows"], self.op,
                 x2=a["x2"].pointer() if "x2" in a else 0, across=self.across, reverse=self.reverse,
                 dtype=ELTYPES[a["x"].eltype][0], ld_x=ld(a["x"]), ld_x2=ld(a["x2"]) if "x2" in a else None,
                 ld_y=ld(a["y"]), workspace=self.workspace.data_ptr() if self.workspace is not None else 0,
                 workspace_bytes=self.workspace_bytes, stream=current_stream())


def dense_matrix(buffer, eltype, rows, cols, value=0, offset=0):
    """A Julia (rows, cols) matrix, dense column-major."""
    return Strided(eltype, offset, (rows, cols), (1, rows), buffer, value)


def dense_heads(buffer, eltype, d, heads, positions, batch, value=0):
    """A Julia (d, heads, positions, batch) array, dense."""
    return Strided(eltype, 0, (d, heads, positions, batch), (1, d, d * heads, d * heads * positions), buffer, value)


def _dense(s: "Strided") -> bool:
    expect = 1
    for size, stride in zip(s.size, s.strides):
        if size > 1 and stride != expect:
            return False
        expect *= size
    return True


class LinearLaunch:
    """One product with its fused epilogue on fixed operands (tb200_gemm).  `pick`: the variant a tuning run chose
    (tile_n, split_k, direct_epilogue of the descriptor); none: the library's own choice."""

    def __init__(self, binding: Binding, pick=None):
        self.binding = binding
        self.epilogue = LINEAR_SPELLINGS[binding.template][1]
        self.pick = dict(pick or {})

    def _options(self):
        a, e = self.binding.arrays, self.binding.extents
        w, x, y = a["w"], a["x"], a["y"]
        return dict(lda=x.strides[1], ldb=w.strides[1], ldc=y.strides[1], a_layout=lib.K_MAJOR, b_layout=lib.MN_MAJOR,
                    in_dtype=ELTYPES[w.eltype][0], epilogue=self.epilogue)

    def tune(self):
        """Times the compiled-in variants on the launch's own operands (y is overwritten with the product's result)
        and keeps the fastest; returns the pick."""
        a, e = self.binding.arrays, self.binding.extents
        d = lib.gemm_desc(e["n"], e["m"], e["k"], **self._options())
        lib.gemm_tune_desc(d, a["x"].pointer(), a["w"].pointer(), a["y"].pointer(),
                           bias=a["b"].pointer() if "b" in a else 0, stream=current_stream())
        # a split needs scratch the launch does not bring: the pick keeps the unsplit form
        self.pick = {"tile_n": d.tile_n, "direct_epilogue": d.direct_epilogue}
        return dict(self.pick)

    def repoints(self) -> bool:
        return True

    def repoint(self, value: int, buffer) -> "LinearLaunch":
        for s in self.binding.arrays.values():
            if s.value == value:
                s.buffer = buffer
        return self

    @staticmethod
    def check():
        """Synchronises and raises if a tensor-core kernel gave up a bounded wait since the last poll
        (the launch itself only enqueues and cannot know): call it where the results are about to be read."""
        lib.check_device()

    def __call__(self):
        a, e = self.binding.arrays, self.binding.extents
        w, x, y = a["w"], a["x"], a["y"]
        # memory: x [n][k] is the K-major A, w [k][m] the MN-major B, y [n][m] the result
        lib.gemm(x.pointer(), w.pointer(), y.pointer(), e["n"], e["m"], e["k"], **self._options(), **self.pick,
                 bias=a["b"].pointer() if "b" in a else 0, stream=current_stream())


class ProductsLaunch:
    """Plain products alike as one launch, by arrays of their operands' addresses on the device (tb200_gemm_pointers):
    the mirror of the reference's `Products` (ext/cuBLASExt.jl:273-330), which is built from several bindings of one
    shape and rewrites its address arrays in `repoint!`.  The arrays are written on the current stream, after the
    launches before that read them."""

    def __init__(self, bindings):
        import torch
        self.bindings = list(bindings)
        first = self.bindings[0]
        e, a = first.extents, first.arrays
        for b in self.bindings:
            if b.template != "linear" or dict(b.extents) != dict(e):
                raise ValueError("products alike: every binding is a plain `linear` of the same extents")
            for name in ("w", "x", "y"):
                if b.arrays[name].eltype != a[name].eltype or b.arrays[name].strides != a[name].strides:
                    raise ValueError("products alike: the operands' element types and strides agree")
        w, x, y = a["w"], a["x"], a["y"]
        self.desc = lib.gemm_desc(e["n"], e["m"], e["k"], lda=x.strides[1], ldb=w.strides[1], ldc=y.strides[1],
                                  a_layout=lib.K_MAJOR, b_layout=lib.MN_MAJOR, in_dtype=ELTYPES[w.eltype][0],
                                  out_dtype=ELTYPES[y.eltype][0])
        self.count = len(self.bindings)
        self._torch = torch
        self.addresses = {name: torch.empty(self.count, dtype=torch.int64, device="cuda") for name in ("x", "w", "y")}
        for name in self.addresses:
            self._write(name)

    def _write(self, name):
        host = self._torch.tensor([b.arrays[name].pointer() for b in self.bindings], dtype=self._torch.int64).pin_memory()
        self.addresses[name].copy_(host, non_blocking=True)
        self._keep = host   # until the copy has run

    def repoints(self) -> bool:
        return True

    def repoint(self, value: int, buffer) -> "ProductsLaunch":
        for name in self.addresses:
            moved = False
            for b in self.bindings:
                if b.arrays[name].value == value:
                    b.arrays[name].buffer = buffer
                    moved = True
            if moved:
                self._write(name)
        return self

    def __call__(self):
        lib.gemm_pointers(self.desc, self.addresses["x"].data_ptr(), self.addresses["w"].data_ptr(),
                          self.addresses["y"].data_ptr(), self.count, stream=current_stream())


class AttentionLaunch:
    """Attention forward or its pullback on fixed operands."""

    def __init__(self, binding: Binding, workspace=None, workspace_bytes=0):
        self.binding = binding
        e = binding.extents
        self.desc = lib.attn_desc(e["b"], e["h"], e["m"], e["n"], e["d"], "causal" in binding.template,
                                  kv_heads=e["hk"])
        self.workspace, self.workspace_bytes = workspace, workspace_bytes

    def repoints(self) -> bool:
        return True

    def repoint(self, value: int, buffer) -> "AttentionLaunch":
        for s in self.binding.arrays.values():
            if s.value == value:
                s.buffer = buffer
        return self

    @staticmethod
    def check():
        """Synchronises and raises if a tensor-core kernel gave up a bounded wait since the last poll
        (the launch itself only enqueues and cannot know): call it where the results are about to be read."""
        lib.check_device()

    def __call__(self):
        a = self.binding.arrays
        stream = current_stream()
        if "start" in a or "lengths" in a:
            mask = lib.attn_mask(doc_start=a["start"].pointer() if "start" in a else 0,
                                 kv_len=a["lengths"].pointer() if "lengths" in a else 0)
            if not self.binding.template.endswith("_pullback"):
                lib.attention_fwd_masked(self.desc, mask, a["q"].pointer(), a["k"].pointer(), a["v"].pointer(),
                                         a["o"].pointer(), a["lse"].pointer() if "lse" in a else 0, stream)
                return
            operands = (a["q"].pointer(), a["k"].pointer(), a["v"].pointer(), a["o"].pointer(), a["lse"].pointer(),
                        a["g"].pointer(), a["dq"].pointer(), a["dk"].pointer(), a["dv"].pointer())
            if self.workspace is not None:   # 128 features: the tensor-core kernels, which want scratch
                lib.attention_bwd_masked_ws(self.desc, mask, *operands, self.workspace.data_ptr(), self.workspace_bytes,
                                            stream)
            else:
                lib.attention_bwd_masked(self.desc, mask, *operands, stream)
            return
        if self.binding.template.endswith("_pullback"):
            lib.attention_bwd(self.desc, a["q"].pointer(), a["k"].pointer(), a["v"].pointer(), a["o"].pointer(),
                              a["lse"].pointer(), a["g"].pointer(), a["dq"].pointer(), a["dk"].pointer(),
                              a["dv"].pointer(), self.workspace.data_ptr(), self.workspace_bytes, stream)
        else:
            lib.attention_fwd(self.desc, a["q"].pointer(), a["k"].pointer(), a["v"].pointer(), a["o"].pointer(),
                              a["lse"].pointer() if "lse" in a else 0, stream)


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


def row_eltype(binding: "Binding") -> str:
    """Element type of a row binding's rows: that of its arrays other than the statistics (`lse`,
    `mean`, `rstd`), which may be Float32 beside BFloat16 rows and may come first in the dictionary."""
    for name, s in binding.arrays.items():
        if name not in ("lse", "mean", "rstd"):
            return s.eltype
    raise ValueError(f"{binding.template}: a binding with statistics only has no rows")


class RowLaunch:
    """One fused row kernel on fixed operands.  Calling it enqueues the kernel;
    `repoint` replaces the buffer of one value (ext/cuDNNExt.jl:207-218)."""

    def __init__(self, binding: Binding, eps: float, workspace, workspace_bytes: int):
        self.binding = binding
        self.eps = eps
        self.workspace = workspace
        self.workspace_bytes = workspace_bytes
        self.dtype = ELTYPES[row_eltype(binding)][0]
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


_ATTENTION_KERNELS = {
    lib.ATTN_FORM_CUDA_CORES: "CUDA-core kernels",
    lib.ATTN_FORM_TILE: "tensor cores, one query tile a block",
    lib.ATTN_FORM_TWO_TILES: "tensor cores, two query tiles a block",
    lib.ATTN_FORM_ONE_KERNEL: "tensor cores, one kernel (dq added in L2)",
    lib.ATTN_FORM_TWO_KERNELS: "tensor cores, two kernels (deterministic)",
}


def _attention_kernels(desc, masked, pullback) -> str:
    """The kernels a built attention launch runs, for its description (tb200_attention_form)."""
    return _ATTENTION_KERNELS[lib.attention_form(desc, masked=masked, pullback=pullback)]


class B200Kernels:
    """The library (`<: Library`): which templates it computes, whether it takes
    a binding, what a launch costs, and the launch itself."""

    def __init__(self, eps: float = 1.0e-5, record=None):
        """`record`: a `tuning.TuningRecord`; with one, `build` measures a product's variants (and an attention
        pullback's two forms) the first time it meets a shape, keeps the pick in the record's file, and reads it back
        in later sessions instead of measuring again."""
        self.eps = eps
        self.record = record

    def templates(self, target: Target):
        # the row kernels and attention fold each statistic in one pass, which a target that
        # forbids the online rewrites does not permit (ext/cuDNNExt.jl:60-62); products always apply
        online = ROW_TEMPLATES + ATTENTION_TEMPLATES + ATTENTION_PULLBACKS + ATTENTION_MASKED if target.online else ()
        return LINEAR_TEMPLATES + SCAN_TEMPLATES + online

    def resources(self, target: Target) -> Resources:
        return Resources()

    def package_of(self) -> str:
        """The package whose kernels the launches run (src/Compiler/Implement/Implement.jl:91)."""
        return PACKAGE

    @staticmethod
    def loaded() -> bool:
        """Whether the library can be made (src/Compiler/Implement/Implement.jl:99)."""
        return library_loaded()

    def supports(self, target: Target, b: Binding) -> bool:
        if b.template in LINEAR_SPELLINGS:
            types = {s.eltype for s in b.arrays.values()}
            if len(types) != 1 or types.pop() not in ELTYPES:
                return False
            # the contracted axis of x and the output axis of w and y must be contiguous
            return all(s.strides[0] == 1 or s.size[0] == 1 for s in b.arrays.values())
        if _scan_parts(b.template) is not None:
            types = {s.eltype for s in b.arrays.values()}
            if len(types) != 1 or types.pop() not in ELTYPES or ("x2" in b.arrays) != b.template.startswith("recurrence"):
                return False
            return all(s.strides[0] == 1 or s.size[0] == 1 for s in b.arrays.values())   # rows contiguous
        if b.template.startswith("attention"):
            e = b.extents
            if not 0 < e.get("d", 0) <= 256 or e.get("h", 0) % max(e.get("hk", 1), 1) != 0:
                return False   # as cuDNNAttention declines what its engines do not take (ext/cuDNNExt.jl:90-109)
            if "causal" in b.template and e.get("m") != e.get("n"):
                return False
            masked = "documents" in b.template or "lengths" in b.template
            if masked and ("start" in b.arrays) != ("documents" in b.template):
                return False
            if masked and ("lengths" in b.arrays) != ("_lengths" in b.template):
                return False
            for name, s in b.arrays.items():
                want = "Float32" if name == "lse" else "Int32" if name in ("start", "lengths") else "BFloat16"
                if s.eltype != want or not _dense(s):
                    return False
            return True
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
        return True

    def estimate(self, target: Target, b: Binding):
        if _scan_parts(b.template) is not None:
            e = b.extents
            size = ELTYPES[b.arrays["x"].eltype][1]
            across = _scan_parts(b.template)[1]
            moved = len(b.arrays) * e["n"] * e["rows"] * size
            if across and e["rows"] >= 128 and (e["n"] + 255) // 256 < 8 * 148:
                # in slabs (scratch from the executable's resources): the inputs are read twice, the slabs' totals pass
                # between the two launches
                inputs = (len(b.arrays) - 1) * e["n"] * e["rows"] * size
                return [Work(bytes=moved, blocks=(e["n"] + 255) // 256, launches=2, reread=inputs, split=True)]
            return [Work(bytes=moved, blocks=(e["n"] + 255) // 256 if across else e["rows"])]
        if b.template in LINEAR_SPELLINGS:
            e = b.extents
            size = ELTYPES[b.arrays["w"].eltype][1]
            moved = size * (e["m"] * e["k"] + e["k"] * e["n"] + e["m"] * e["n"])
            # the kernel's M is Tempest's n (the batch), its N Tempest's m; every tile row fetches w again and every
            # tile column x, from L2 once the first has brought them in
            form = lib.gemm_tile_form(lib.gemm_desc(e["n"], e["m"], e["k"]))
            tile_m, tile_n = (256, 256) if form == 512 else (128, max(form, 128))
            tiles_m, tiles_n = -(-e["n"] // tile_m), -(-e["m"] // tile_n)
            reread = size * (e["m"] * e["k"] * (tiles_m - 1) + e["k"] * e["n"] * (tiles_n - 1))
            return [Work(bytes=moved, flops=2.0 * e["m"] * e["n"] * e["k"], factor=b.arrays["w"].eltype,
                         blocks=tiles_m * tiles_n, reread=reread, steps=-(-e["k"] // 64))]
        if b.template.startswith("attention"):
            e = b.extents
            flops = 4.0 * e["d"] * e["h"] * e["m"] * e["b"] * e["n"]     # both products (ext/cuDNNExt.jl:141-145)
            flops = flops / 2 if "causal" in b.template else flops
            moved = 2 * e["d"] * e["b"] * (2 * e["h"] * e["m"] + 2 * e["hk"] * e["n"])
            q_tiles, k_tiles = -(-e["m"] // 128), -(-e["n"] // 128)
            items = q_tiles * e["h"] * e["b"]
            keys = 2 * e["d"] * e["b"] * 2 * e["hk"] * e["n"]            # K and V: fetched again by every query tile
            seen = 0.5 if "causal" in b.template else 1.0
            if b.template.endswith("_pullback"):
                # the scores are formed again (one of the five products), dq passes through Float32 scratch in the
                # one-kernel form, statistics + the rounding kernel are launches of their own
                return [Work(bytes=2 * moved, flops=2.5 * flops, launches=3, recomputed=0.5 * flops, factor="BFloat16",
                             blocks=k_tiles * e["hk"] * e["b"], passed=2 * 4 * e["d"] * e["h"] * e["m"] * e["b"],
                             reread=int(seen * (k_tiles - 1) * 2 * e["d"] * e["b"] * 2 * e["h"] * e["m"]),
                             steps=max(1, int(seen * q_tiles)))]
            return [Work(bytes=moved, flops=flops, recomputed=0.5 * flops, factor="BFloat16", blocks=items,
                         reread=int(seen * (q_tiles * e["h"] // e["hk"] - 1) * keys), steps=max(1, int(seen * k_tiles)))]
        size = ELTYPES[row_eltype(b)][1]
        n, rows = b.extents["n"], b.extents["rows"]
        op = _ROWOP[b.template]
        launches = 2 if (op == lib.LAYERNORM_BWD or n > 16384) else 1
        # what passes between the launches: the row blocks' partial weight gradients, or a long row's chunk states
        passed = lib.rowop_workspace_bytes(op, n, rows, ELTYPES[row_eltype(b)][0]) if launches > 1 else 0
        return [Work(bytes=_STREAMS[op] * n * rows * size, blocks=rows, launches=launches, passed=passed,
                     split=n > 16384)]

    def build_alike(self, target: Target, bindings, resources: Optional[Resources] = None):
        """Several plain products of one shape as one launch (the reference's `build(::cuBLASProducts, target,
        bs::Vector{Binding}, scratch)`, ext/cuBLASExt.jl:273-284)."""
        bindings = list(bindings)
        for b in bindings:
            if b.template != "linear" or not self.supports(target, b):
                raise ValueError("B200Kernels.build_alike takes plain `linear` bindings it supports")
            for s in b.arrays.values():
                if s.buffer is None:
                    raise ValueError("build needs every array's buffer")
        e = bindings[0].extents
        return (ProductsLaunch(bindings),
                f"B200 {len(bindings)} products alike, {e['m']} x {e['n']} over {e['k']}, {bindings[0].arrays['w'].eltype}")

    def build(self, target: Target, b: Binding, resources: Optional[Resources] = None):
        if not self.supports(target, b):
            raise ValueError(f"B200Kernels does not compute this binding of {b.template}")
        for s in b.arrays.values():
            if s.buffer is None:
                raise ValueError("build needs every array's buffer")
        if b.template in LINEAR_SPELLINGS:
            e = b.extents
            launch, how = LinearLaunch(b), ""
            if self.record is not None:
                key = self.record.key(b.template, e["m"], e["n"], e["k"], b.arrays["w"].eltype)
                pick = self.record.lookup("product", key)
                if pick is None:
                    pick = self.record.keep("product", key, launch.tune())
                    how = ", variants measured"
                else:
                    how = ", variant from the tuning record"
                launch.pick = pick
                how += f" (tile_n {pick.get('tile_n', 0)})"
            return launch, f"B200 {b.template}, {e['m']} x {e['n']} over {e['k']}, {b.arrays['w'].eltype}{how}"
        if _scan_parts(b.template) is not None:
            e = b.extents
            return ScanLaunch(b, resources), f"B200 {b.template}, {e['rows']} rows of {e['n']} {b.arrays['x'].eltype}"
        if b.template.startswith("attention"):
            launch = AttentionLaunch(b)
            if "documents" in b.template or "lengths" in b.template:
                e = b.extents
                if b.template.endswith("_pullback") and e["d"] == 128:
                    # the tensor-core pullback: repeatable bits when the target asks, else the one-kernel form
                    launch.desc.deterministic = int(bool(target.deterministic))
                    need = lib.attention_bwd_masked_workspace_bytes(launch.desc)
                    resources = resources if resources is not None else Resources()
                    launch.workspace, launch.workspace_bytes = resources.workspace(need), need
                what = "the starts of packed documents" if "documents" in b.template else "lengths"
                kernels = _attention_kernels(launch.desc, masked=True, pullback=b.template.endswith("_pullback"))
                return launch, (f"B200 {b.template}, {what} read on the device, {e['h']} heads over {e['hk']} of "
                                f"{e['d']} features, {e['m']} queries by {e['n']} keys, batch {e['b']}, {kernels}")
            if b.template.endswith("_pullback"):
                # a target that wants repeatable bits gets the two-kernel form; any other gets whichever of the two
                # forms measures faster on these operands (the measured stage of the cover's search over variants)
                launch.desc.deterministic = 0
                need = lib.attention_bwd_workspace_bytes(launch.desc)
                resources = resources if resources is not None else Resources()
                launch.workspace, launch.workspace_bytes = resources.workspace(need), need
                e = b.extents
                key = None if self.record is None else self.record.key(
                    b.template, e["d"], e["h"], e["hk"], e["m"], e["n"], e["b"], int(bool(launch.desc.causal)))
                kept = self.record.lookup("attention_pullback", key) if key else None
                if target.deterministic:
                    launch.desc.deterministic = 1
                elif kept is not None:
                    launch.desc.deterministic = kept["deterministic"]
                else:
                    a = b.arrays
                    launch.desc.deterministic = lib.attention_bwd_tune(
                        launch.desc, a["q"].pointer(), a["k"].pointer(), a["v"].pointer(), a["o"].pointer(),
                        a["lse"].pointer(), a["g"].pointer(), a["dq"].pointer(), a["dk"].pointer(), a["dv"].pointer(),
                        launch.workspace.data_ptr(), need, current_stream())
                    if key:
                        self.record.keep("attention_pullback", key, {"deterministic": launch.desc.deterministic})
            form = ", " + _attention_kernels(launch.desc, masked=False, pullback=b.template.endswith("_pullback"))
            e = b.extents
            return launch, (f"B200 {b.template}, {e['h']} heads over {e['hk']} of {e['d']} features, "
                            f"{e['m']} queries by {e['n']} keys, batch {e['b']}{form}")
        eltype = row_eltype(b)
        dtype = ELTYPES[eltype][0]
        n, rows = b.extents["n"], b.extents["rows"]
        need = lib.rowop_workspace_bytes(_ROWOP[b.template], n, rows, dtype)
        resources = resources if resources is not None else Resources()
        ws = resources.workspace(need) if need else None
        launch = RowLaunch(b, self.eps, ws, need)
        schedule = "split" if n > 16384 else "resident"
        return launch, f"B200 {b.template}, {rows} rows of {n} {eltype}, {schedule}"


# ---------------------------------------------------------------- generic groups ----
#
# The second door of the reference's plugin API (src/Compiler/Implement/Implement.jl:108-175): an
# `Implementation` is asked for `claims` on a `GroupView`, states each claim's cost with `estimate`, and turns
# the chosen one into a launch with `build_claim(impl, claim, target, g, buffers, resources)`, where
# `buffers[v]` is the device vector of value `v`.  `B200Generator` is that protocol over `groups.Group`.

@dataclass(frozen=True)
class RowClaim:
    """What the generator offers for a group: one launch, rows spread over groups of `threads` threads;
    `compiled` = the group's own NVRTC-compiled kernel instead of the term interpreter."""
    threads: int
    phases: int
    compiled: bool = False


class GroupLaunch:
    """Callable with no arguments; enqueues on the current stream; `repoint` swaps one buffer."""

    def __init__(self, group, inputs, outputs, compiled=False):
        self.group, self.desc, self.compiled = group, group.desc(), compiled
        self.inputs, self.outputs = list(inputs), list(outputs)   # (value id, buffer)

    def repoints(self) -> bool:
        return True

    def repoint(self, value: int, buffer) -> "GroupLaunch":
        self.inputs = [(v, buffer if v == value else b) for v, b in self.inputs]
        self.outputs = [(v, buffer if v == value else b) for v, b in self.outputs]
        return self

    def __call__(self):
        address = lambda b: b.data_ptr() if hasattr(b, "data_ptr") else int(b)  # noqa: E731
        run = lib.rowreduce_compiled if self.compiled else lib.rowreduce_generic
        run(self.desc, [address(b) for _, b in self.inputs], [address(b) for _, b in self.outputs], _torch_stream())


@dataclass(frozen=True)
class AttentionClaim:
    """What the generator offers for the attention group (recomputed scores, mask, log-sum-exp, weighted value
    rows): the attention kernels, reached through the descriptor's own structure."""
    causal: bool


class RoutedAttentionLaunch(GroupLaunch):
    """The launch of a group `lib.group_route` recognised as attention; `outer` = (heads, kv_heads, batch), the
    domain's outer axes, the buffers the reference's whole (features, heads, positions, batch) arrays."""

    def __init__(self, group, inputs, outputs, outer):
        super().__init__(group, inputs, outputs, compiled=True)
        self.outer = outer

    def __call__(self):
        address = lambda b: b.data_ptr() if hasattr(b, "data_ptr") else int(b)  # noqa: E731
        lib.group_attention(self.desc, *self.outer, [address(b) for _, b in self.inputs],
                            [address(b) for _, b in self.outputs], _torch_stream())


@dataclass(frozen=True)
class ColumnClaim:
    """What the generator offers for a group whose folds run over the rows: partial folds per row slab
    (one thread per column) and an ordered merge, two launches, compiled by NVRTC."""
    launches: int = 2


class ColumnLaunch(GroupLaunch):
    """The launch of a group that folds the other axis; holds the scratch for the slabs' partial folds."""

    def __init__(self, group, inputs, outputs, workspace, workspace_bytes):
        super().__init__(group, inputs, outputs, compiled=True)
        self.workspace, self.workspace_bytes = workspace, workspace_bytes

    def __call__(self):
        address = lambda b: b.data_ptr() if hasattr(b, "data_ptr") else int(b)  # noqa: E731
        lib.colreduce_compiled(self.desc, [address(b) for _, b in self.inputs], [address(b) for _, b in self.outputs],
                               address(self.workspace), self.workspace_bytes, _torch_stream())


@dataclass(frozen=True)
class RecurrenceClaim:
    """What the generator offers for a `:recurrence` group whose step is a map over the parallel axis (the state is
    carried per position, no reduction inside the step): one launch, one thread per position walking the steps
    with the state in registers, compiled by NVRTC."""
    states: int


class RecurrenceLaunch(GroupLaunch):
    """The launch of a recurrence whose step is a map (tb200_recurrence_compiled)."""

    def __init__(self, group, inputs, outputs):
        super().__init__(group, inputs, outputs, compiled=True)

    def __call__(self):
        address = lambda b: b.data_ptr() if hasattr(b, "data_ptr") else int(b)  # noqa: E731
        lib.recurrence_compiled(self.desc, [address(b) for _, b in self.inputs], [address(b) for _, b in self.outputs],
                                _torch_stream())


PACKAGE = "tempest_b200"
_LOWERED = frozenset(name for name, arity in groups.ARITY.items() if arity > 0)
_LOWERED_CODES = frozenset(groups.OPS.values())


def library_loaded() -> bool:
    """Whether the shared library can be loaded in this process."""
    try:
        lib.load()
    except (RuntimeError, OSError):
        return False
    return True


class B200Generator:
    """`<: Implementation` for row groups: claims every group whose descriptor the library accepts."""

    def claims(self, target: Target, group):
        try:
            desc = group.desc()
        except ValueError:
            return ()                                  # too large for one descriptor: decline
        if getattr(group, "kind", "") == "recurrence":  # a step that is a map: the compiled form or nothing
            try:
                lib.recurrence_compile(desc)
            except lib.TB200Error:
                return ()
            return (RecurrenceClaim(desc.n_states),)
        if getattr(group, "across", False):            # folds over the other axis: the compiled form or nothing
            try:
                lib.colreduce_compile(desc)
            except lib.TB200Error:
                return ()
            return (ColumnClaim(),)
        route = lib.group_route(desc)
        if route in (lib.ROUTE_ATTENTION, lib.ROUTE_ATTENTION_CAUSAL):
            return (AttentionClaim(route == lib.ROUTE_ATTENTION_CAUSAL),)
        if lib.rowreduce_generic_check(desc) != 0:
            return ()
        threads = 8
        while threads < 256 and threads * 4 < group.n:
            threads *= 2
        phases = 1 + max((fold[2] for fold in group.folds), default=-1) + 1
        claims = [RowClaim(threads, phases)]
        if lib.rowreduce_compile(desc) == 0:           # NVRTC at hand and the generated source compiles
            claims.insert(0, RowClaim(threads, phases, compiled=True))
        return tuple(claims)

    def variants(self, target: Target, group, claim):
        return ()                                      # one schedule per claim: nothing further to search

    # ---- the rest of the protocol (src/Compiler/Implement/Implement.jl:85-214): what the cover asks before it
    # offers a group, each with the reference default's meaning
    def package_of(self) -> str:
        """The package whose kernels the launches run: the line of the rates file they are priced on (:91)."""
        return PACKAGE

    @staticmethod
    def loaded() -> bool:
        """Whether the implementation can be made (:99): whether the shared library is there to load."""
        return library_loaded()

    def resources(self, target: Target) -> Resources:
        """One executable's scratch, shared by its launches (:141): the column groups' partial sums."""
        return Resources()

    def candidates(self, target: Target, plan):
        """No regrouping of the plan's values is proposed (:186): the generator takes the groups as cut."""
        return []

    def record_name(self, claim) -> str:
        """A claim's name in the tuning record (:189); claims hold schedules, never value numbers."""
        return f"{type(self).__name__} {claim}"

    def recomputes_folds(self, target: Target) -> bool:
        """A fold formed where it is read (`recomputed` terms: attention's scores) is computed in the reading
        kernel, by the term interpreter and by the attention kernels a group's terms lead to (:192)."""
        return True

    def lowers(self, target: Target, term, group=None) -> bool:
        """Whether a group applying `term` can be realized (:214): `term` is a scalar function's name, or the
        number of a term of `group`.  What has no code in `groups.OPS` is declared here, before any claim."""
        if isinstance(term, int):
            code = group.terms[term][0]
            return code in _LOWERED_CODES
        return term in _LOWERED

    def estimate(self, claim: RowClaim, target: Target, group):
        """One launch moving the group's bytes once; the interpreter also pays for every term of every element
        (`applied` in the reference's Work, src/Compiler/Implement/Implement.jl:61-82)."""
        if isinstance(claim, AttentionClaim):
            d = group.inputs[0][2]
            flops = 4.0 * d * group.n * group.rows * (0.5 if claim.causal else 1.0)
            return [Work(bytes=2 * d * (2 * group.rows + 2 * group.n), flops=flops)]
        if isinstance(claim, ColumnClaim):
            return [Work(bytes=group.bytes(), blocks=(group.n + 255) // 256, launches=claim.launches, applied=0)]
        if isinstance(claim, RecurrenceClaim):
            return [Work(bytes=group.bytes(), blocks=(group.n + 255) // 256, launches=1, applied=0)]
        applied = 0 if claim.compiled else len(group.terms) * claim.phases
        return [Work(bytes=group.bytes(), blocks=group.rows, launches=1, applied=applied)]

    def in_place(self, claim: RowClaim) -> bool:
        """Every element an output needs is read before that output's sweep starts only for folds; the output
        sweep re-reads its inputs, so an output may alias an input only when nothing else reads that input --
        the generator does not promise it."""
        return False

    def build_claim(self, claim: RowClaim, target: Target, group, buffers, resources=None):
        """`buffers`: {"inputs": [...], "outputs": [...]} device buffers in the group's order, or a flat
        {value id: buffer} with inputs numbered first."""
        if not self.claims(target, group):
            raise ValueError("B200Generator does not compute this group")
        if "inputs" in buffers:
            ins, outs = list(enumerate(buffers["inputs"])), list(enumerate(buffers["outputs"], len(buffers["inputs"])))
        else:
            k = len(group.inputs)
            ins = [(v, buffers[v]) for v in range(k)]
            outs = [(v, buffers[v]) for v in range(k, k + len(group.outputs))]
        if len(ins) != len(group.inputs) or len(outs) != len(group.outputs):
            raise ValueError("build_claim needs one buffer per input and per output")
        if isinstance(claim, AttentionClaim):
            heads, kv_heads, batch = buffers.get("outer", (1, 1, 1))
            d = group.inputs[0][2]
            return (RoutedAttentionLaunch(group, ins, outs, (heads, kv_heads, batch)),
                    f"B200 attention{' (causal)' if claim.causal else ''} reached from the group's terms, {heads} heads "
                    f"over {kv_heads} of {d} features, {group.rows} queries by {group.n} keys, batch {batch}")
        if isinstance(claim, RecurrenceClaim):
            return (RecurrenceLaunch(group, ins, outs),
                    f"B200 compiled recurrence, {group.n} positions over {group.rows} steps"
                    f"{' in reverse' if group.reverse else ''}, {claim.states} states in registers, {len(group.terms)} terms")
        if isinstance(claim, ColumnClaim):
            need = lib.colreduce_workspace_bytes(group.desc())
            resources = resources if resources is not None else Resources()
            return (ColumnLaunch(group, ins, outs, resources.workspace(need), need),
                    f"B200 compiled columns, {group.n} columns over {group.rows} rows, {len(group.terms)} terms, "
                    f"{len(group.folds)} folds, slabs + ordered merge")
        if claim.compiled:
            status = lib.rowreduce_compile(group.desc())
            if status != 0:
                raise ValueError(f"the group's kernel did not compile: {lib.rowreduce_compile_log()[:400]}")
        kind = "compiled" if claim.compiled else "interpreted"
        return GroupLaunch(group, ins, outs, claim.compiled), (f"B200 {kind} rows, {group.rows} rows of {group.n}, {len(group.terms)} terms, "
                                                f"{len(group.folds)} folds in {claim.phases} sweeps")
