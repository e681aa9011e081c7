"""ctypes binding of libtempest_b200.so: one Python function per C-ABI entry point.

Arguments are raw device addresses (ints), extents and strides in elements,
and a CUDA stream handle; nothing here touches torch.  A missing or unbuilt
library raises: there is no CPU fallback.
"""
import ctypes
import os

F32, BF16, F16 = 0, 1, 2
SOFTMAX_FWD, SOFTMAX_BWD, LAYERNORM_FWD, LAYERNORM_BWD = 0, 1, 2, 3

K_MAJOR, MN_MAJOR = 0, 1
EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_TANH, EPI_MUL_GELU_GRAD, EPI_MUL_TANH_GRAD, EPI_AXPY = range(7)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtempest_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "tempest_b200.h")

_p, _i, _i64, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t



class GemmDesc(ctypes.Structure):
    """tb200_gemm_desc of include/tempest_b200.h."""
    _fields_ = [("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
                ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
                ("ld_aux", ctypes.c_int64), ("ld_aux_out", ctypes.c_int64),
                ("a_layout", ctypes.c_int), ("b_layout", ctypes.c_int),
                ("in_dtype", ctypes.c_int), ("out_dtype", ctypes.c_int),
                ("epilogue", ctypes.c_int), ("alpha", ctypes.c_float),
                ("tile_n", ctypes.c_int), ("force_simt", ctypes.c_int), ("direct_epilogue", ctypes.c_int),
                ("batch", ctypes.c_int64), ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64),
                ("stride_c", ctypes.c_int64), ("stride_bias", ctypes.c_int64), ("stride_aux", ctypes.c_int64),
                ("stride_aux_out", ctypes.c_int64), ("split_k", ctypes.c_int), ("workspace", ctypes.c_void_p),
                ("workspace_bytes", ctypes.c_size_t), ("debug", ctypes.c_int)]


class AttnDesc(ctypes.Structure):
    """tb200_attn_desc of include/tempest_b200.h."""
    _fields_ = [("batch", ctypes.c_int), ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int),
                ("queries", ctypes.c_int), ("keys", ctypes.c_int), ("head_dim", ctypes.c_int),
                ("causal", ctypes.c_int), ("scale", ctypes.c_float), ("dtype", ctypes.c_int),
                ("deterministic", ctypes.c_int), ("value_dim", ctypes.c_int)]


class AttnMask(ctypes.Structure):
    """tb200_attn_mask of include/tempest_b200.h."""
    _fields_ = [("doc_start", ctypes.c_void_p), ("kv_len", ctypes.c_void_p),
                ("q_stride", ctypes.c_int64 * 3), ("kv_stride", ctypes.c_int64 * 3)]


class DeltanetDesc(ctypes.Structure):
    """tb200_deltanet_desc of include/tempest_b200.h."""
    _fields_ = [("heads", ctypes.c_int), ("positions", ctypes.c_int), ("dk", ctypes.c_int), ("dv", ctypes.c_int),
                ("chunk", ctypes.c_int), ("dtype", ctypes.c_int)]


class ScanDesc(ctypes.Structure):
    """tb200_scan_desc of include/tempest_b200.h."""
    _fields_ = [("n", ctypes.c_int64), ("rows", ctypes.c_int64), ("ld_x", ctypes.c_int64), ("ld_x2", ctypes.c_int64),
                ("ld_y", ctypes.c_int64), ("batch", ctypes.c_int64), ("stride_x", ctypes.c_int64),
                ("stride_x2", ctypes.c_int64), ("stride_y", ctypes.c_int64), ("op", ctypes.c_int),
                ("across", ctypes.c_int), ("reverse", ctypes.c_int), ("dtype", ctypes.c_int),
                ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t)]


SCAN_SUM, SCAN_PROD, SCAN_MAX, SCAN_MIN, SCAN_AFFINE, SCAN_VARIANCE = range(6)


class DpDesc(ctypes.Structure):
    """tb200_dp_desc of include/tempest_b200.h."""
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("blocks", ctypes.c_int), ("dtype", ctypes.c_int),
                ("count", ctypes.c_int64), ("alpha", ctypes.c_float),
                ("grads", ctypes.c_void_p * 16), ("params", ctypes.c_void_p * 16), ("signals", ctypes.c_void_p * 16),
                ("grads_multicast", ctypes.c_void_p), ("params_multicast", ctypes.c_void_p), ("state", ctypes.c_void_p)]


GROUP_MAX_INPUTS, GROUP_MAX_TERMS, GROUP_MAX_FOLDS, GROUP_MAX_OUTPUTS = 8, 48, 8, 8


class GroupInput(ctypes.Structure):
    _fields_ = [("shape", ctypes.c_int), ("dtype", ctypes.c_int), ("ld", ctypes.c_int64)]


class GroupTerm(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int), ("a", ctypes.c_int), ("b", ctypes.c_int), ("c", ctypes.c_int),
                ("imm", ctypes.c_float)]


class GroupFold(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("term", ctypes.c_int), ("phase", ctypes.c_int), ("payload", ctypes.c_int)]


class GroupOutput(ctypes.Structure):
    _fields_ = [("source", ctypes.c_int), ("index", ctypes.c_int), ("dtype", ctypes.c_int), ("ld", ctypes.c_int64)]


class GroupDesc(ctypes.Structure):
    """tb200_group_desc of include/tempest_b200.h (`source` is the header's `from`)."""
    _fields_ = [("n", ctypes.c_int64), ("rows", ctypes.c_int64),
                ("n_inputs", ctypes.c_int), ("n_terms", ctypes.c_int), ("n_folds", ctypes.c_int),
                ("n_outputs", ctypes.c_int),
                ("inputs", GroupInput * GROUP_MAX_INPUTS), ("terms", GroupTerm * GROUP_MAX_TERMS),
                ("folds", GroupFold * GROUP_MAX_FOLDS), ("outputs", GroupOutput * GROUP_MAX_OUTPUTS)]


class StateDesc(ctypes.Structure):
    _fields_ = [("start", ctypes.c_int), ("next", ctypes.c_int)]


class RecurrenceDesc(ctypes.Structure):
    """tb200_recurrence_desc of include/tempest_b200.h."""
    _fields_ = [("body", GroupDesc), ("n_states", ctypes.c_int), ("states", StateDesc * 4), ("reverse", ctypes.c_int)]


# name -> (restype, argtypes): the declarations of include/tempest_b200.h
SIGNATURES = {
    "tb200_version": (_i, []),
    "tb200_strerror": (ctypes.c_char_p, [_i]),
    "tb200_last_cuda_error": (ctypes.c_char_p, []),
    "tb200_sm_count": (_i, []),
    "tb200_rowop_workspace_bytes": (_sz, [_i, _i64, _i64, _i]),
    "tb200_softmax_fwd": (_i, [_p, _p, _p, _i64, _i64, _i64, _i, _i, _p, _sz, _p]),
    "tb200_softmax_bwd": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _i, _i, _p, _sz, _p]),
    "tb200_layernorm_fwd": (_i, [_p, _p, _p, _p, _p, _p, _f, _i64, _i64, _i64, _i, _p, _sz, _p]),
    "tb200_layernorm_bwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _f, _i64, _i64, _i64, _i, _p, _sz, _p]),
    "tb200_layernorm_bwd_noalloc_max_row": (_sz, []),
    "tb200_layernorm_bwd_noalloc": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _f, _i64, _i64, _i64, _i, _p]),
    "tb200_gemm": (_i, [ctypes.POINTER(GemmDesc), _p, _p, _p, _p, _p, _p, _p]),
    "tb200_gemm_workspace_bytes": (_sz, [ctypes.POINTER(GemmDesc)]),
    "tb200_gemm_tile_form": (_i, [ctypes.POINTER(GemmDesc)]),
    "tb200_attention_form": (_i, [ctypes.POINTER(AttnDesc), _i, _i]),
    "tb200_gemm_plan_create": (_i, [ctypes.POINTER(GemmDesc), _p, _p, _p, _p, _p, _p, ctypes.POINTER(_p)]),
    "tb200_gemm_plan_launch": (_i, [_p, _p]),
    "tb200_gemm_plan_repoint": (_i, [_p, _i, _p]),
    "tb200_gemm_plan_destroy": (None, [_p]),
    "tb200_gemm_tune_desc": (_i, [ctypes.POINTER(GemmDesc), _p, _p, _p, _p, _p, _p, _p]),
    "tb200_device_error": (_i, []),
    "tb200_attention_fwd": (_i, [ctypes.POINTER(AttnDesc), _p, _p, _p, _p, _p, _p]),
    "tb200_attention_device_error": (_i, []),
    "tb200_attention_bwd_workspace_bytes": (_sz, [ctypes.POINTER(AttnDesc)]),
    "tb200_attention_bwd": (_i, [ctypes.POINTER(AttnDesc), _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "tb200_attention_bwd_tune": (_i, [ctypes.POINTER(AttnDesc), _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "tb200_attention_bwd_device_error": (_i, []),
    "tb200_device_errors": (_i, []),
    "tb200_rows_device_error": (_i, []),
    "tb200_deltanet_device_error": (_i, []),
    "tb200_deltanet_workspace_bytes": (_sz, [ctypes.POINTER(DeltanetDesc)]),
    "tb200_deltanet_fwd": (_i, [ctypes.POINTER(DeltanetDesc), _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "tb200_gemm_tune": (_i, [ctypes.POINTER(GemmDesc), _p, _p, _p, _p, _p, _p, _p]),
    "tb200_attention_fwd_masked": (_i, [ctypes.POINTER(AttnDesc), ctypes.POINTER(AttnMask), _p, _p, _p, _p, _p, _p]),
    "tb200_attention_bwd_masked": (_i, [ctypes.POINTER(AttnDesc), ctypes.POINTER(AttnMask)] + [_p] * 10),
    "tb200_attention_bwd_masked_workspace_bytes": (_sz, [ctypes.POINTER(AttnDesc)]),
    "tb200_attention_bwd_masked_ws": (_i, [ctypes.POINTER(AttnDesc), ctypes.POINTER(AttnMask)] + [_p] * 10 + [_sz, _p]),
    "tb200_group_route": (_i, [ctypes.POINTER(GroupDesc)]),
    "tb200_group_attention": (_i, [ctypes.POINTER(GroupDesc), _i, _i, _i, ctypes.POINTER(_p), ctypes.POINTER(_p), _p]),
    "tb200_rowreduce_generic_check": (_i, [ctypes.POINTER(GroupDesc)]),
    "tb200_rowreduce_generic": (_i, [ctypes.POINTER(GroupDesc), ctypes.POINTER(_p), ctypes.POINTER(_p), _p]),
    "tb200_rowreduce_compile": (_i, [ctypes.POINTER(GroupDesc), ctypes.c_uint, ctypes.c_uint]),
    "tb200_rowreduce_compiled": (_i, [ctypes.POINTER(GroupDesc), ctypes.POINTER(_p), ctypes.POINTER(_p), _p]),
    "tb200_rowreduce_source": (_sz, [ctypes.POINTER(GroupDesc), ctypes.c_uint, ctypes.c_uint, ctypes.c_char_p, _sz]),
    "tb200_rowreduce_compile_log": (ctypes.c_char_p, []),
    "tb200_colreduce_workspace_bytes": (_sz, [ctypes.POINTER(GroupDesc)]),
    "tb200_colreduce_compile": (_i, [ctypes.POINTER(GroupDesc)]),
    "tb200_colreduce_compiled": (_i, [ctypes.POINTER(GroupDesc), ctypes.POINTER(_p), ctypes.POINTER(_p), _p, _sz, _p]),
    "tb200_colreduce_source": (_sz, [ctypes.POINTER(GroupDesc), ctypes.c_char_p, _sz]),
    "tb200_deltanet_bwd_workspace_bytes": (_sz, [ctypes.POINTER(DeltanetDesc)]),
    "tb200_deltanet_bwd": (_i, [ctypes.POINTER(DeltanetDesc)] + [_p] * 12 + [_sz, _p]),
    "tb200_recurrence_compile": (_i, [ctypes.POINTER(RecurrenceDesc)]),
    "tb200_recurrence_source": (_sz, [ctypes.POINTER(RecurrenceDesc), ctypes.c_char_p, _sz]),
    "tb200_recurrence_compiled": (_i, [ctypes.POINTER(RecurrenceDesc), _p, _p, _p]),
    "tb200_gemm_pointers": (_i, [ctypes.POINTER(GemmDesc), _p, _p, _p, _i64, _p]),
    "tb200_scan_workspace_bytes": (_sz, [ctypes.POINTER(ScanDesc)]),
    "tb200_scan": (_i, [ctypes.POINTER(ScanDesc), _p, _p, _p, _p]),
    "tb200_dp_signal_bytes": (_sz, []),
    "tb200_dp_state_bytes": (_sz, []),
    "tb200_dp_update": (_i, [ctypes.POINTER(DpDesc), _p]),
    "tb200_dp_error": (_i, []),
    "tb200_workspace_clear": (_i, [_p, _sz, _p]),
    "tb200_squared_error_workspace_bytes": (_sz, []),
    "tb200_squared_error": (_i, [_p, _p, _p, _p, _i64, _f, _f, _i, _i, _p, _sz, _p]),
    "tb200_colsum_workspace_bytes": (_sz, [_i64, _i64]),
    "tb200_colsum": (_i, [_p, _p, _i64, _i64, _i64, _f, _i, _p, _sz, _p]),
    "tb200_axpy": (_i, [_p, _p, _f, _i64, _i, _i, _p]),
}


class TB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn, status, text):
        super().__init__(f"{fn}: status {status}: {text}")
        self.fn, self.status = fn, status


_lib = None


def load(path=None):
    """The loaded library (dlopen once). Raises if it has not been built."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python tempest.jl_b200/csrc/build.py` "
            "(the backend has no CPU fallback)")
    handle = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype, fn.argtypes = res, args
    _lib = handle
    return handle


def check(fn, status):
    if status != 0:
        lib = load()
        text = lib.tb200_strerror(status).decode()
        if status == -6:
            text += ": " + lib.tb200_last_cuda_error().decode()
        raise TB200Error(fn, status, text)


def version():
    return load().tb200_version()


def sm_count():
    n = load().tb200_sm_count()
    if n < 0:
        check("tb200_sm_count", n)
    return n


def rowop_workspace_bytes(op, n, rows, dtype):
    return load().tb200_rowop_workspace_bytes(op, n, rows, dtype)


def softmax_fwd(x, y, lse, n, rows, ld, dtype, stat_dtype=F32, workspace=0, workspace_bytes=0, stream=0):
    check("tb200_softmax_fwd", load().tb200_softmax_fwd(
        x, y, lse or None, n, rows, ld, dtype, stat_dtype, workspace or None, workspace_bytes, stream or None))


def softmax_bwd(y_or_x, lse, dy, dx, n, rows, ld, dtype, stat_dtype=F32, workspace=0, workspace_bytes=0, stream=0):
    check("tb200_softmax_bwd", load().tb200_softmax_bwd(
        y_or_x, lse or None, dy, dx, n, rows, ld, dtype, stat_dtype, workspace or None, workspace_bytes,
        stream or None))


def layernorm_fwd(x, gamma, beta, y, mean, rstd, eps, n, rows, ld, dtype, workspace=0, workspace_bytes=0, stream=0):
    check("tb200_layernorm_fwd", load().tb200_layernorm_fwd(
        x, gamma, beta or None, y, mean or None, rstd or None, eps, n, rows, ld, dtype, workspace or None,
        workspace_bytes, stream or None))


def layernorm_bwd(x, gamma, dy, mean, rstd, dx, dgamma, dbeta, eps, n, rows, ld, dtype, workspace=0,
                  workspace_bytes=0, stream=0):
    check("tb200_layernorm_bwd", load().tb200_layernorm_bwd(
        x, gamma, dy, mean or None, rstd or None, dx, dgamma or None, dbeta or None, eps, n, rows, ld, dtype,
        workspace or None, workspace_bytes, stream or None))


GEMM_A, GEMM_B, GEMM_C, GEMM_BIAS, GEMM_AUX, GEMM_AUX_OUT, GEMM_WORKSPACE = range(7)


def gemm_desc(m, n, k, *, lda=None, ldb=None, ldc=None, a_layout=K_MAJOR, b_layout=MN_MAJOR, in_dtype=BF16,
              out_dtype=None, epilogue=EPI_NONE, ld_aux=None, ld_aux_out=None, alpha=1.0, tile_n=0, force_simt=False,
              direct_epilogue=False, batch=1, stride_a=None, stride_b=None, stride_c=None, stride_bias=0,
              stride_aux=None, stride_aux_out=None, split_k=0, workspace=0, workspace_bytes=0, debug=0):
    """tb200_gemm_desc with dense defaults: leading dimensions from the layouts, batch members one after another."""
    d = GemmDesc()
    d.m, d.n, d.k = m, n, k
    d.lda = lda if lda is not None else (m if a_layout == MN_MAJOR else k)
    d.ldb = ldb if ldb is not None else (n if b_layout == MN_MAJOR else k)
    d.ldc = ldc if ldc is not None else n
    d.ld_aux = ld_aux if ld_aux is not None else n
    d.ld_aux_out = ld_aux_out if ld_aux_out is not None else n
    d.a_layout, d.b_layout = a_layout, b_layout
    d.in_dtype = in_dtype
    d.out_dtype = in_dtype if out_dtype is None else out_dtype
    d.epilogue, d.alpha, d.tile_n, d.force_simt = epilogue, alpha, tile_n, int(force_simt)
    d.direct_epilogue = int(direct_epilogue)
    d.batch = batch
    a_rows = k if a_layout == MN_MAJOR else m
    b_rows = k if b_layout == MN_MAJOR else n
    d.stride_a = stride_a if stride_a is not None else a_rows * d.lda
    d.stride_b = stride_b if stride_b is not None else b_rows * d.ldb
    d.stride_c = stride_c if stride_c is not None else m * d.ldc
    d.stride_bias = stride_bias
    d.stride_aux = stride_aux if stride_aux is not None else m * d.ld_aux
    d.stride_aux_out = stride_aux_out if stride_aux_out is not None else m * d.ld_aux_out
    d.split_k = split_k
    d.workspace, d.workspace_bytes = workspace or None, workspace_bytes
    d.debug = debug
    return d


def gemm(a, b, c, m, n, k, *, bias=0, aux=0, aux_out=0, stream=0, tune=False, **options):
    """C[m][n] = epilogue(alpha * A * B) (`options`: the fields of `gemm_desc`).  With `tune` the compiled-in tile
    variants are timed on these operands and the faster tile_n is returned (the product's result is in C either
    way).  a_layout K_MAJOR: A is [m][k]; MN_MAJOR: [k][m].  b_layout K_MAJOR: B is [n][k]; MN_MAJOR: [k][n] (a
    Julia (out,in) weight for y = w*x).  batch > 1: that many alike products, operands `stride_*` elements apart."""
    d = gemm_desc(m, n, k, **options)
    if tune:
        width = load().tb200_gemm_tune(ctypes.byref(d), a or None, b or None, c or None, bias or None,
                                       aux or None, aux_out or None, stream or None)
        check("tb200_gemm_tune", min(width, 0))
        return width
    check("tb200_gemm", load().tb200_gemm(ctypes.byref(d), a or None, b or None, c or None, bias or None,
                                          aux or None, aux_out or None, stream or None))


def gemm_pointers(desc, a, b, c, count, stream=0):
    """`count` products alike (tb200_gemm_pointers): a, b, c are device arrays of `count` device addresses."""
    check("tb200_gemm_pointers", load().tb200_gemm_pointers(ctypes.byref(desc), a, b, c, count, stream or None))


def gemm_tile_form(desc):
    """128 / 256: single-CTA tiles of that many columns; 512: 256 x 256 tiles by pairs of CTAs (tb200_gemm_tile_form)."""
    return load().tb200_gemm_tile_form(ctypes.byref(desc))


ATTN_FORM_CUDA_CORES, ATTN_FORM_TILE, ATTN_FORM_TWO_TILES, ATTN_FORM_ONE_KERNEL, ATTN_FORM_TWO_KERNELS = range(5)


def attention_form(desc, masked=False, pullback=False):
    """Which kernels compute the descriptor (tb200_attention_form): an ATTN_FORM_* value; no device needed."""
    form = load().tb200_attention_form(ctypes.byref(desc), int(masked), int(pullback))
    if form < 0:
        check("tb200_attention_form", form)
    return form


def gemm_workspace_bytes(desc):
    """Scratch a split of the product's sum wants (0: it would not split)."""
    return load().tb200_gemm_workspace_bytes(ctypes.byref(desc))


def gemm_tune_desc(desc, a, b, c, bias=0, aux=0, aux_out=0, stream=0):
    """Times every compiled-in variant (tile width, split or not, how results are stored) and leaves the fastest
    one's choices in `desc`."""
    check("tb200_gemm_tune_desc", load().tb200_gemm_tune_desc(ctypes.byref(desc), a or None, b or None, c or None,
                                                              bias or None, aux or None, aux_out or None,
                                                              stream or None))
    return desc


class GemmPlan:
    """A prepared product (tb200_gemm_plan): validation, schedule and TMA descriptors built once; `launch(stream)`
    is one C call and one kernel launch; `repoint(operand, address)` moves one operand."""

    def __init__(self, desc, a, b, c, bias=0, aux=0, aux_out=0):
        self._handle = _p()
        self.desc = desc
        check("tb200_gemm_plan_create", load().tb200_gemm_plan_create(
            ctypes.byref(desc), a or None, b or None, c or None, bias or None, aux or None, aux_out or None,
            ctypes.byref(self._handle)))
        self._launch = load().tb200_gemm_plan_launch

    def launch(self, stream=0):
        st = self._launch(self._handle, stream or None)
        if st:
            check("tb200_gemm_plan_launch", st)

    def repoint(self, operand, address):
        check("tb200_gemm_plan_repoint", load().tb200_gemm_plan_repoint(self._handle, operand, address or None))
        return self

    def close(self):
        if self._handle:
            load().tb200_gemm_plan_destroy(self._handle)
            self._handle = _p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass


def device_error():
    code = load().tb200_device_error()
    if code < 0:
        check("tb200_device_error", code)
    return code


def rows_device_error():
    """0, or 1 when a row kernel fed through shared memory gave up a bounded wait since the last call (synchronises)."""
    code = load().tb200_rows_device_error()
    if code < 0:
        check("tb200_rows_device_error", code)
    return code


def deltanet_device_error():
    """0, or 1 (forward scan) / 2 (reverse scan) when a DeltaNet scan gave up a bounded wait since the last call."""
    code = load().tb200_deltanet_device_error()
    if code < 0:
        check("tb200_deltanet_device_error", code)
    return code


def device_errors():
    """Synchronises the device; product | attention forward << 8 | attention backward << 16 | row kernels << 24 |
    DeltaNet scans << 28 of the codes the kernels record when a bounded wait gives up (0 = none), cleared by the call."""
    code = load().tb200_device_errors()
    if code < 0:
        check("tb200_device_errors", code)
    return code


def check_device():
    """Raises if any tensor-core kernel launched since the last poll gave up a bounded wait: its outputs
    are not to be used.  Call where the host synchronises anyway."""
    code = device_errors()
    if code:
        raise TB200Error("tb200_device_errors", code, "a tensor-core kernel gave up a bounded wait "
                         f"(product {code & 0xff}, attention forward {(code >> 8) & 0xff}, "
                         f"attention backward {(code >> 16) & 0xff}); results of that launch are invalid")


def workspace_clear(workspace, nbytes, stream=0):
    check("tb200_workspace_clear", load().tb200_workspace_clear(workspace, nbytes, stream or None))


def squared_error_workspace_bytes():
    return load().tb200_squared_error_workspace_bytes()


def squared_error(a, b, grad, loss, count, scale, grad_scale, through_tanh, dtype, workspace, workspace_bytes,
                  stream=0):
    check("tb200_squared_error", load().tb200_squared_error(
        a, b or None, grad or None, loss, count, scale, grad_scale, int(through_tanh), dtype, workspace,
        workspace_bytes, stream or None))


def colsum_workspace_bytes(rows, n):
    return load().tb200_colsum_workspace_bytes(rows, n)


def colsum(x, out, rows, n, ld, scale, dtype, workspace, workspace_bytes, stream=0):
    check("tb200_colsum", load().tb200_colsum(x, out, rows, n, ld, scale, dtype, workspace or None, workspace_bytes,
                                              stream or None))


def axpy(y, x, alpha, count, y_dtype, x_dtype, stream=0):
    check("tb200_axpy", load().tb200_axpy(y, x, alpha, count, y_dtype, x_dtype, stream or None))


def layernorm_bwd_noalloc_max_row():
    return load().tb200_layernorm_bwd_noalloc_max_row()


def layernorm_bwd_noalloc(x, gamma, dy, mean, rstd, dx, dgamma, dbeta, eps, n, rows, ld, dtype, stream=0):
    """tb200_layernorm_bwd for callers without scratch memory to give: the partial
    sums use the library's built-in 8 MiB array (see the header for the limits)."""
    check("tb200_layernorm_bwd_noalloc", load().tb200_layernorm_bwd_noalloc(
        x, gamma, dy, mean or None, rstd or None, dx, dgamma or None, dbeta or None, eps, n, rows, ld, dtype,
        stream or None))


def attn_desc(batch, heads, queries, keys, head_dim, causal, scale=None, kv_heads=None, dtype=BF16,
              deterministic=False, value_dim=0):
    d = AttnDesc()
    d.deterministic = int(deterministic)
    d.value_dim = int(value_dim)
    d.batch, d.heads, d.kv_heads = batch, heads, kv_heads or heads
    d.queries, d.keys, d.head_dim = queries, keys, head_dim
    d.causal = int(causal)
    d.scale = scale if scale is not None else head_dim ** -0.5
    d.dtype = dtype
    return d


def attention_fwd(desc, q, k, v, o, lse=0, stream=0):
    """q, o: [batch][queries][heads][head_dim]; k, v: [batch][keys][kv_heads][head_dim]; lse: [batch][queries][heads]."""
    check("tb200_attention_fwd", load().tb200_attention_fwd(ctypes.byref(desc), q, k, v, o, lse or None,
                                                            stream or None))


def attention_device_error():
    code = load().tb200_attention_device_error()
    if code < 0:
        check("tb200_attention_device_error", code)
    return code


def attention_bwd_workspace_bytes(desc):
    return load().tb200_attention_bwd_workspace_bytes(ctypes.byref(desc))


def attention_bwd(desc, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream=0):
    check("tb200_attention_bwd", load().tb200_attention_bwd(
        ctypes.byref(desc), q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream or None))


def attention_bwd_tune(desc, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream=0):
    """Times the pullback's two forms on these operands; returns the `deterministic` value (0 or 1) of the faster."""
    form = load().tb200_attention_bwd_tune(ctypes.byref(desc), q, k, v, o, lse, dout, dq, dk, dv, workspace,
                                           workspace_bytes, stream or None)
    check("tb200_attention_bwd_tune", min(form, 0))
    return form


def attention_bwd_device_error():
    code = load().tb200_attention_bwd_device_error()
    if code < 0:
        check("tb200_attention_bwd_device_error", code)
    return code


def deltanet_desc(heads, positions, dk=128, dv=128, chunk=64, dtype=BF16):
    d = DeltanetDesc()
    d.heads, d.positions, d.dk, d.dv, d.chunk, d.dtype = heads, positions, dk, dv, chunk, dtype
    return d


def deltanet_workspace_bytes(desc):
    return load().tb200_deltanet_workspace_bytes(ctypes.byref(desc))


def deltanet_fwd(desc, q, k, v, a, beta, o, workspace, workspace_bytes, stream=0):
    """q, k [heads][T][dk], v [heads][T][dv] BFloat16; a, beta [heads][T] Float32; o [heads][dv][T] BFloat16."""
    check("tb200_deltanet_fwd", load().tb200_deltanet_fwd(ctypes.byref(desc), q, k, v, a, beta, o, workspace,
                                                          workspace_bytes, stream or None))


def deltanet_bwd_workspace_bytes(desc):
    return load().tb200_deltanet_bwd_workspace_bytes(ctypes.byref(desc))


def deltanet_bwd(desc, q, k, v, a, beta, dout, dq, dk, dv, da, dbeta, workspace, workspace_bytes, stream=0):
    """Pullback of `deltanet_fwd`: dout [heads][dv][T]; dq, dk, dv in the inputs' layouts (BFloat16); da, dbeta Float32."""
    check("tb200_deltanet_bwd", load().tb200_deltanet_bwd(ctypes.byref(desc), q, k, v, a, beta, dout, dq, dk, dv, da,
                                                          dbeta, workspace, workspace_bytes, stream or None))


def rowreduce_generic_check(desc):
    return load().tb200_rowreduce_generic_check(ctypes.byref(desc))


def rowreduce_generic(desc, inputs, outputs, stream=0):
    """Runs a generic map -> fold row group: `inputs`, `outputs` are device addresses in the descriptor's order."""
    ins = (_p * max(len(inputs), 1))(*inputs)
    outs = (_p * max(len(outputs), 1))(*outputs)
    check("tb200_rowreduce_generic", load().tb200_rowreduce_generic(ctypes.byref(desc), ins, outs, stream or None))


def rowreduce_compile(desc, vector_inputs=0xff, vector_outputs=0xff):
    """Compiles (and caches) the group's own kernel; needs NVRTC, not a device.  Returns the status."""
    return load().tb200_rowreduce_compile(ctypes.byref(desc), vector_inputs, vector_outputs)


def rowreduce_source(desc, vector_inputs=0xff, vector_outputs=0xff):
    need = load().tb200_rowreduce_source(ctypes.byref(desc), vector_inputs, vector_outputs, None, 0)
    if not need:
        return ""
    buf = ctypes.create_string_buffer(need)
    load().tb200_rowreduce_source(ctypes.byref(desc), vector_inputs, vector_outputs, buf, need)
    return buf.value.decode()


def rowreduce_compile_log():
    return (load().tb200_rowreduce_compile_log() or b"").decode()


def rowreduce_compiled(desc, inputs, outputs, stream=0):
    """The compiled form of `rowreduce_generic`: same arguments, the group's own kernel."""
    ins = (_p * max(len(inputs), 1))(*inputs)
    outs = (_p * max(len(outputs), 1))(*outputs)
    check("tb200_rowreduce_compiled", load().tb200_rowreduce_compiled(ctypes.byref(desc), ins, outs, stream or None))


def colreduce_workspace_bytes(desc):
    return load().tb200_colreduce_workspace_bytes(ctypes.byref(desc))


def colreduce_compile(desc):
    """Compiles a group whose folds run over the rows (needs NVRTC, no device)."""
    check("tb200_colreduce_compile", load().tb200_colreduce_compile(ctypes.byref(desc)))


def colreduce_source(desc):
    need = load().tb200_colreduce_source(ctypes.byref(desc), None, 0)
    if not need:
        return ""
    buf = ctypes.create_string_buffer(need)
    load().tb200_colreduce_source(ctypes.byref(desc), buf, need)
    return buf.value.decode()


def colreduce_compiled(desc, inputs, outputs, workspace=0, workspace_bytes=0, stream=0):
    """A group whose folds run over the rows: outputs[j] receives `n` values of fold outputs[j].index."""
    ins = (_p * max(len(inputs), 1))(*inputs)
    outs = (_p * max(len(outputs), 1))(*outputs)
    check("tb200_colreduce_compiled", load().tb200_colreduce_compiled(ctypes.byref(desc), ins, outs, workspace or None,
                                                                      workspace_bytes, stream or None))


def attn_mask(doc_start=0, kv_len=0, q_stride=(0, 0, 0), kv_stride=(0, 0, 0)):
    m = AttnMask()
    m.doc_start, m.kv_len = doc_start or None, kv_len or None
    m.q_stride[:] = q_stride
    m.kv_stride[:] = kv_stride
    return m


def attention_fwd_masked(desc, mask, q, k, v, o, lse=0, stream=0):
    check("tb200_attention_fwd_masked", load().tb200_attention_fwd_masked(
        ctypes.byref(desc), ctypes.byref(mask), q, k, v, o, lse or None, stream or None))


def attention_bwd_masked(desc, mask, q, k, v, o, lse, dout, dq, dk, dv, stream=0):
    check("tb200_attention_bwd_masked", load().tb200_attention_bwd_masked(
        ctypes.byref(desc), ctypes.byref(mask), q, k, v, o, lse, dout, dq, dk, dv, stream or None))


def attention_bwd_masked_workspace_bytes(desc):
    return load().tb200_attention_bwd_masked_workspace_bytes(ctypes.byref(desc))


def attention_bwd_masked_ws(desc, mask, q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes, stream=0):
    """The masked pullback on the tensor cores (128 features, dense arrays), either form (`desc.deterministic`)."""
    check("tb200_attention_bwd_masked_ws", load().tb200_attention_bwd_masked_ws(
        ctypes.byref(desc), ctypes.byref(mask), q, k, v, o, lse, dout, dq, dk, dv, workspace, workspace_bytes,
        stream or None))


def dp_signal_bytes():
    return load().tb200_dp_signal_bytes()


def dp_state_bytes():
    return load().tb200_dp_state_bytes()


def dp_desc(rank, world, count, alpha, grads, params, signals, state, grads_multicast=0, params_multicast=0, blocks=0):
    """tb200_dp_desc: `grads`, `params`, `signals` are lists of addresses in rank order (this process's mappings)."""
    d = DpDesc()
    d.rank, d.world, d.blocks, d.dtype, d.count, d.alpha = rank, world, blocks, BF16, count, alpha
    for i in range(world):
        d.grads[i], d.params[i], d.signals[i] = grads[i] or None, params[i] or None, signals[i] or None
    d.grads_multicast, d.params_multicast = grads_multicast or None, params_multicast or None
    d.state = state or None
    return d


def dp_update(desc, stream=0):
    check("tb200_dp_update", load().tb200_dp_update(ctypes.byref(desc), stream or None))


def dp_error():
    code = load().tb200_dp_error()
    if code < 0:
        check("tb200_dp_error", code)
    return code


def recurrence_compile(desc):
    check("tb200_recurrence_compile", load().tb200_recurrence_compile(ctypes.byref(desc)))


def recurrence_source(desc):
    need = load().tb200_recurrence_source(ctypes.byref(desc), None, 0)
    if need == 0:
        return ""
    buf = ctypes.create_string_buffer(need)
    load().tb200_recurrence_source(ctypes.byref(desc), buf, need)
    return buf.value.decode()


def recurrence_compiled(desc, inputs, outputs, stream=0):
    """A recurrence whose step is a map (tb200_recurrence_compiled): inputs / outputs in the descriptor's order."""
    ins = (ctypes.c_void_p * max(len(inputs), 1))(*inputs)
    outs = (ctypes.c_void_p * max(len(outputs), 1))(*outputs)
    check("tb200_recurrence_compiled", load().tb200_recurrence_compiled(ctypes.byref(desc), ins, outs, stream or None))


def scan_desc(n, rows, op, *, across=False, reverse=False, dtype=F32, ld_x=None, ld_x2=None, ld_y=None, batch=1,
              stride_x=None, stride_x2=None, stride_y=None, workspace=0, workspace_bytes=0):
    d = ScanDesc()
    d.n, d.rows, d.op, d.across, d.reverse, d.dtype, d.batch = n, rows, op, int(across), int(reverse), dtype, batch
    d.ld_x = n if ld_x is None else ld_x
    d.ld_x2 = n if ld_x2 is None else ld_x2
    d.ld_y = n if ld_y is None else ld_y
    d.stride_x = rows * d.ld_x if stride_x is None else stride_x
    d.stride_x2 = rows * d.ld_x2 if stride_x2 is None else stride_x2
    d.stride_y = rows * d.ld_y if stride_y is None else stride_y
    d.workspace, d.workspace_bytes = workspace or None, workspace_bytes
    return d


def scan_workspace_bytes(desc):
    """Scratch with which a scan across the rows is split into slabs of rows (0: the form has no use for it)."""
    return load().tb200_scan_workspace_bytes(ctypes.byref(desc))


def scan(x, y, n, rows, op, *, x2=0, across=False, reverse=False, dtype=F32, ld_x=None, ld_x2=None, ld_y=None, batch=1,
         stride_x=None, stride_x2=None, stride_y=None, workspace=0, workspace_bytes=0, stream=0):
    """y = running fold of x (tb200_scan): along each row of the (n, rows) matrix, or across its rows."""
    d = ScanDesc()
    d.workspace, d.workspace_bytes = workspace or None, workspace_bytes
    d.n, d.rows, d.op, d.across, d.reverse, d.dtype, d.batch = n, rows, op, int(across), int(reverse), dtype, batch
    d.ld_x = n if ld_x is None else ld_x
    d.ld_x2 = n if ld_x2 is None else ld_x2
    d.ld_y = n if ld_y is None else ld_y
    d.stride_x = rows * d.ld_x if stride_x is None else stride_x
    d.stride_x2 = rows * d.ld_x2 if stride_x2 is None else stride_x2
    d.stride_y = rows * d.ld_y if stride_y is None else stride_y
    check("tb200_scan", load().tb200_scan(ctypes.byref(d), x or None, x2 or None, y or None, stream or None))


ROUTE_NONE, ROUTE_ATTENTION, ROUTE_ATTENTION_CAUSAL = 0, 1, 2


def group_route(desc):
    """Which dedicated kernel computes this group (ROUTE_*), judged by the structure of its terms."""
    r = load().tb200_group_route(ctypes.byref(desc))
    if r < 0:
        check("tb200_group_route", r)
    return r


def group_attention(desc, heads, kv_heads, batch, inputs, outputs, stream=0):
    """Runs a descriptor that `group_route` recognised as attention on the attention kernels."""
    ins = (_p * max(len(inputs), 1))(*inputs)
    outs = (_p * max(len(outputs), 1))(*outputs)
    check("tb200_group_attention", load().tb200_group_attention(ctypes.byref(desc), heads, kv_heads, batch, ins, outs,
                                                                stream or None))
