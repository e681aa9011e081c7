"""ctypes binding of libtempest_b200.so: one Python function per C-ABI entry point.

Arguments are raw device addresses (ints), extents and strides in elements,
and a CUDA stream handle; nothing here touches torch.  A missing or unbuilt
library raises: there is no CPU fallback.
"""
import ctypes
import os

F32, BF16 = 0, 1
SOFTMAX_FWD, SOFTMAX_BWD, LAYERNORM_FWD, LAYERNORM_BWD = 0, 1, 2, 3

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtempest_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "tempest_b200.h")

_p, _i, _i64, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t

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
