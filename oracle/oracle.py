"""Python face of the CPU oracle (test infrastructure only).

Loads oracle/liboracle.so (the C restatement of Tempest.jl's reference CPU
path, built by `make -C oracle`) and wraps each function over numpy arrays.
BFloat16 arrays are numpy uint16 holding the bit patterns.  Only the tests,
the smoke check and the benchmark's CPU-baseline leg may import this module.

Also here: the reference's deterministic test-data generator
`data(dims...; scale) = 2 sin(scale * (1:n))` (test/setup.jl:33), the seeded
N(0,1) generator every config's synthetic inputs come from, and Float64
closed forms used as a second yardstick.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i64, _int, _flt, _void = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def build(force=False):
    srcs = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".c", ".inc"))]
    srcs.append(os.path.join(os.path.dirname(HERE), "include", "tempest_b200.h"))   # group.c reads its data layouts
    if force or not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in srcs):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB


_lib = None


def load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_sum_f32.restype = ctypes.c_float
        _lib.oracle_sum_abs2_f32.restype = ctypes.c_float
        _lib.oracle_sum_bf16.restype = ctypes.c_uint16
        _lib.oracle_logsumexp_f32.restype = ctypes.c_float
        _lib.oracle_readme_loss_grad.restype = ctypes.c_float
        _lib.oracle_gelu_tanh.restype = ctypes.c_float
        _lib.oracle_gelu_tanh.argtypes = [_flt]
        _lib.oracle_gelu_tanh_grad.restype = ctypes.c_float
        _lib.oracle_gelu_tanh_grad.argtypes = [_flt]
    return _lib


def threads_available():
    """Host cores this process may use."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover
        return os.cpu_count() or 1


def _over_rows(call, rows, threads):
    """Runs call(r0, r1) over [0, rows): on this thread, or on `threads`
    threads over disjoint row ranges (rows are independent items, and ctypes
    releases the GIL, so results are the single-thread results)."""
    if threads <= 1 or rows < 2:
        call(0, rows)
        return
    from concurrent.futures import ThreadPoolExecutor
    parts = min(threads * 4, rows)
    edges = [rows * i // parts for i in range(parts + 1)]
    with ThreadPoolExecutor(threads) as pool:
        list(pool.map(lambda i: call(edges[i], edges[i + 1]), range(parts)))


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_void)


# ------------------------------------------------------------------ data ----

def data(*dims, scale=1.0):
    """test/setup.jl:33 -- 2 sin(scale * k), k = 1..prod(dims), as a Julia
    column-major array of `dims`; returned as the numpy array whose C-order
    memory is the Julia array's memory (axes reversed)."""
    n = int(np.prod(dims))
    flat = 2.0 * np.sin(scale * np.arange(1, n + 1, dtype=np.float64))
    return flat.reshape(tuple(reversed(dims)))


def normal(shape, seed, dtype=np.float32):
    """Seeded N(0,1) draws (numpy Philox, counter-based): the synthetic inputs."""
    g = np.random.Generator(np.random.Philox(seed))
    return g.standard_normal(shape, dtype=np.float32).astype(dtype, copy=False)


def to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    load().oracle_bf16_from_f32(_ptr(x), _ptr(out), _i64(x.size))
    return out


def from_bf16(h):
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, np.float32)
    load().oracle_f32_from_bf16(_ptr(h), _ptr(out), _i64(h.size))
    return out


# ----------------------------------------------------------------- folds ----

def sum_f32(x):
    x = np.ascontiguousarray(x, np.float32)
    return float(load().oracle_sum_f32(_ptr(x), _i64(x.size)))


def sum_abs2_f32(x):
    x = np.ascontiguousarray(x, np.float32)
    return float(load().oracle_sum_abs2_f32(_ptr(x), _i64(x.size)))


def sum_bf16(h):
    h = np.ascontiguousarray(h, np.uint16)
    return int(load().oracle_sum_bf16(_ptr(h), _i64(h.size)))


def logsumexp_f32(x):
    x = np.ascontiguousarray(x, np.float32)
    return float(load().oracle_logsumexp_f32(_ptr(x), _i64(x.size)))


def mean_var_f32(x):
    x = np.ascontiguousarray(x, np.float32)
    m, v = ctypes.c_float(), ctypes.c_float()
    load().oracle_mean_var_f32(_ptr(x), _i64(x.size), ctypes.byref(m), ctypes.byref(v))
    return m.value, v.value


def scan(x, op, x2=None, across=False, reverse=False):
    """The running fold of a [rows][n] Float32 array (or BFloat16 bits: widened, scanned in Float32, rounded once),
    element after element in sequence: along each row, or across the rows (one scan per column).  op: "sum", "prod",
    "max", "min", "affine" (h = x h + x2 from h = 0), "variance" (running population variance)."""
    code = {"sum": 0, "prod": 1, "max": 2, "min": 3, "affine": 4, "variance": 5}[op]
    if x.dtype == np.uint16:
        out = scan(from_bf16(x), op, None if x2 is None else from_bf16(x2), across, reverse)
        return to_bf16(out)
    x = np.ascontiguousarray(x, np.float32)
    x2c = None if x2 is None else np.ascontiguousarray(x2, np.float32)
    y = np.empty_like(x)
    rows, n = x.shape
    fn = load().oracle_scan_f32
    for k in range(n if across else rows):
        off = k if across else k * n
        fn(_ptr(x.reshape(-1)[off:]), None if x2c is None else _ptr(x2c.reshape(-1)[off:]), _ptr(y.reshape(-1)[off:]),
           _i64(rows if across else n), _i64(n if across else 1), _int(code), _int(int(reverse)))
    return y


# ------------------------------------------------------------ row kernels ----

def _rows(x):
    assert x.ndim == 2 and x.flags.c_contiguous
    return x.shape[1], x.shape[0]


def softmax_fwd(x, faithful=True, threads=1):
    """x: [rows][n] float32 or uint16 (bf16 bits) -> (y, lse float32)."""
    n, rows = _rows(x)
    y = np.empty_like(x)
    lse = np.empty(rows, np.float32)
    L = load()

    def call(r0, r1):
        if x.dtype == np.float32:
            L.oracle_softmax_fwd_f32(_ptr(x[r0:r1]), _ptr(y[r0:r1]), _ptr(lse[r0:r1]), _i64(n), _i64(r1 - r0), _i64(n))
        else:
            L.oracle_softmax_fwd_bf16(_ptr(x[r0:r1]), _ptr(y[r0:r1]), _ptr(lse[r0:r1]), _i64(n), _i64(r1 - r0),
                                      _i64(n), _int(int(faithful)))
    _over_rows(call, rows, threads)
    return y, lse


def softmax_bwd(y, g, faithful=True, threads=1):
    n, rows = _rows(y)
    dx = np.empty_like(y)
    L = load()

    def call(r0, r1):
        if y.dtype == np.float32:
            L.oracle_softmax_bwd_f32(_ptr(y[r0:r1]), _ptr(g[r0:r1]), _ptr(dx[r0:r1]), _i64(n), _i64(r1 - r0), _i64(n))
        else:
            L.oracle_softmax_bwd_bf16(_ptr(y[r0:r1]), _ptr(g[r0:r1]), _ptr(dx[r0:r1]), _i64(n), _i64(r1 - r0),
                                      _i64(n), _int(int(faithful)))
    _over_rows(call, rows, threads)
    return dx


def layernorm_fwd(x, gamma, beta=None, eps=1e-5, faithful=True, threads=1):
    n, rows = _rows(x)
    y = np.empty_like(x)
    mean, rstd = np.empty(rows, np.float32), np.empty(rows, np.float32)
    L = load()

    def call(r0, r1):
        if x.dtype == np.float32:
            L.oracle_layernorm_fwd_f32(_ptr(x[r0:r1]), _ptr(gamma), _ptr(beta), _ptr(y[r0:r1]), _ptr(mean[r0:r1]),
                                       _ptr(rstd[r0:r1]), _flt(eps), _i64(n), _i64(r1 - r0), _i64(n))
        else:
            L.oracle_layernorm_fwd_bf16(_ptr(x[r0:r1]), _ptr(gamma), _ptr(beta), _ptr(y[r0:r1]), _ptr(mean[r0:r1]),
                                        _ptr(rstd[r0:r1]), _flt(eps), _i64(n), _i64(r1 - r0), _i64(n),
                                        _int(int(faithful)))
    _over_rows(call, rows, threads)
    return y, mean, rstd


def layernorm_bwd(x, gamma, g, eps=1e-5, wide=False, threads=1):
    """With threads > 1 only dx is formed (per row range); dgamma and dbeta, sums
    over all rows in order, need the single thread and come back as None."""
    n, rows = _rows(x)
    dx = np.empty_like(x)
    fn = load().oracle_layernorm_bwd_f32 if x.dtype == np.float32 else load().oracle_layernorm_bwd_bf16
    if threads <= 1:
        dgamma, dbeta = np.empty(n, x.dtype), np.empty(n, x.dtype)
        fn(_ptr(x), _ptr(gamma), _ptr(g), _ptr(dx), _ptr(dgamma), _ptr(dbeta), _flt(eps), _i64(n), _i64(rows),
           _i64(n), _int(int(wide)))
        return dx, dgamma, dbeta

    def call(r0, r1):
        fn(_ptr(x[r0:r1]), _ptr(gamma), _ptr(g[r0:r1]), _ptr(dx[r0:r1]), None, None, _flt(eps), _i64(n),
           _i64(r1 - r0), _i64(n), _int(0))
    _over_rows(call, rows, threads)
    return dx, None, None


# ------------------------------------------------------------------ GEMM ----

def gemm(A, B, bias=None, M=None, N=None, K=None, a_km=False, b_kn=True, epilogue=0, threads=1, want_pre=False):
    """C[M][N] = A * B (+bias, activation); float32 or bf16 bits (uint16)."""
    C = np.empty((M, N), A.dtype)
    if A.dtype == np.float32:
        load().oracle_gemm_f32(_ptr(A), _ptr(B), _ptr(bias), _ptr(C), _i64(M), _i64(N), _i64(K), _int(int(a_km)),
                               _int(int(b_kn)), _int(epilogue))
        return C
    pre = np.empty((M, N), np.float32) if want_pre else None
    load().oracle_gemm_bf16(_ptr(A), _ptr(B), _ptr(bias), _ptr(C), _ptr(pre), _i64(M), _i64(N), _i64(K),
                            _int(int(a_km)), _int(int(b_kn)), _int(epilogue))
    return (C, pre) if want_pre else C


def gelu_tanh(x):
    return load().oracle_gelu_tanh(float(x))


def gelu_tanh_grad(x):
    return load().oracle_gelu_tanh_grad(float(x))


def readme_loss_grad(w, b, x):
    """w: Julia (I,J) as numpy [J][I]; b: [J]; x: Julia (I,N) as numpy [N][I]."""
    J, I = w.shape
    N = x.shape[0]
    dw, db, dx = np.empty_like(w), np.empty_like(b), np.empty_like(x)
    loss = load().oracle_readme_loss_grad(_ptr(w), _ptr(b), _ptr(x), _ptr(dw), _ptr(db), _ptr(dx), _i64(I), _i64(J),
                                          _i64(N))
    return float(loss), dw, db, dx


# ------------------------------------------------- Float64 closed forms -----

def softmax_fwd_f64(x):
    x = x.astype(np.float64)
    m = x.max(axis=1, keepdims=True)
    e = np.exp(x - m)
    s = e.sum(axis=1, keepdims=True)
    return e / s, (m + np.log(s))[:, 0]


def softmax_bwd_f64(y, g):
    y, g = y.astype(np.float64), g.astype(np.float64)
    return y * (g - (y * g).sum(axis=1, keepdims=True))


def layernorm_fwd_f64(x, gamma, beta=None, eps=1e-5):
    x = x.astype(np.float64)
    m = x.mean(axis=1, keepdims=True)
    v = ((x - m) ** 2).mean(axis=1, keepdims=True)
    y = (x - m) / np.sqrt(v + eps) * gamma.astype(np.float64)
    return y if beta is None else y + beta.astype(np.float64)


def layernorm_bwd_f64(x, gamma, g, eps=1e-5):
    x, g, gamma = x.astype(np.float64), g.astype(np.float64), gamma.astype(np.float64)
    m = x.mean(axis=1, keepdims=True)
    v = ((x - m) ** 2).mean(axis=1, keepdims=True)
    rstd = 1.0 / np.sqrt(v + eps)
    xh = (x - m) * rstd
    gh = g * gamma
    dx = rstd * (gh - gh.mean(axis=1, keepdims=True) - xh * (gh * xh).mean(axis=1, keepdims=True))
    return dx, (g * xh).sum(axis=0), g.sum(axis=0)


# ------------------------------------------------------------ MLP step ----

def _gelu_grad_f32(z):
    z = z.astype(np.float32)
    u = np.float32(0.7978846) * (z + np.float32(0.044715) * z * z * z)
    t = np.tanh(u)
    du = np.float32(0.7978846) * (np.float32(1.0) + np.float32(3.0 * 0.044715) * z * z)
    return (np.float32(0.5) * (1 + t) + np.float32(0.5) * z * (1 - t * t) * du).astype(np.float32)


def mlp_step(ws, bs, x, y, rate, global_batch=None):
    """One training step of examples/mlp.jl:13-35 with GELU(tanh) between layers
    (test/fixtures/programs.jl:19), BFloat16 arrays (uint16 bit patterns), every
    product accumulated in Float32 and rounded once (program/interpret.jl:59-63),
    every stored array rounded to BFloat16, everything in between Float32.
    ws[i] is a Julia (out, in) weight, i.e. numpy [in][out]; x [batch][in]; y [batch][out].
    Returns loss, [dz], [dw (Float32, before rounding)], [db (Float32)], new ws, new bs."""
    L = len(ws)
    batch = x.shape[0]
    gb = global_batch or batch
    a, z = [x], []
    for i in range(L):
        fin, fout = ws[i].shape
        out, pre = gemm(a[-1], ws[i], bias=bs[i], M=batch, N=fout, K=fin, a_km=False, b_kn=True,
                        epilogue=1 if i == L - 1 else 2, want_pre=True)
        a.append(out)
        z.append(to_bf16(pre))
    d = from_bf16(a[-1]) - from_bf16(y)
    loss = float(np.sum(d.astype(np.float64) ** 2) / gb)
    dz = [None] * L
    dz[L - 1] = to_bf16((np.float32(1.0 / gb) * (np.float32(2.0) * d)).astype(np.float32))
    dws, dbs, new_w, new_b = [None] * L, [None] * L, [None] * L, [None] * L
    for i in range(L - 1, -1, -1):
        fin, fout = ws[i].shape
        if i > 0:
            _, acc = gemm(dz[i], ws[i], M=batch, N=fin, K=fout, a_km=False, b_kn=False, epilogue=0, want_pre=True)
            dz[i - 1] = to_bf16(acc * _gelu_grad_f32(from_bf16(z[i - 1])))
        dbs[i] = from_bf16(dz[i]).astype(np.float64).sum(axis=0).astype(np.float32)
        _, dws[i] = gemm(a[i], dz[i], M=fin, N=fout, K=batch, a_km=True, b_kn=True, epilogue=0, want_pre=True)
        new_w[i] = to_bf16(from_bf16(ws[i]) - np.float32(rate) * dws[i])
        new_b[i] = to_bf16(from_bf16(bs[i]) - np.float32(rate) * from_bf16(to_bf16(dbs[i])))
    return loss, dz, dws, dbs, new_w, new_b, a, z


def mlp_step_blas(ws, bs, x, y, rate, global_batch=None):
    """`mlp_step` at sizes the scalar products cannot reach (the benchmark's 1024-4096-4096-4096-1024 at batch
    8192 is 2 TFLOP): the same arithmetic with the same rounding points -- BFloat16 arrays widened to Float32,
    every product accumulated in Float32 and rounded once where it is stored -- but the products taken by
    numpy's Float32 matmul (BLAS) instead of sequential sums, which changes the order of summation only.
    Returns loss, [dz bits], [dw Float32], [db Float32], [new w bits], [new b bits], [a bits], [z bits]."""
    L = len(ws)
    batch = x.shape[0]
    gb = global_batch or batch
    W = [from_bf16(w) for w in ws]
    a, z = [x], []
    h = from_bf16(x)
    for i in range(L):
        pre = h @ W[i] + from_bf16(bs[i])[None, :]
        zb = to_bf16(pre)
        z.append(zb)
        if i == L - 1:
            out = zb
        else:
            u = np.float32(0.7978846) * (pre + np.float32(0.044715) * pre * pre * pre)
            out = to_bf16(np.float32(0.5) * pre * (np.float32(1.0) + np.tanh(u)))
        a.append(out)
        h = from_bf16(out)
    d = from_bf16(a[-1]) - from_bf16(y)
    loss = float(np.sum(d.astype(np.float64) ** 2) / gb)
    dz = [None] * L
    dz[L - 1] = to_bf16((np.float32(1.0 / gb) * (np.float32(2.0) * d)).astype(np.float32))
    dws, dbs, new_w, new_b = [None] * L, [None] * L, [None] * L, [None] * L
    for i in range(L - 1, -1, -1):
        g = from_bf16(dz[i])
        if i > 0:
            dz[i - 1] = to_bf16((g @ W[i].T) * _gelu_grad_f32(from_bf16(z[i - 1])))
        dbs[i] = g.astype(np.float64).sum(axis=0).astype(np.float32)
        dws[i] = from_bf16(a[i]).T @ g
        new_w[i] = to_bf16(W[i] - np.float32(rate) * dws[i])
        new_b[i] = to_bf16(from_bf16(bs[i]) - np.float32(rate) * from_bf16(to_bf16(dbs[i])))
    return loss, dz, dws, dbs, new_w, new_b, a, z


# ------------------------------------------------------------- attention ----

def _pool(jobs, threads):
    if threads <= 1:
        for j in jobs:
            j()
        return
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(threads) as pool:
        list(pool.map(lambda j: j(), jobs))


def attention_fwd(q, k, v, causal, scale=None, round_p=False, threads=1):
    """q [B][S][H][D], k/v [B][Skv][Hkv][D] as BFloat16 bits (uint16).  Returns (o bits, lse float32 [B][S][H])."""
    B, S, H, D = q.shape
    _, Skv, Hkv, _ = k.shape
    scale = float(D) ** -0.5 if scale is None else scale
    o = np.empty_like(q)
    lse = np.empty((B, S, H), np.float32)
    fn = load().oracle_attention_fwd_rows
    step = max(1, S // max(1, threads // max(1, B * H) + 1))
    jobs = []
    for b in range(B):
        for h in range(H):
            for m0 in range(0, S, step):
                jobs.append(lambda b=b, h=h, m0=m0: fn(
                    _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _int(B), _int(H), _int(Hkv), _int(S), _int(Skv),
                    _int(D), _int(int(causal)), _flt(scale), _int(b), _int(h), _int(m0), _int(min(S, m0 + step)),
                    _int(int(round_p))))
    _pool(jobs, threads)
    return o, lse


def attention_bwd(q, k, v, o, lse, dout, causal, scale=None, round_p=False, threads=1):
    """The pullback of attention_fwd: (dq, dk, dv) as BFloat16 bits."""
    B, S, H, D = q.shape
    _, Skv, Hkv, _ = k.shape
    scale = float(D) ** -0.5 if scale is None else scale
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    fn = load().oracle_attention_bwd_head
    jobs = [lambda b=b, hk=hk: fn(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(dout), _ptr(dq), _ptr(dk),
                                  _ptr(dv), _int(B), _int(H), _int(Hkv), _int(S), _int(Skv), _int(D),
                                  _int(int(causal)), _flt(scale), _int(b), _int(hk), _int(int(round_p)))
            for b in range(B) for hk in range(Hkv)]
    _pool(jobs, threads)
    return dq, dk, dv


def attention_f64(q, k, v, causal, scale=None, dout=None, doc_start=None, kv_len=None):
    """Float64 closed form on the BFloat16 inputs: (o, lse) and, with dout, (dq, dk, dv).
    doc_start [B][S] (0-based first key each query sees) and kv_len [B] are the masks of the reference's
    packed-documents and decode programs (test/cuda/attention.jl:223-228, 256-260); a query that sees no key
    gets a zero output, a log-sum-exp of -Inf and no gradient."""
    qf, kf, vf = (from_bf16(a).astype(np.float64) for a in (q, k, v))
    B, S, H, D = qf.shape
    Skv, Hkv = kf.shape[1], kf.shape[2]
    g = H // Hkv
    scale = float(D) ** -0.5 if scale is None else scale
    kx, vx = np.repeat(kf, g, axis=2), np.repeat(vf, g, axis=2)
    s = np.einsum("bmhd,bnhd->bhmn", qf, kx) * scale
    if causal:
        mask = np.arange(Skv)[None, :] > np.arange(S)[:, None]
        s = np.where(mask[None, None], -np.inf, s)
    if doc_start is not None:
        before = np.arange(Skv)[None, None, :] < np.asarray(doc_start)[:, :, None]      # [B][S][Skv]
        s = np.where(before[:, None], -np.inf, s)
    if kv_len is not None:
        beyond = np.arange(Skv)[None, :] >= np.asarray(kv_len)[:, None]                  # [B][Skv]
        s = np.where(beyond[:, None, None, :], -np.inf, s)
    mx = s.max(axis=-1, keepdims=True)
    mx = np.where(np.isfinite(mx), mx, 0.0)
    e = np.exp(s - mx)
    l = e.sum(axis=-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        p = np.where(l > 0, e / l, 0.0)
        lse = np.where(l > 0, mx + np.log(l), -np.inf)[..., 0].transpose(0, 2, 1)
    o = np.einsum("bhmn,bnhd->bmhd", p, vx)
    if dout is None:
        return o, lse
    go = from_bf16(dout).astype(np.float64)
    dvx = np.einsum("bhmn,bmhd->bnhd", p, go)
    dp = np.einsum("bmhd,bnhd->bhmn", go, vx)
    delta = (go * o).sum(axis=-1).transpose(0, 2, 1)[..., None]
    ds = p * (dp - delta)
    dq = np.einsum("bhmn,bnhd->bmhd", ds, kx) * scale
    dkx = np.einsum("bhmn,bmhd->bnhd", ds, qf) * scale
    dk = dkx.reshape(B, Skv, Hkv, g, D).sum(axis=3)
    dv = dvx.reshape(B, Skv, Hkv, g, vf.shape[-1]).sum(axis=3)   # the values may have features of their own
    return o, lse, dq, dk, dv


# -------------------------------------------------------------- DeltaNet ----

def group_eval(desc, inputs, outputs, threads=1, wide=False):
    """Runs a generic map -> fold row group (a `tb200_group_desc` ctypes structure) on the host, rows in
    order: the floor of src/Compiler/codegen/scalar.jl:200-256 over the descriptor.  `inputs`, `outputs`:
    numpy arrays (uint16 for BFloat16) in the descriptor's order; outputs are written in place.
    `wide` evaluates in Float64 instead (same storage types)."""
    fn = load().oracle_group_rows_f64 if wide else load().oracle_group_rows
    fn.restype = ctypes.c_int
    ins = (ctypes.c_void_p * max(len(inputs), 1))(*[a.ctypes.data for a in inputs])
    outs = (ctypes.c_void_p * max(len(outputs), 1))(*[a.ctypes.data for a in outputs])

    def call(r0, r1):
        if fn(ctypes.byref(desc), ins, outs, _i64(r0), _i64(r1)) != 0:
            raise ValueError("oracle cannot run this group")
    _over_rows(call, int(desc.rows), threads)
    return outputs


def group_eval_cols(desc, inputs, wide=False):
    """A generic group whose folds run over the rows (the other axis), on the host: the term DAG evaluated per
    element, then each column folded over its rows in order (the sequential floor of
    src/Compiler/codegen/scalar.jl:200-256 for a fold over the second axis).  Float32 arithmetic, or Float64
    with `wide`.  `inputs`: numpy arrays in the descriptor's order (uint16 for BFloat16; full inputs
    [rows][ld]).  Returns one array of `n` values per output, in its storage type."""
    F = np.float64 if wide else np.float32
    n, rows = int(desc.n), int(desc.rows)
    vals = []
    for i in range(desc.n_inputs):
        inp = desc.inputs[i]
        a = np.asarray(inputs[i])
        a = from_bf16(a) if inp.dtype == 1 else a
        a = a.astype(F)
        if inp.shape == 0:
            a = a.reshape(rows, -1)[:, :n]
        elif inp.shape == 1:
            a = a.reshape(1, n)
        elif inp.shape == 2:
            a = a.reshape(rows, 1)
        else:
            a = a.reshape(1, 1)
        vals.append(a)
    unary = {11: lambda x: -x, 12: np.exp, 13: np.log, 14: np.tanh, 15: np.sqrt, 16: lambda x: F(1) / np.sqrt(x),
             17: np.abs, 18: lambda x: x * x, 19: lambda x: F(1) / x, 20: lambda x: F(1) / (F(1) + np.exp(-x)),
             23: lambda x: from_bf16(to_bf16(x.astype(np.float32))).astype(F)}
    binary = {5: np.add, 6: np.subtract, 7: np.multiply, 8: np.divide, 9: np.maximum, 10: np.minimum}
    t = []
    with np.errstate(all="ignore"):
        for k in range(desc.n_terms):
            T = desc.terms[k]
            if T.op == 0:
                v = vals[T.a]
            elif T.op == 1:
                v = np.full((1, 1), T.imm, F)
            elif T.op == 2:
                v = np.arange(n, dtype=F).reshape(1, n)
            elif T.op in binary:
                v = binary[T.op](t[T.a], t[T.b]).astype(F)
            elif T.op in unary:
                v = unary[T.op](t[T.a]).astype(F)
            elif T.op == 21:
                v = (t[T.a].astype(np.float64) * t[T.b] + t[T.c]).astype(F) if not wide else t[T.a] * t[T.b] + t[T.c]
            elif T.op == 22:
                v = np.where(t[T.a] > 0, t[T.b], t[T.c]).astype(F)
            else:
                raise ValueError("oracle cannot run this group")
            t.append(v)
        folded = []
        for j in range(desc.n_folds):
            kind, term = desc.folds[j].kind, desc.folds[j].term
            v = np.broadcast_to(t[term], (rows, n))
            if kind == 4:
                # the online log-sum-exp, row after row: (maximum, sum of exp(y - maximum)) rebased when the maximum
                # moves (src/Compiler/IR/folds.jl:123-198)
                m, ssum = np.full(n, -np.inf, F), np.zeros(n, F)
                for r in range(rows):
                    m2 = np.maximum(m, v[r])
                    shift = np.where(np.isfinite(m2), m2, F(0))
                    ssum = (ssum * np.exp(m - shift) + np.exp(v[r] - shift)).astype(F)
                    m = m2.astype(F)
                folded.append((np.where(ssum > 0, m + np.log(ssum), m).astype(F), None))
                continue
            if kind == 5:
                # Welford's update of (count, mean, centred sum of squares), row after row (folds.jl:143, 166-182)
                mean, m2s = np.zeros(n, F), np.zeros(n, F)
                for r in range(rows):
                    d = (v[r] - mean).astype(F)
                    mean = (mean + d / F(r + 1)).astype(F)
                    m2s = (m2s + d * (v[r] - mean)).astype(F)
                folded.append((mean, (m2s / F(max(rows, 1))).astype(F)))
                continue
            ident = {0: 0.0, 1: -np.inf, 2: np.inf, 3: 1.0}[kind]
            step = {0: np.add, 1: np.maximum, 2: np.minimum, 3: np.multiply}[kind]
            acc = np.full(n, ident, F)
            for r in range(rows):
                acc = step(acc, v[r]).astype(F)
            folded.append((acc, None))
    outs = []
    for o in range(desc.n_outputs):
        first, second = folded[desc.outputs[o].index]
        v = (second if desc.outputs[o].source == 2 else first).astype(np.float32)
        outs.append(to_bf16(v) if desc.outputs[o].dtype == 1 else v)
    return outs


def deltanet_sequential(q, k, v, a, beta, threads=1):
    """The gated delta rule token by token in Float64 (examples/deltanet.jl:89-101).
    q, k [heads][T][dk], v [heads][T][dv] BFloat16 bits; a, beta [heads][T] float32.
    Returns o [heads][dv][T] float64 (the Julia (T, dv, heads) result's memory)."""
    Hn, T, dk = q.shape
    dv = v.shape[2]
    o = np.zeros((Hn, dv, T), np.float64)
    a = np.ascontiguousarray(a, np.float32)
    beta = np.ascontiguousarray(beta, np.float32)
    fn = load().oracle_deltanet_head
    jobs = [lambda h=h: fn(_ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(beta), _ptr(o), _int(T), _int(dk), _int(dv), _int(h))
            for h in range(Hn)]
    _pool(jobs, threads)
    return o


def deltanet_sequential_bwd(q, k, v, a, beta, dout):
    """Pullback of the token-by-token rule (examples/deltanet.jl:89-101) in Float64, by reverse
    accumulation over positions: with r = k' S_prev, Y = S_prev - beta k r', S = g Y + beta k v', o = S' q,
      dS += q do';  dq = S do;  dg = <dS, Y>;  dY = g dS;
      dbeta = k' dS v - k' dY r;  dv = beta dS' k;  dk = beta dS v - beta (dY r + S_prev dY' k);
      dS_prev = dY - beta k (k' dY);  da = dg g.
    q, k, v BFloat16 bits [heads][T][d]; a, beta float32 [heads][T]; dout float64 [heads][dv][T].
    Returns dq, dk, dv [heads][T][d], da, dbeta [heads][T], all float64.  Keeps every state: small T only."""
    Q, K, V = (from_bf16(x).astype(np.float64) for x in (q, k, v))
    A, B = a.astype(np.float64), beta.astype(np.float64)
    Hn, T, dk = Q.shape
    dv_ = V.shape[2]
    dQ, dK, dV = np.zeros_like(Q), np.zeros_like(K), np.zeros_like(V)
    dA, dB = np.zeros_like(A), np.zeros_like(B)
    for h in range(Hn):
        states = np.zeros((T + 1, dk, dv_))
        for t in range(T):
            S, kt, g, b = states[t], K[h, t], np.exp(A[h, t]), B[h, t]
            states[t + 1] = g * (S - b * np.outer(kt, kt @ S)) + b * np.outer(kt, V[h, t])
        dS = np.zeros((dk, dv_))
        for t in range(T - 1, -1, -1):
            Sp, S, kt, vt, g, b = states[t], states[t + 1], K[h, t], V[h, t], np.exp(A[h, t]), B[h, t]
            do = dout[h, :, t]
            dS = dS + np.outer(Q[h, t], do)
            dQ[h, t] = S @ do
            r = kt @ Sp
            Y = Sp - b * np.outer(kt, r)
            dA[h, t] = (dS * Y).sum() * g
            dY = g * dS
            dSv, dYr, dYk = dS @ vt, dY @ r, dY.T @ kt
            dB[h, t] = kt @ dSv - kt @ dYr
            dV[h, t] = b * (dS.T @ kt)
            dK[h, t] = b * dSv - b * (dYr + Sp @ dYk)
            dS = dY - b * np.outer(kt, dYk)
    return dQ, dK, dV, dA, dB


def deltanet_inputs(heads, T, dk, dv, seed):
    """The benchmark's distributions: q, k ~ N(0,1) L2-normalised per position, v ~ N(0,1),
    beta = sigmoid(N(0,1)), a = -softplus(N(0,1))."""
    q = normal((heads, T, dk), seed)
    k = normal((heads, T, dk), seed + 1)
    q /= np.linalg.norm(q, axis=-1, keepdims=True)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = normal((heads, T, dv), seed + 2)
    beta = (1.0 / (1.0 + np.exp(-normal((heads, T), seed + 3)))).astype(np.float32)
    a = (-np.log1p(np.exp(normal((heads, T), seed + 4)))).astype(np.float32)
    return to_bf16(q), to_bf16(k), to_bf16(v), a, beta


def recurrence_eval(desc, inputs):
    """A recurrence whose step is a map (include/tempest_b200.h, tb200_recurrence_desc), step by step in Float32 as the
    reference's CPU path runs a recurrence (one step at a time, every member as its node's eltype: Float32 here, results
    rounded once where they are stored): inputs in the descriptor's order (numpy; BFloat16 as uint16 bits).  Returns
    the outputs in the descriptor's order (Float32 arrays, or uint16 bits for BFloat16 outputs)."""
    import numpy as np
    d = desc.body
    n, steps = int(d.n), int(d.rows)
    f32 = np.float32
    arrays = []
    for i in range(d.n_inputs):
        a = np.asarray(inputs[i])
        arrays.append(from_bf16(a).astype(f32) if d.inputs[i].dtype == 1 else a.astype(f32))
    def start(k):
        i = desc.states[k].start
        v = arrays[i].reshape(-1)
        return np.full(n, v[0], f32) if d.inputs[i].shape == 3 else v[:n].astype(f32).copy()
    state = [start(k) for k in range(desc.n_states)]
    outs = []
    for o in range(d.n_outputs):
        outs.append(np.zeros((steps, n), f32) if d.outputs[o].source == 0 else np.zeros(n, f32))
    cols = np.arange(n, dtype=f32)
    unary = {11: lambda a: -a, 12: np.exp, 13: np.log, 14: np.tanh, 15: np.sqrt, 16: lambda a: f32(1) / np.sqrt(a), 17: np.abs,
             18: lambda a: a * a, 19: lambda a: f32(1) / a, 20: lambda a: f32(1) / (f32(1) + np.exp(-a)),
             23: lambda a: from_bf16(to_bf16(a)).astype(f32)}
    binary = {5: np.add, 6: np.subtract, 7: np.multiply, 8: np.divide, 9: np.maximum, 10: np.minimum}
    with np.errstate(all="ignore"):
        for s in range(steps):
            row = steps - 1 - s if desc.reverse else s
            t = []
            for k in range(d.n_terms):
                T = d.terms[k]
                if T.op == 0:
                    shape = d.inputs[T.a].shape
                    a = arrays[T.a]
                    v = (a.reshape(steps, -1)[row, :n] if shape == 0 else a.reshape(-1)[:n] if shape == 1
                         else np.full(n, a.reshape(-1)[row], f32) if shape == 2 else np.full(n, a.reshape(-1)[0], f32))
                elif T.op == 1:
                    v = np.full(n, T.imm, f32)
                elif T.op == 2:
                    v = cols
                elif T.op == 25:
                    v = np.full(n, row, f32)
                elif T.op == 26:
                    v = state[T.a]
                elif T.op in binary:
                    v = binary[T.op](t[T.a], t[T.b])
                elif T.op == 21:
                    v = (t[T.a].astype(np.float64) * t[T.b].astype(np.float64) + t[T.c].astype(np.float64))   # fused: one rounding
                elif T.op == 22:
                    v = np.where(t[T.a] > 0, t[T.b], t[T.c])
                else:
                    v = unary[T.op](t[T.a])
                t.append(np.asarray(v).astype(f32))
            for o in range(d.n_outputs):
                if d.outputs[o].source == 0:
                    outs[o][row] = t[d.outputs[o].index]
            state = [t[desc.states[k].next].copy() for k in range(desc.n_states)]
    for o in range(d.n_outputs):
        if d.outputs[o].source == 3:
            outs[o] = state[d.outputs[o].index]
        if d.outputs[o].dtype == 1:
            outs[o] = to_bf16(outs[o])
    return outs
