"""Parity of the fused row kernels with the CPU oracle, through the C ABI
(Binding -> build -> launch).  Shapes follow the reference's fold tests
(test/cuda/folds.jl:16-25: 256x700, 9000x40, 512x300, ...) plus ragged,
unaligned, empty and split-schedule cases; the full benchmark shape
(4096 x 65536) is checked on sampled rows and through properties that hold at
any size."""
import numpy as np
import pytest

from helpers import ATOL_BF16, RTOL_F32, Runner, agree, agree_bf16

pytestmark = pytest.mark.gpu

# (rows, n): reduced axis n is contiguous
SHAPES = [
    (700, 256), (40, 9000), (300, 512), (64, 4096),      # reference fold tests + the config's row length
    (1, 1), (3, 1), (1, 7), (133, 8), (70, 33), (5, 200), (129, 1000),  # ragged / tiny
    (9, 4100), (6, 16384), (3, 12288),                    # widest resident rows
    (5, 20000), (2, 70001), (3, 32768), (1, 262144),      # split schedule
]


@pytest.fixture(scope="module")
def run(pkg, cuda):
    return Runner(pkg, cuda)


def inputs(oracle, rows, n, seed):
    x = oracle.normal((rows, n), seed)
    g = oracle.normal((rows, n), seed + 1)
    w = (1.0 + 0.25 * oracle.normal((n,), seed + 2)).astype(np.float32)
    b = (0.5 * oracle.normal((n,), seed + 3)).astype(np.float32)
    return x, g, w, b


@pytest.mark.parametrize("rows,n", SHAPES)
def test_softmax_f32(run, oracle, rows, n):
    x, g, _, _ = inputs(oracle, rows, n, 100 + n)
    y, lse = run.softmax(x)
    y_ref, lse_ref = oracle.softmax_fwd(x)
    agree(y, y_ref, RTOL_F32)
    agree(lse, lse_ref, RTOL_F32)
    y64, lse64 = oracle.softmax_fwd_f64(x)
    agree(y, y64, RTOL_F32)
    dx = run.softmax_pullback(y_ref, g)
    agree(dx, oracle.softmax_bwd(y_ref, g), RTOL_F32)
    agree(dx, oracle.softmax_bwd_f64(y_ref, g), RTOL_F32)
    # the planner's other choice: y recomputed from x and the saved log-sum-exp
    agree(run.softmax_pullback_recomputed(x, lse_ref, g), oracle.softmax_bwd_f64(y64, g), 2 * RTOL_F32)


@pytest.mark.parametrize("rows,n", SHAPES)
def test_layernorm_f32(run, oracle, rows, n):
    x, g, w, b = inputs(oracle, rows, n, 200 + n)
    y, mean, rstd = run.layernorm(x, w, b, stats=True)
    y_ref, mean_ref, rstd_ref = oracle.layernorm_fwd(x, w, b)
    if n > 1:
        y64 = oracle.layernorm_fwd_f64(x, w, b)
        agree(y, y64, RTOL_F32)
        # the oracle folds each row sequentially in Float32 as the reference's CPU path does, which
        # itself drifts from Float64 as rows grow: allow its own distance on top of the tolerance
        drift = np.linalg.norm(y_ref - y64) / np.linalg.norm(y64)
        agree(y, y_ref, RTOL_F32 + drift)
        agree(rstd, rstd_ref, RTOL_F32 + drift)
    agree(mean, x.astype(np.float64).mean(axis=1), RTOL_F32)
    agree(run.layernorm(x, w), oracle.layernorm_fwd_f64(x, w), RTOL_F32)
    dx, dw, db = run.layernorm_pullback(x, w, g)
    dx64, dw64, db64 = oracle.layernorm_bwd_f64(x, w, g)
    agree(dx, dx64, 2 * RTOL_F32)
    agree(dw, dw64, 2 * RTOL_F32)
    agree(db, db64, RTOL_F32)
    dx_ref, dw_ref, db_ref = oracle.layernorm_bwd(x, w, g, wide=True)
    agree(dx, dx_ref, 4 * RTOL_F32)
    agree(dw, dw_ref, 4 * RTOL_F32)
    # with the forward's saved statistics instead of recomputing them
    dx2, dw2, db2 = run.layernorm_pullback(x, w, g, mean_ref, rstd_ref)
    agree(dx2, dx64, 4 * RTOL_F32)
    agree(db2, db64, RTOL_F32)


BF16_SHAPES = [(700, 256), (64, 4096), (40, 9000), (7, 24), (5, 333), (3, 16384), (2, 40000), (4, 32768)]


@pytest.mark.parametrize("rows,n", BF16_SHAPES)
def test_softmax_bf16(run, oracle, rows, n):
    x, g, _, _ = inputs(oracle, rows, n, 300 + n)
    xb, gb = oracle.to_bf16(x), oracle.to_bf16(g)
    y, lse = run.softmax(xb)
    y_ref, lse_ref = oracle.softmax_fwd(xb, faithful=False)  # Float32 inside, one rounding
    agree_bf16(y, oracle.from_bf16(y_ref), oracle)
    y64, lse64 = oracle.softmax_fwd_f64(oracle.from_bf16(xb))
    agree_bf16(y, y64, oracle)
    agree(lse, lse64, RTOL_F32)
    # statistic stored in the element type, as the plan's value has it
    _, lse_b = run.softmax(xb, stat="BFloat16")
    agree_bf16(lse_b, lse64, oracle)
    dx = run.softmax_pullback(y_ref, gb)
    agree_bf16(dx, oracle.softmax_bwd_f64(oracle.from_bf16(y_ref), oracle.from_bf16(gb)), oracle)
    agree_bf16(dx, oracle.from_bf16(oracle.softmax_bwd(y_ref, gb, faithful=False)), oracle)


@pytest.mark.parametrize("rows,n", BF16_SHAPES)
def test_layernorm_bf16(run, oracle, rows, n):
    x, g, w, b = inputs(oracle, rows, n, 400 + n)
    xb, gb, wb, bb = (oracle.to_bf16(a) for a in (x, g, w, b))
    xf, gf, wf, bf = (oracle.from_bf16(a) for a in (xb, gb, wb, bb))
    y = run.layernorm(xb, wb, bb)
    agree_bf16(y, oracle.layernorm_fwd_f64(xf, wf, bf), oracle)
    agree_bf16(y, oracle.from_bf16(oracle.layernorm_fwd(xb, wb, bb, faithful=False)[0]), oracle)
    dx, dw, db = run.layernorm_pullback(xb, wb, gb)
    dx64, dw64, db64 = oracle.layernorm_bwd_f64(xf, wf, gf)
    agree_bf16(dx, dx64, oracle)
    agree_bf16(dw, dw64, oracle)
    agree_bf16(db, db64, oracle)


@pytest.mark.parametrize("eltype", ["Float32", "BFloat16"])
@pytest.mark.parametrize("rows,n", [(64, 1024), (6, 2048), (1000, 4096), (7, 4096), (2, 4096), (1500, 2048)])
def test_layernorm_pullback_with_saved_statistics(run, oracle, rows, n, eltype):
    """Rows of 1024, 2048 and 4096 elements with the forward's mean and rstd handed in take the kernel that is fed
    through a ring in shared memory (several rows a block, rows in whole turns; an odd row count falls back to the
    resident kernels): the same results as the Float64 pullback, and nothing recorded by its bounded waits."""
    x, g, w, _ = inputs(oracle, rows, n, 900 + n + rows)
    if eltype == "BFloat16":
        xb, gb, wb = (oracle.to_bf16(a) for a in (x, g, w))
        xf, gf, wf = (oracle.from_bf16(a) for a in (xb, gb, wb))
    else:
        xb, gb, wb = xf, gf, wf = x, g, w
    x64 = xf.astype(np.float64)
    mean = x64.mean(axis=1).astype(np.float32)
    rstd = (1.0 / np.sqrt(x64.var(axis=1) + 1e-5)).astype(np.float32)
    dx, dw, db = run.layernorm_pullback(xb, wb, gb, mean, rstd)
    dx64, dw64, db64 = oracle.layernorm_bwd_f64(xf, wf, gf)
    if eltype == "BFloat16":
        agree_bf16(dx, dx64, oracle)
        agree_bf16(dw, dw64, oracle)
        agree_bf16(db, db64, oracle)
    else:
        agree(dx, dx64, 4 * RTOL_F32)
        agree(dw, dw64, 4 * RTOL_F32)
        agree(db, db64, RTOL_F32)
    again = run.layernorm_pullback(xb, wb, gb, mean, rstd)
    for a, b in zip((dx, dw, db), again):
        assert np.array_equal(a, b)
    assert run.pkg.lib.rows_device_error() == 0


def test_leading_dimension_and_unaligned_views(run, oracle, cuda):
    """Rows with a leading dimension larger than n, and views that start off a
    16-byte boundary (a value at an offset inside a shared slot)."""
    L = run.pkg.lib
    rows, n, ld = 37, 1000, 1003
    x = oracle.normal((rows, n), 7)
    buf = cuda.zeros(rows * ld + 8, device="cuda")
    out = cuda.full((rows * ld + 8,), -7.0, device="cuda")
    for off in (0, 1, 3):
        view = buf[off:off + rows * ld].view(rows, ld)
        view[:, :n] = cuda.from_numpy(x).cuda()
        I = run.I
        b = I.Binding("softmax_columns", {"n": n, "rows": rows},
                      {"x": I.Strided("Float32", off, (n, rows), (1, ld), buf, 1),
                       "y": I.Strided("Float32", off, (n, rows), (1, ld), out, 2)})
        launch, _ = run.lib.build(run.target, b, run.resources)
        launch()
        cuda.cuda.synchronize()
        got = out[off:off + rows * ld].view(rows, ld).cpu().numpy()
        agree(got[:, :n], oracle.softmax_fwd(x)[0], RTOL_F32)
        assert (got[:, n:] == -7.0).all(), "wrote outside the rows"
        out.fill_(-7.0)


def test_in_place_and_repoint(run, oracle, cuda):
    """y may share x's storage (`in_place`), and `repoint!` moves an operand."""
    I = run.I
    rows, n = 50, 2048
    x = oracle.normal((rows, n), 9)
    a, b2 = run.dev(x), run.dev(x * 0.5)
    bind = I.Binding("softmax_columns", {"n": n, "rows": rows},
                     {"x": I.dense_columns(a, "Float32", n, rows, 1), "y": I.dense_columns(a, "Float32", n, rows, 1)})
    launch, _ = run.lib.build(run.target, bind, run.resources)
    launch()
    cuda.cuda.synchronize()
    agree(a.cpu().numpy(), oracle.softmax_fwd(x)[0], RTOL_F32)
    launch.repoint(1, b2)
    launch()
    cuda.cuda.synchronize()
    agree(b2.cpu().numpy(), oracle.softmax_fwd(x * 0.5)[0], RTOL_F32)


def test_empty_and_infinite_rows(run, oracle, cuda):
    L = run.pkg.lib
    stream = cuda.cuda.current_stream().cuda_stream
    # rows of no elements: the log-sum-exp of nothing is -Inf (src/Compiler/IR/folds.jl:121-127)
    lse = cuda.zeros(5, device="cuda")
    L.softmax_fwd(0, 0, lse.data_ptr(), 0, 5, 0, L.F32, stream=stream)
    cuda.cuda.synchronize()
    assert (lse.cpu().numpy() == -np.inf).all()
    # no rows: nothing runs, nothing is read
    L.softmax_fwd(0, 0, 0, 128, 0, 128, L.F32, stream=stream)
    # a row holding -Inf entries (a causal mask's) and one holding +Inf
    x = oracle.normal((4, 64), 3)
    x[0, 10:] = -np.inf
    x[1, :] = -np.inf
    x[2, 5] = np.inf
    y, lse = run.softmax(x)
    y_ref, lse_ref = oracle.softmax_fwd(x)
    assert np.array_equal(np.isnan(y), np.isnan(y_ref))
    ok = ~np.isnan(y_ref)
    agree(y[ok], y_ref[ok], RTOL_F32)
    assert lse[1] == -np.inf and lse[2] == np.inf
    agree(lse[[0, 3]], lse_ref[[0, 3]], RTOL_F32)


def test_errors_are_statuses(run, oracle, cuda):
    L = run.pkg.lib
    x = run.dev(oracle.normal((2, 40000), 1))
    with pytest.raises(L.TB200Error) as e:  # split schedule without its workspace
        L.softmax_fwd(x.data_ptr(), x.data_ptr(), 0, 40000, 2, 40000, L.F32)
    assert e.value.status == -5
    with pytest.raises(L.TB200Error) as e:  # the streamed LayerNorm backward (long rows) without its workspace
        L.layernorm_bwd(x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, 0, x.data_ptr(), 0, 0, 1e-5, 40000, 2, 40000,
                        L.F32)
    assert e.value.status == -5
    # the context is still usable
    y, _ = run.softmax(oracle.normal((2, 64), 2))
    assert np.isfinite(y).all()


def test_runs_repeat_bit_for_bit(run, oracle):
    x, g, w, _ = inputs(oracle, 300, 4096, 77)
    first = run.layernorm_pullback(x, w, g)
    again = run.layernorm_pullback(x, w, g)
    for a, b in zip(first, again):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("eltype", ["Float32", "BFloat16"])
def test_full_size_config(run, oracle, cuda, eltype):
    """The benchmark shape, X 4096 x 65536: sampled rows against the oracle,
    and properties that hold at any size (softmax rows sum to one, its
    pullback's rows to zero; LayerNorm rows have mean 0 and variance 1; the
    pullbacks are linear in the upstream gradient)."""
    I, L, torch = run.I, run.pkg.lib, cuda
    rows, n = 65536, 4096
    dt = torch.float32 if eltype == "Float32" else torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(20261125)
    x = torch.randn(rows, n, device="cuda", generator=gen, dtype=torch.float32).to(dt)
    g = torch.randn(rows, n, device="cuda", generator=gen, dtype=torch.float32).to(dt)
    w = torch.ones(n, device="cuda", dtype=dt)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    lse = torch.empty(rows, device="cuda")
    sample = np.r_[0:8, 30000:30008, rows - 8:rows]

    def host(t, idx=sample):
        t = t[torch.from_numpy(idx).cuda()]
        return t.view(torch.int16).cpu().numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.cpu().numpy()

    def check(got, want64):
        if eltype == "Float32":
            agree(got, want64, 2 * RTOL_F32)
        else:
            agree_bf16(got, want64, oracle)

    def widen(a):
        return a if a.dtype == np.float32 else oracle.from_bf16(a)

    def launch(template, arrays):
        b = I.Binding(template, {"n": n, "rows": rows}, arrays)
        fn, _ = run.lib.build(run.target, b, run.resources)
        fn()
        torch.cuda.synchronize()

    col = lambda t, v: I.dense_columns(t, eltype, n, rows, v)
    xs, gs = host(x), host(g)
    # softmax forward
    launch("softmax_columns_lse", {"x": col(x, 1), "y": col(y, 2), "lse": I.Strided("Float32", 0, (1, rows), (1, 1), lse, 3)})
    y64, lse64 = oracle.softmax_fwd_f64(widen(xs))
    check(host(y), y64)
    agree(host(lse), lse64, RTOL_F32)
    sums = y.float().sum(dim=1)
    assert float((sums - 1).abs().max()) < (1e-4 if eltype == "Float32" else 2e-2)
    # softmax pullback: rows sum to zero; linear in g
    ys = host(y)
    launch("softmax_columns_pullback", {"y": col(y, 1), "g": col(g, 2), "dx": col(dx, 3)})
    check(host(dx), oracle.softmax_bwd_f64(widen(ys), widen(gs)))
    assert float(dx.float().sum(dim=1).abs().max()) < (1e-4 if eltype == "Float32" else 2e-2)
    # LayerNorm forward: normalised rows
    launch("layernorm", {"x": col(x, 1), "w": I.dense_vector(w, eltype, n, 2), "y": col(y, 3)})
    check(host(y), oracle.layernorm_fwd_f64(widen(xs), np.ones(n, np.float32)))
    yf = y.float()
    assert float(yf.mean(dim=1).abs().max()) < (1e-4 if eltype == "Float32" else 1e-2)
    assert float((yf.var(dim=1, unbiased=False) - 1).abs().max()) < (1e-3 if eltype == "Float32" else 2e-2)
    # LayerNorm pullback: sampled dx, and dbeta = column sums of g over all 65536 rows
    dw, db = torch.empty_like(w), torch.empty_like(w)
    launch("layernorm_pullback", {"x": col(x, 1), "w": I.dense_vector(w, eltype, n, 2), "g": col(g, 3),
                                  "dx": col(dx, 4), "dw": I.dense_vector(dw, eltype, n, 5),
                                  "db": I.dense_vector(db, eltype, n, 6)})
    dx64, _, _ = oracle.layernorm_bwd_f64(widen(xs), np.ones(n, np.float32), widen(gs))
    check(host(dx), dx64)
    db_ref = g.double().sum(dim=0)
    xh = (x.double() - x.double().mean(dim=1, keepdim=True))
    xh = xh / torch.sqrt((xh * xh).mean(dim=1, keepdim=True) + 1e-5)
    dw_ref = (g.double() * xh).sum(dim=0)
    if eltype == "Float32":
        agree(db.cpu().numpy(), db_ref.cpu().numpy(), RTOL_F32)
        agree(dw.cpu().numpy(), dw_ref.cpu().numpy(), 2 * RTOL_F32)
    else:
        # sums of 65536 terms reach hundreds: one BFloat16 ulp of the value
        full = np.arange(n)
        agree_bf16(db.view(torch.int16).cpu().numpy().view(np.uint16), db_ref.cpu().numpy(), oracle)
        agree_bf16(dw.view(torch.int16).cpu().numpy().view(np.uint16), dw_ref.cpu().numpy(), oracle)
