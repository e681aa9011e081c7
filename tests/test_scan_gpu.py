"""Scans through the C ABI against the CPU oracle's sequential sweeps, on the shapes and folds of the reference's
scan tests (test/cuda/scans.jl:12-34): cumulative sums along the first axis, a middle one and the last, of a long
vector and of a matrix taken whole, cumprod, accumulate(max), the GenericFold recurrence and variance, BFloat16,
reversed scans, and the degenerate shapes.  Tolerance: the reference's own rtol 1e-4 (its `agree`), since a scan
spread over threads combines partial states in another order than the sequential sweep."""
import numpy as np
import pytest

from helpers import agree

pytestmark = pytest.mark.gpu

OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "affine": 4, "variance": 5}


def run(pkg, torch, x, op, x2=None, across=False, reverse=False, slabs=False):
    """x: [batch][rows][n] or [rows][n] numpy (Float32, or uint16 BFloat16 bits).  `slabs`: hand over the scratch
    with which a scan across the rows is split into runs of rows."""
    L = pkg.lib
    bf = x.dtype == np.uint16
    to = lambda a: (torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16) if bf else torch.from_numpy(np.ascontiguousarray(a))).cuda()  # noqa: E731
    xd = to(x)
    x2d = to(x2) if x2 is not None else None
    y = torch.full_like(xd, float("nan"))
    batch = x.shape[0] if x.ndim == 3 else 1
    rows, n = x.shape[-2], x.shape[-1]
    ws, need = None, 0
    if slabs:
        need = L.scan_workspace_bytes(L.scan_desc(n, rows, OPS[op], across=across, reverse=reverse,
                                                   dtype=L.BF16 if bf else L.F32, batch=batch))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    L.scan(xd.data_ptr(), y.data_ptr(), n, rows, OPS[op], x2=x2d.data_ptr() if x2d is not None else 0, across=across,
           reverse=reverse, dtype=L.BF16 if bf else L.F32, batch=batch, workspace=ws.data_ptr() if ws is not None else 0,
           workspace_bytes=need)
    torch.cuda.synchronize()
    return y.view(torch.int16).cpu().numpy().view(np.uint16) if bf else y.cpu().numpy()


def want(oracle, x, op, x2=None, across=False, reverse=False):
    if x.ndim == 3:
        return np.stack([oracle.scan(x[i], op, None if x2 is None else x2[i], across, reverse) for i in range(x.shape[0])])
    return oracle.scan(x, op, x2, across, reverse)


def single(a):
    return np.ascontiguousarray(a, np.float32)


@pytest.mark.parametrize("reverse", [False, True])
def test_cumulative_sums(pkg, cuda, oracle, reverse):
    x = single(oracle.data(1000, 64))                       # Julia (1000, 64): memory [64][1000]
    for across in (False, True):                            # dims = 1 (along), dims = 2 (across)
        agree(run(pkg, cuda, x, "sum", across=across, reverse=reverse), want(oracle, x, "sum", across=across, reverse=reverse), 1e-4)
    v = single(oracle.data(5000)).reshape(1, 5000)          # cumsum of a vector: more than one tile of a block
    agree(run(pkg, cuda, v, "sum", reverse=reverse), want(oracle, v, "sum", reverse=reverse), 1e-4)
    m = single(oracle.data(16, 300, 8))                     # dims = 2 of (16, 300, 8): across 300 rows of 16, a batch of 8
    agree(run(pkg, cuda, m, "sum", across=True, reverse=reverse), want(oracle, m, "sum", across=True, reverse=reverse), 1e-4)
    w = single(oracle.data(30, 40)).reshape(1, 1200)        # accumulate(+, x) over the whole matrix in memory order
    agree(run(pkg, cuda, w, "sum", reverse=reverse), want(oracle, w, "sum", reverse=reverse), 1e-4)


def test_products_extrema_and_user_folds(pkg, cuda, oracle):
    x = single(oracle.data(1000, 64))
    p = single(1 + 0.001 * x)
    agree(run(pkg, cuda, p, "prod"), want(oracle, p, "prod"), 1e-4)
    for op in ("max", "min"):
        for across in (False, True):
            assert np.array_equal(run(pkg, cuda, x, op, across=across), want(oracle, x, op, across=across))   # no rounding in an extremum
    a = single(0.9 + 0.1 * oracle.data(700, 32, scale=0.3))
    b = single(oracle.data(700, 32, scale=0.7))
    for across in (False, True):
        for reverse in (False, True):
            agree(run(pkg, cuda, a, "affine", b, across=across, reverse=reverse),
                  want(oracle, a, "affine", b, across=across, reverse=reverse), 1e-4)
    v = single(oracle.data(300, 20))
    agree(run(pkg, cuda, v, "variance"), want(oracle, v, "variance"), 1e-4)
    agree(run(pkg, cuda, v, "variance", across=True), want(oracle, v, "variance", across=True), 1e-4)
    # the recurrence's documented answer (src/Compiler/IR/folds.jl:279-288)
    got = run(pkg, cuda, np.full((1, 3), 0.5, np.float32), "affine", np.ones((1, 3), np.float32))
    assert got.ravel().tolist() == [1.0, 1.5, 1.75]


def test_bfloat16_and_long_rows(pkg, cuda, oracle):
    h = oracle.to_bf16(single(oracle.data(500, 16)))        # cumsum of BFloat16.(data(500, 16)) along dims = 1
    got, ref = run(pkg, cuda, h, "sum"), want(oracle, h, "sum")
    gf, rf = oracle.from_bf16(got).astype(np.float64), oracle.from_bf16(ref).astype(np.float64)
    assert (np.abs(gf - rf) <= 2.0 ** -7 * np.abs(rf) + 1e-3).all()      # one BFloat16 ulp where the sums round apart
    got = run(pkg, cuda, h, "sum", across=True)
    rf = oracle.from_bf16(want(oracle, h, "sum", across=True)).astype(np.float64)
    assert (np.abs(oracle.from_bf16(got) - rf) <= 2.0 ** -7 * np.abs(rf) + 1e-3).all()
    long = single(oracle.normal((3, 70001), 5))             # rows of many tiles, a ragged last one
    agree(run(pkg, cuda, long, "sum"), want(oracle, long, "sum"), 1e-4)
    agree(run(pkg, cuda, long, "max", reverse=True), want(oracle, long, "max", reverse=True), 1e-6)


def test_degenerate_shapes_and_refusals(pkg, cuda, oracle):
    torch, L = cuda, pkg.lib
    one = np.array([[3.0]], np.float32)
    assert run(pkg, cuda, one, "sum").tolist() == [[3.0]] and run(pkg, cuda, one, "variance").tolist() == [[0.0]]
    row = single(oracle.data(1, 3))                         # cumsum(x; dims = 1) of a (1, 3) matrix: three scans of one element
    assert np.array_equal(run(pkg, cuda, row, "sum"), row)
    col = single(oracle.data(3, 1))                         # sum(abs2, cumsum(x; dims = 2)) of (3, 1): across one row
    assert np.array_equal(run(pkg, cuda, col, "sum", across=True), col)
    x = torch.zeros(8, device="cuda")
    L.scan(0, 0, 0, 5, 0)                                   # nothing to scan
    with pytest.raises(L.TB200Error) as e:
        L.scan(x.data_ptr(), x.data_ptr(), 8, 1, 9)
    assert e.value.status == -7
    with pytest.raises(L.TB200Error) as e:
        L.scan(x.data_ptr(), x.data_ptr(), 8, 1, OPS["affine"])     # the recurrence needs its second array
    assert e.value.status == -1
    with pytest.raises(L.TB200Error) as e:
        L.scan(x.data_ptr(), x.data_ptr(), 8, 1, 0, ld_x=4)
    assert e.value.status == -2


@pytest.mark.parametrize("reverse", [False, True])
def test_across_rows_in_slabs(pkg, cuda, oracle, reverse):
    """With scratch a scan across many rows of few columns is cut into runs of rows (totals, then a second sweep
    from the totals before each run): the same results as the sequential sweep, for every fold, a batch, a row
    count that does not divide, and BFloat16; and without need for scratch the entry says so (0 bytes)."""
    L = pkg.lib
    x = single(oracle.data(200, 3001))                       # 3001 rows of 200 columns
    assert L.scan_workspace_bytes(L.scan_desc(200, 3001, 0, across=True)) > 0
    assert L.scan_workspace_bytes(L.scan_desc(200, 3001, 0)) == 0          # along the rows: no use for it
    assert L.scan_workspace_bytes(L.scan_desc(200, 40, 0, across=True)) == 0   # too few rows to split
    for op in ("sum", "max", "min", "variance"):
        got, ref = run(pkg, cuda, x, op, across=True, reverse=reverse, slabs=True), want(oracle, x, op, across=True, reverse=reverse)
        if op in ("max", "min"):
            assert np.array_equal(got, ref)
        else:
            agree(got, ref, 1e-4)
    a = single(0.9 + 0.1 * oracle.data(96, 2000, scale=0.3))
    b = single(oracle.data(96, 2000, scale=0.7))
    agree(run(pkg, cuda, a, "affine", b, across=True, reverse=reverse, slabs=True),
          want(oracle, a, "affine", b, across=True, reverse=reverse), 1e-4)
    m = single(oracle.data(16, 900, 5))                      # a batch of five
    agree(run(pkg, cuda, m, "sum", across=True, reverse=reverse, slabs=True), want(oracle, m, "sum", across=True, reverse=reverse), 1e-4)
    h = oracle.to_bf16(single(0.05 * oracle.data(64, 1500)))
    got, ref = run(pkg, cuda, h, "sum", across=True, reverse=reverse, slabs=True), want(oracle, h, "sum", across=True, reverse=reverse)
    gf, rf = oracle.from_bf16(got).astype(np.float64), oracle.from_bf16(ref).astype(np.float64)
    assert (np.abs(gf - rf) <= 2.0 ** -7 * np.abs(rf) + 1e-3).all()
    # rows that are not whole groups of four columns take one column a thread; and a row count that leaves the
    # last slabs without rows (1024 slabs of 65 rows cover more than 65537)
    odd = single(oracle.data(203, 1500))
    agree(run(pkg, cuda, odd, "sum", across=True, reverse=reverse, slabs=True), want(oracle, odd, "sum", across=True, reverse=reverse), 1e-4)
    long = single(0.01 * oracle.data(8, 65537))
    assert np.array_equal(run(pkg, cuda, long, "max", across=True, reverse=reverse, slabs=True),
                          want(oracle, long, "max", across=True, reverse=reverse))
    # scratch that is too small is refused
    d = L.scan_desc(200, 3001, 0, across=True)
    xd = cuda.zeros(3001, 200, device="cuda")
    with pytest.raises(L.TB200Error) as e:
        L.scan(xd.data_ptr(), xd.data_ptr(), 200, 3001, 0, across=True, workspace=xd.data_ptr(), workspace_bytes=16)
    assert e.value.status == -5
