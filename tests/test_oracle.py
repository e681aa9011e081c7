"""The CPU oracle against the reference's known-answer literals and against
Float64 closed forms (runs without a GPU)."""
import numpy as np
import pytest

from helpers import agree


def test_sum_abs2_known_answer(oracle):
    # compile(x -> sum(abs2, x))([1, 2, 3, 4]) == 30.0   (src/Compiler/runtime/compile.jl:36-39)
    assert oracle.sum_abs2_f32(np.array([1, 2, 3, 4], np.float32)) == 30.0


def test_contract_known_answer(oracle):
    # contract([1 2; 3 4], [5 6; 7 8], (1,2), (2,3), (1,3)) == [19 22; 43 50]   (program/tracing.jl:872-875)
    # Julia column-major [1 2;3 4] is memory 1,3,2,4: as row-major [K][M] that is A read "a_km".
    A = np.array([[1, 3], [2, 4]], np.float32).T.copy()  # row-major [M][K]
    B = np.array([[5, 6], [7, 8]], np.float32)           # row-major [K][N]
    C = oracle.gemm(A, B, M=2, N=2, K=2)
    assert (C == np.array([[19, 22], [43, 50]], np.float32)).all()


def test_bf16_sum_accumulates_in_float32(oracle):
    # 4096 BFloat16 gradients of 0.01 at one position sum to 41, not 4   (test/codegen/floor.jl:28-32)
    h = oracle.to_bf16(np.full(4096, 0.01, np.float32))
    total = oracle.from_bf16(np.array([oracle.sum_bf16(h)], np.uint16))[0]
    assert total == 41.0


def test_bf16_round_to_nearest_even(oracle):
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, np.inf, 0.0], np.float32)
    back = oracle.from_bf16(oracle.to_bf16(x))
    # 1 + 2^-8 is a tie between 1 and 1 + 2^-7: to even (1.0); 1 + 3*2^-8 ties to 1 + 2^-6
    assert back[0] == 1.0 and back[1] == 1.0 and back[2] == 1.015625 and back[3] == -2.5
    assert np.isinf(back[5]) and back[6] == 0.0


def test_logsumexp_fold_edge_cases(oracle):
    # an empty or all -Inf slice sums to zero; +Inf gives +Inf   (src/Compiler/IR/folds.jl:121-127)
    assert oracle.logsumexp_f32(np.array([], np.float32)) == -np.inf
    assert oracle.logsumexp_f32(np.array([-np.inf, -np.inf], np.float32)) == -np.inf
    assert oracle.logsumexp_f32(np.array([1.0, np.inf], np.float32)) == np.inf
    assert abs(oracle.logsumexp_f32(np.array([0.0, 0.0], np.float32)) - np.log(2.0)) < 1e-7


def test_welford_fold(oracle):
    x = oracle.data(300, scale=0.37).astype(np.float32).ravel()
    m, v = oracle.mean_var_f32(x)
    assert abs(m - x.astype(np.float64).mean()) < 1e-6
    assert abs(v - x.astype(np.float64).var()) < 1e-5


def test_data_generator(oracle):
    # data(dims...; scale) = 2 sin(scale * k)   (test/setup.jl:33): a Julia (3, 2) array's memory
    d = oracle.data(3, 2, scale=0.5)
    assert d.shape == (2, 3)
    assert np.allclose(d.ravel(), 2 * np.sin(0.5 * np.arange(1, 7)))


# the reduced-axis lengths and column counts of the reference's fold tests
# (test/cuda/folds.jl:16-25) and a few ragged ones
SHAPES = [(700, 256), (40, 9000), (300, 512), (5, 1), (3, 133), (17, 70)]


@pytest.mark.parametrize("rows,n", SHAPES)
def test_softmax_against_float64(oracle, rows, n):
    x = oracle.data(n, rows, scale=0.3).astype(np.float32)
    g = oracle.data(n, rows, scale=0.7).astype(np.float32)
    y, lse = oracle.softmax_fwd(x)
    y64, lse64 = oracle.softmax_fwd_f64(x)
    agree(y, y64, 1e-5)
    agree(lse, lse64, 1e-5)
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-4)
    agree(oracle.softmax_bwd(y, g), oracle.softmax_bwd_f64(y, g), 1e-5)


@pytest.mark.parametrize("rows,n", SHAPES)
def test_layernorm_against_float64(oracle, rows, n):
    x = oracle.data(n, rows, scale=0.3).astype(np.float32)
    g = oracle.data(n, rows, scale=0.7).astype(np.float32)
    w = oracle.data(n, scale=0.1).astype(np.float32).ravel()
    b = oracle.data(n, scale=0.2).astype(np.float32).ravel()
    y, mean, rstd = oracle.layernorm_fwd(x, w, b)
    agree(y, oracle.layernorm_fwd_f64(x, w, b), 2e-5)
    dx, dw, db = oracle.layernorm_bwd(x, w, g)
    dx64, dw64, db64 = oracle.layernorm_bwd_f64(x, w, g)
    agree(dx, dx64, 5e-5)
    agree(dw, dw64, 5e-5)
    agree(db, db64, 5e-5)


def test_bf16_paths(oracle):
    x = oracle.to_bf16(oracle.normal((33, 256), 5))
    y_faithful, _ = oracle.softmax_fwd(x, faithful=True)
    y_f32, _ = oracle.softmax_fwd(x, faithful=False)
    y64, _ = oracle.softmax_fwd_f64(oracle.from_bf16(x))
    assert np.abs(oracle.from_bf16(y_f32) - y64).max() < 2e-3
    # per-operation rounding drifts further than one final rounding, but stays close
    assert np.abs(oracle.from_bf16(y_faithful) - y64).max() < 2e-2


def test_threads_change_nothing(oracle):
    x = oracle.normal((64, 512), 3)
    a, la = oracle.softmax_fwd(x, threads=1)
    b, lb = oracle.softmax_fwd(x, threads=4)
    assert (a == b).all() and (la == lb).all()


def test_readme_loss_gradient(oracle):
    # loss(w, b, x) = sum(abs2, tanh.(w' * x .+ b)), w 32x64, b 64, x 32x16   (README.md:15)
    w = oracle.normal((64, 32), 1)
    b = oracle.normal((64,), 2)
    x = oracle.normal((16, 32), 3)
    loss, dw, db, dx = oracle.readme_loss_grad(w, b, x)
    z = x.astype(np.float64) @ w.astype(np.float64).T + b
    y = np.tanh(z)
    assert abs(loss - (y ** 2).sum()) / (y ** 2).sum() < 1e-5
    gz = 2 * y * (1 - y ** 2)
    agree(dw, gz.T @ x.astype(np.float64), 1e-5)
    agree(db, gz.sum(axis=0), 1e-5)
    agree(dx, gz @ w.astype(np.float64), 1e-5)
    # and a central difference on one weight
    eps = 1e-3
    wp, wm = w.copy(), w.copy()
    wp[5, 7] += eps
    wm[5, 7] -= eps
    fd = (oracle.readme_loss_grad(wp, b, x)[0] - oracle.readme_loss_grad(wm, b, x)[0]) / (2 * eps)
    assert abs(fd - dw[5, 7]) < 5e-2 * max(1.0, abs(dw[5, 7]))


def test_deltanet_pullback_against_autograd_and_differences(oracle):
    """The hand-written reverse accumulation against torch's Float64 autograd of the same rule and
    against a central difference of the C oracle's forward in one direction."""
    import torch
    H, T, d = 2, 48, 16
    q, k, v, a, beta = oracle.deltanet_inputs(H, T, d, d, 77)
    dout = oracle.normal((H, d, T), 78).astype(np.float64)
    got = oracle.deltanet_sequential_bwd(q, k, v, a, beta, dout)
    leaves = [torch.tensor(oracle.from_bf16(x).astype(np.float64), requires_grad=True) for x in (q, k, v)]
    leaves += [torch.tensor(x.astype(np.float64), requires_grad=True) for x in (a, beta)]
    tq, tk, tv, ta, tb = leaves
    total = 0.0
    for h in range(H):
        S = torch.zeros(d, d, dtype=torch.float64)
        for t in range(T):
            kt = tk[h, t]
            S = torch.exp(ta[h, t]) * (S - tb[h, t] * torch.outer(kt, kt @ S)) + tb[h, t] * torch.outer(kt, tv[h, t])
            total = total + ((S.T @ tq[h, t]) * torch.tensor(dout[h, :, t])).sum()
    total.backward()
    for mine, leaf in zip(got, leaves):
        want = leaf.grad.numpy()
        assert np.abs(mine - want).max() <= 1e-10 * max(1.0, np.abs(want).max())
    # central difference along one direction of the gates, through the C forward
    da = oracle.normal((H, T), 79).astype(np.float32) * np.float32(2.0 ** -10)
    up = oracle.deltanet_sequential(q, k, v, a + da, beta)
    dn = oracle.deltanet_sequential(q, k, v, a - da, beta)
    step = ((a + da).astype(np.float64) - (a - da).astype(np.float64))
    assert abs(((up - dn) * dout).sum() - (got[3] * step).sum()) <= 1e-4 * abs((got[3] * step).sum()) + 1e-9


def test_mlp_step_by_blas_equals_the_sequential_restatement(oracle):
    """The BLAS form used at the benchmark's size takes the same step as the sequential restatement (only the
    order of summation differs)."""
    sizes, batch, rate = (24, 40, 32, 8), 16, 1e-2
    ws = [oracle.to_bf16(0.3 * oracle.normal((sizes[i], sizes[i + 1]), 80 + i)) for i in range(3)]
    bs = [oracle.to_bf16(0.1 * oracle.normal((sizes[i + 1],), 90 + i)) for i in range(3)]
    x = oracle.to_bf16(oracle.normal((batch, sizes[0]), 95))
    y = oracle.to_bf16(oracle.normal((batch, sizes[-1]), 96))
    seq = oracle.mlp_step(ws, bs, x, y, rate)
    fast = oracle.mlp_step_blas(ws, bs, x, y, rate)
    assert abs(seq[0] - fast[0]) <= 1e-5 * abs(seq[0])
    for i in range(3):
        assert np.abs(oracle.from_bf16(seq[1][i]) - oracle.from_bf16(fast[1][i])).max() <= 2e-3   # dz, one ulp apart at most
        assert np.linalg.norm(seq[2][i] - fast[2][i]) <= 1e-2 * np.linalg.norm(seq[2][i])       # dw (from dz a BFloat16 ulp apart)
        assert np.abs(seq[3][i] - fast[3][i]).max() <= 1e-2 * max(1.0, np.abs(seq[3][i]).max())
        for k, j in ((4, i), (5, i), (6, i + 1), (7, i)):   # updated w and b, the activations, what the activation saw
            assert np.abs(oracle.from_bf16(seq[k][j]) - oracle.from_bf16(fast[k][j])).max() <= 2e-2


def test_generic_fold_recurrence_known_answer(oracle):
    # accumulate(recurrence, [(0.5, 1.0), (0.5, 1.0), (0.5, 1.0)]) == [1.0, 1.5, 1.75] with
    # combine((a1, b1), (a2, b2)) = (a2 a1, a2 b1 + b2), observe = last   (src/Compiler/IR/folds.jl:279-288)
    a = np.full((1, 3), 0.5, np.float32)
    b = np.ones((1, 3), np.float32)
    assert oracle.scan(a, "affine", b).ravel().tolist() == [1.0, 1.5, 1.75]
    assert oracle.scan(a.T.copy(), "affine", b.T.copy(), across=True).ravel().tolist() == [1.0, 1.5, 1.75]


def test_scans_against_numpy(oracle):
    x = oracle.data(40, 7, scale=0.37).astype(np.float32)          # [7][40]
    assert np.allclose(oracle.scan(x, "sum"), np.cumsum(x.astype(np.float64), axis=1), rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle.scan(x, "sum", across=True), np.cumsum(x.astype(np.float64), axis=0), rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle.scan(x, "max", reverse=True), np.maximum.accumulate(x[:, ::-1], axis=1)[:, ::-1])
    assert np.allclose(oracle.scan(1 + 0.01 * x, "prod"), np.cumprod(1 + 0.01 * x.astype(np.float64), axis=1), rtol=1e-5)
    var = np.array([[x[r, : i + 1].astype(np.float64).var() for i in range(40)] for r in range(7)])
    assert np.allclose(oracle.scan(x, "variance"), var, rtol=1e-4, atol=1e-5)


def test_updated_state_and_its_sum_known_answer(oracle):
    # f!(s, x) = (s .= 0.5 .* s .+ x; sum(s)) with s = [1, 2], x = [1, 1] gives (3.5, [1.5, 2.0])
    # (docs/src/compiling.md:23-29): the update is the affine step h = a h + b per element, the value a plain sum
    # written as two-element scans, one per entry of s: the first step loads s (a = 0, b = s), the second is the update
    a = np.array([[0.0, 0.5], [0.0, 0.5]], np.float32)
    b = np.array([[1.0, 1.0], [2.0, 1.0]], np.float32)
    new = oracle.scan(a, "affine", b)[:, 1]
    assert new.tolist() == [1.5, 2.0] and oracle.sum_f32(new) == 3.5
