"""Generic map -> fold row groups on the host: the descriptor builder, the checks the C entry makes
before any launch, and the C oracle for groups pinned on the named operators' oracles (which are pinned on
the reference's known answers) and on Float64 closed forms."""
import numpy as np
import pytest


def run_oracle(oracle, group, inputs, threads=2):
    d = group.desc()
    outs = []
    for source, _, dtype, _ in group.outputs:
        shape = (group.rows, group.n) if source == 0 else (group.rows,)
        outs.append(np.zeros(shape, np.float32 if dtype == 0 else np.uint16))
    oracle.group_eval(d, [np.ascontiguousarray(a) for a in inputs], outs, threads=threads)
    return outs


def test_softmax_group_is_the_named_oracle(pkg, oracle):
    G = pkg.groups
    n, rows = 300, 37
    x = oracle.normal((rows, n), 5) * 3
    y, lse = run_oracle(oracle, G.softmax(n, rows), [x])
    y_named, lse_named = oracle.softmax_fwd(x)
    assert np.abs(lse - lse_named).max() <= 1e-6 * np.abs(lse_named).max()
    assert np.abs(y - y_named).max() <= 1e-6
    y64, lse64 = oracle.softmax_fwd_f64(x)
    assert np.abs(y - y64).max() <= 1e-6 and np.abs(lse - lse64).max() <= 1e-5


def test_layernorm_group_both_spellings(pkg, oracle):
    G = pkg.groups
    n, rows = 700, 19
    x = (oracle.normal((rows, n), 6) * 2 + 5).astype(np.float32)
    w, b = oracle.normal((n,), 7), oracle.normal((n,), 8)
    want = oracle.layernorm_fwd_f64(x, w, b)
    named = oracle.layernorm_fwd(x, w, b)[0]
    for two_pass in (False, True):
        (y,) = run_oracle(oracle, G.layernorm(n, rows, two_pass=two_pass), [x, w, b])
        assert np.abs(y - want).max() <= 2e-5 * np.abs(want).max()
        assert np.abs(y - named).max() <= 2e-5 * np.abs(want).max()
    assert G.layernorm(n, rows, two_pass=True).desc().folds[1].phase == 1


def test_rmsnorm_pullback_extrema_and_bf16(pkg, oracle):
    G = pkg.groups
    n, rows = 129, 23
    x = oracle.normal((rows, n), 9)
    w = oracle.normal((n,), 10)
    (y,) = run_oracle(oracle, G.rmsnorm(n, rows), [x, w])
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.abs(y - want).max() <= 1e-5 * np.abs(want).max()
    yb = oracle.to_bf16(oracle.softmax_fwd_f64(x)[0].astype(np.float32))
    gb = oracle.to_bf16(oracle.normal((rows, n), 11))
    (dx,) = run_oracle(oracle, G.softmax_pullback(n, rows, "BFloat16"), [yb, gb])
    want = oracle.softmax_bwd_f64(oracle.from_bf16(yb), oracle.from_bf16(gb))
    assert np.abs(oracle.from_bf16(dx) - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6
    small = (1.0 + 0.01 * oracle.normal((rows, n), 12)).astype(np.float32)
    mx, mn, sm, pr = run_oracle(oracle, G.row_extrema(n, rows), [small])
    assert np.array_equal(mx, small.max(axis=1)) and np.array_equal(mn, small.min(axis=1))
    assert np.abs(sm - small.astype(np.float64).sum(axis=1)).max() <= 1e-5 * n
    assert np.abs(pr / np.prod(small.astype(np.float64), axis=1) - 1).max() <= 1e-5


def test_known_answer_sum_abs2(pkg, oracle):
    """compile(x -> sum(abs2, x))([1, 2, 3, 4]) == 30  (src/Compiler/runtime/compile.jl:36-39)."""
    g = pkg.groups.Group(4, 1)
    g.output_stat(g.fold("sum", g.abs2(g.load(g.input()))))
    (s,) = run_oracle(oracle, g, [np.array([[1, 2, 3, 4]], np.float32)], threads=1)
    assert s[0] == 30.0


def test_descriptor_checks(pkg):
    """tb200_rowreduce_generic_check runs on the host: what it refuses never reaches a launch."""
    G, L = pkg.groups, pkg.lib
    assert L.rowreduce_generic_check(G.softmax(4096, 65536).desc()) == 0
    assert L.rowreduce_generic_check(G.layernorm(128, 3, "BFloat16", two_pass=True).desc()) == 0
    d = G.softmax(16, 2).desc()
    d.terms[2].a = 7                      # an argument that comes after its use
    assert L.rowreduce_generic_check(d) == -2
    d = G.softmax(16, 2).desc()
    d.folds[0].phase = 1                  # the output sweep's statistic is fine, but ...
    d.terms[1].op, d.terms[1].a = 3, 0    # ... a fold that reads its own statistic is not
    d.folds[0].term = 1
    assert L.rowreduce_generic_check(d) == -2
    d = G.softmax(16, 2).desc()
    d.terms[0].op = 99
    assert L.rowreduce_generic_check(d) == -7
    d = G.softmax(16, 2).desc()
    d.inputs[0].ld = 8                    # rows overlap
    assert L.rowreduce_generic_check(d) == -2
    d = G.softmax(16, 2).desc()
    d.outputs[0].dtype = 5
    assert L.rowreduce_generic_check(d) == -3
    g = G.Group(8, 1)
    x = g.load(g.input())
    for _ in range(60):
        x = g.neg(x)
    g.output(x)
    with pytest.raises(ValueError):
        g.desc()


def test_generated_kernels_compile(pkg):
    """The generator's source for every spelling and schedule compiles for sm_100a (NVRTC needs no device):
    resident and streamed rows, whole and ragged chunks, vector and scalar accesses, both element types."""
    G, L = pkg.groups, pkg.lib
    if L.rowreduce_compile(G.softmax(64, 4).desc()) == -7 and "nvrtc" not in L.rowreduce_compile_log().lower():
        pytest.skip("NVRTC cannot be loaded here")
    for n in (5, 300, 4096, 70001):
        for eltype in ("Float32", "BFloat16"):
            for group in (G.softmax(n, 7, eltype), G.log_softmax(n, 7, eltype), G.layernorm(n, 7, eltype),
                          G.layernorm(n, 7, eltype, two_pass=True), G.rmsnorm(n, 7, eltype),
                          G.softmax_pullback(n, 7, eltype), G.row_extrema(n, 7, eltype)):
                for vectors in (0xff, 0):
                    assert L.rowreduce_compile(group.desc(), vectors, vectors) == 0, (n, eltype, L.rowreduce_compile_log())
    source = L.rowreduce_source(G.layernorm(4096, 65536).desc())
    assert "constexpr int N = 4096, V = 4, TPR = 256, K = 4" in source and "float c0[K][V];" in source   # resident
    assert "float c0[V];" in L.rowreduce_source(G.layernorm(70001, 3).desc())                             # streamed
    bad = G.softmax(16, 2).desc()
    bad.terms[0].op = 99
    assert L.rowreduce_compile(bad) == -7 and L.rowreduce_source(bad) == ""


def test_column_groups_compile_and_refusals(pkg, oracle):
    """Groups whose folds run over the rows: the descriptor compiles (NVRTC, no device), the source names both
    kernels, the oracle's evaluation of the bias gradient is the column sum, and what the form does not take
    is refused with a status."""
    G, L = pkg.groups, pkg.lib
    for make in (G.bias_gradient, G.layernorm_weight_gradients, G.column_extrema):
        for eltype in ("Float32", "BFloat16"):
            d = make(300, 77, eltype).desc()
            assert L.colreduce_workspace_bytes(d) >= 300 * 4
            L.colreduce_compile(d)
            src = L.colreduce_source(d)
            assert "tb200_cols(" in src and "tb200_cols_merge(" in src
    x = oracle.normal((77, 300), 5)
    (db,) = oracle.group_eval_cols(G.bias_gradient(300, 77).desc(), [x])
    assert np.allclose(db, x.astype(np.float64).sum(axis=0), rtol=0, atol=1e-4)
    # a fold along the row's own statistic, or a full-shaped output, is not a column group
    g = G.softmax(300, 77)
    with pytest.raises(L.TB200Error) as e:
        L.colreduce_compile(g.desc())
    assert e.value.status == -7
    # the relative folds run over the rows too (two- and three-word states), and the oracle folds them in sequence
    stats = G.column_statistics(300, 77)
    L.colreduce_compile(stats.desc())
    assert L.colreduce_workspace_bytes(stats.desc()) >= 5 * 300 * 4
    lse, mean, var = oracle.group_eval_cols(stats.desc(), [x])
    xf = x.astype(np.float64)
    assert np.allclose(lse, np.log(np.exp(xf).sum(axis=0)), atol=1e-4) and np.allclose(mean, xf.mean(axis=0), atol=1e-5)
    assert np.allclose(var, xf.var(axis=0), atol=1e-4)
    g = G.Group(300, 77, across=True)
    g.output_stat(g.fold("weighted", g.load(g.input("full"))))
    with pytest.raises(L.TB200Error) as e:
        L.colreduce_compile(g.desc())
    assert e.value.status == -7
    assert L.colreduce_workspace_bytes(g.desc()) == 0
