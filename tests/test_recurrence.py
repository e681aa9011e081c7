"""Recurrences whose step is a map: the descriptor builder, the checks the C entry makes before any launch, the
generated source (NVRTC needs no device), and the oracle's step-by-step evaluation pinned on closed forms and on the
scan oracle (an affine recurrence is a scan)."""
import numpy as np
import pytest


def test_oracle_against_closed_forms(pkg, oracle):
    G = pkg.groups
    n, steps = 5, 40
    x = oracle.normal((steps, n), 3)
    # s = 0.5 s + x^2 from a scalar start: the closed form sum_k 0.5^(T-1-k) x_k^2 + 0.5^T s0
    (last,) = oracle.recurrence_eval(G.decayed_sum(n, steps).desc(), [x, np.array([2.0], np.float32)])
    x64 = x.astype(np.float64)
    want = sum(0.5 ** (steps - 1 - k) * x64[k] ** 2 for k in range(steps)) + 0.5 ** steps * 2.0
    assert np.abs(last - want).max() <= 1e-5 * np.abs(want).max()
    # the affine recurrence h = a h + b is the scan oracle's (itself pinned on the reference's literal [1.0, 1.5, 1.75])
    g = G.Recurrence(n, steps)
    a_in, b_in, h0 = g.input("full"), g.input("full"), g.input("scalar")
    h = g.state(h0)
    new = g.fma(g.load(a_in), g.carried(h), g.load(b_in))
    g.carry(h, new)
    g.output(new)
    a = (0.9 + 0.1 * oracle.normal((steps, n), 4)).astype(np.float32)
    (hs,) = oracle.recurrence_eval(g.desc(), [a, x, np.zeros(1, np.float32)])
    assert np.abs(hs - oracle.scan(a, "affine", x, True, False)).max() <= 1e-5
    # two states assigned at once: the second lags the first by one step
    ys, y_last, lag_last = oracle.recurrence_eval(G.second_order(n, steps).desc(),
                                                  [x, np.zeros(n, np.float32), np.ones(n, np.float32)])
    assert np.array_equal(y_last, ys[-1]) and np.array_equal(lag_last, ys[-2])
    y, last2 = np.zeros(n), np.ones(n)
    for k in range(steps):
        y, last2 = np.tanh(1.5 * y - 0.5 * last2 + x64[k]), y
    assert np.abs(ys[-1] - y).max() <= 1e-5
    # reversed: the same as the forward recurrence over the rows flipped
    fwd = oracle.recurrence_eval(G.gated_tanh_cell(n, steps).desc(), [x[::-1].copy(), np.full(n, 0.7, np.float32), np.zeros(n, np.float32)])
    rev = oracle.recurrence_eval(G.gated_tanh_cell(n, steps, reverse=True).desc(), [x, np.full(n, 0.7, np.float32), np.zeros(n, np.float32)])
    assert np.array_equal(rev[0], fwd[0][::-1]) and np.array_equal(rev[1], fwd[1])


def test_descriptor_checks_and_source(pkg):
    G, L = pkg.groups, pkg.lib
    d = G.gated_tanh_cell(300, 50).desc()
    source = L.recurrence_source(d)
    assert "tb200_recurrence" in source and "st0 = t" in source and "tanhf" in source
    if L.load().tb200_recurrence_compile(d) == -7 and "nvrtc" not in L.rowreduce_compile_log().lower():
        pytest.skip("NVRTC cannot be loaded here")
    for make in (G.gated_tanh_cell, G.second_order, G.decayed_sum):
        for eltype in ("Float32", "BFloat16"):
            L.recurrence_compile(make(77, 9, eltype).desc())
    L.recurrence_compile(G.gated_tanh_cell(64, 8, reverse=True).desc())
    bad = G.gated_tanh_cell(16, 4).desc()
    bad.states[0].next = 99
    assert L.load().tb200_recurrence_compile(bad) == -2 and L.recurrence_source(bad) == ""
    bad = G.gated_tanh_cell(16, 4).desc()
    bad.states[0].start = 0                    # a state cannot start from a full-shaped input
    assert L.load().tb200_recurrence_compile(bad) == -2
    bad = G.gated_tanh_cell(16, 4).desc()
    bad.body.terms[0].op = 3                   # a statistic of a fold: a recurrence has none
    assert L.load().tb200_recurrence_compile(bad) == -7
    bad = G.gated_tanh_cell(16, 4).desc()
    bad.n_states = 0
    assert L.load().tb200_recurrence_compile(bad) == -2
    with pytest.raises(ValueError):
        g = G.Recurrence(8, 2)
        g.state(g.input("along"))
        g.desc()                               # a state that is never carried
