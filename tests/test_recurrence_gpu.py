"""Recurrences whose step is a map, through the C ABI against the oracle's step-by-step evaluation: the reference's
recurrence programs that are maps (test/runtime/recurrences.jl:14-15, 190-196), Float32 and BFloat16, reversed, ragged
extents, padded rows.  Tolerance: the reference's own for recurrences on the GPU, rtol 1e-4
(test/runtime/recurrences.jl:467-469): tanh and exp differ by units in the last place between the device and numpy,
and a recurrence carries the difference along."""
import numpy as np
import pytest

from helpers import agree

pytestmark = pytest.mark.gpu


def run(pkg, torch, oracle, group, inputs):
    L = pkg.lib
    d = group.desc()
    devs, keep = [], []
    for i, a in enumerate(inputs):
        a = np.ascontiguousarray(a)
        t = torch.from_numpy(a).cuda()
        keep.append(t)
        devs.append(t.data_ptr())
    outs = []
    for o in range(d.body.n_outputs):
        shape = (group.rows, group.n) if d.body.outputs[o].source == 0 else (group.n,)
        dt = torch.float32 if d.body.outputs[o].dtype == L.F32 else torch.int16
        outs.append(torch.full(shape, -7, device="cuda", dtype=dt))
    L.recurrence_compiled(d, devs, [t.data_ptr() for t in outs])
    torch.cuda.synchronize()
    got = [t.cpu().numpy() if t.dtype == torch.float32 else t.cpu().numpy().view(np.uint16) for t in outs]
    return got, oracle.recurrence_eval(d, inputs)


@pytest.mark.parametrize("n,steps", [(300, 64), (1000, 7), (33, 500), (4096, 128), (1, 1)])
@pytest.mark.parametrize("reverse", [False, True])
def test_gated_cell(pkg, cuda, oracle, n, steps, reverse):
    G = pkg.groups
    x = oracle.normal((steps, n), 10 + n)
    a = (0.5 + 0.4 * np.tanh(oracle.normal((n,), 11))).astype(np.float32)
    h0 = oracle.normal((n,), 12)
    got, want = run(pkg, cuda, oracle, G.gated_tanh_cell(n, steps, reverse=reverse), [x, a, h0])
    for g, w in zip(got, want):
        agree(g, w, 1e-4)


def test_states_assigned_at_once_and_scalar_starts(pkg, cuda, oracle):
    G = pkg.groups
    n, steps = 257, 90
    x = oracle.normal((steps, n), 20)
    got, want = run(pkg, cuda, oracle, G.second_order(n, steps), [x, np.zeros(n, np.float32), np.ones(n, np.float32)])
    for g, w in zip(got, want):
        agree(g, w, 1e-4)
    got, want = run(pkg, cuda, oracle, G.decayed_sum(n, steps), [x, np.array([2.0], np.float32)])
    agree(got[0], want[0], 1e-5)


def test_bfloat16_and_padded_rows(pkg, cuda, oracle):
    G, L = pkg.groups, pkg.lib
    n, steps = 200, 48
    x = oracle.to_bf16(oracle.normal((steps, n), 30))
    a = oracle.to_bf16((0.5 + 0.3 * np.tanh(oracle.normal((n,), 31))).astype(np.float32))
    h0 = oracle.to_bf16(oracle.normal((n,), 32))
    got, want = run(pkg, cuda, oracle, G.gated_tanh_cell(n, steps, "BFloat16"), [x, a, h0])
    for g, w in zip(got, want):
        gf, wf = oracle.from_bf16(g).astype(np.float64), oracle.from_bf16(w).astype(np.float64)
        # results are rounded to BFloat16 and carried: a unit in the last place where the roundings part
        assert (np.abs(gf - wf) <= 2.0 ** -7 * np.abs(wf) + 2e-3).all()
    # rows at a pitch larger than n: the pads are neither read nor written
    torch = cuda
    ld = n + 24
    g = G.Recurrence(n, steps)
    xin, s0 = g.input("full", ld=ld), g.input("scalar")
    s = g.state(s0)
    new = g.fma(g.carried(s), g.lit(0.9), g.load(xin))
    g.carry(s, new)
    g.output(new, ld=ld)
    xf = oracle.normal((steps, ld), 33)
    xd = torch.from_numpy(xf).cuda()
    zero = torch.zeros(1, device="cuda")
    y = torch.full((steps, ld), -7.0, device="cuda")
    L.recurrence_compiled(g.desc(), [xd.data_ptr(), zero.data_ptr()], [y.data_ptr()])
    torch.cuda.synchronize()
    yh = y.cpu().numpy()
    assert (yh[:, n:] == -7.0).all()
    want = np.zeros(n, np.float64)
    for k in range(steps):
        want = 0.9 * want + xf[k, :n]
    assert np.abs(yh[-1, :n] - want).max() <= 1e-4


def test_through_the_plugin_mirror(pkg, cuda, oracle):
    """claims -> estimate -> build_claim -> launch -> repoint, as the reference drives an Implementation
    (src/Compiler/Implement/Implement.jl:229-262) for a `:recurrence` group."""
    torch, G, I = cuda, pkg.groups, pkg.implement
    n, steps = 500, 33
    group = G.gated_tanh_cell(n, steps)
    gen, target = I.B200Generator(), I.Target()
    (claim,) = gen.claims(target, group)
    assert isinstance(claim, I.RecurrenceClaim) and claim.states == 1
    (work,) = gen.estimate(claim, target, group)
    assert work.bytes == 4 * (2 * n * steps + 3 * n) and work.launches == 1
    x = oracle.normal((steps, n), 40)
    a = np.full(n, 0.8, np.float32)
    h0 = oracle.normal((n,), 41)
    dev = [torch.from_numpy(v).cuda() for v in (x, a, h0)]
    hs, last = torch.empty(steps, n, device="cuda"), torch.empty(n, device="cuda")
    launch, note = gen.build_claim(claim, target, group, {"inputs": dev, "outputs": [hs, last]})
    assert "recurrence" in note
    launch()
    torch.cuda.synchronize()
    want = oracle.recurrence_eval(group.desc(), [x, a, h0])
    agree(hs.cpu().numpy(), want[0], 1e-4)
    agree(last.cpu().numpy(), want[1], 1e-4)
    x2 = oracle.normal((steps, n), 42)
    launch.repoint(0, torch.from_numpy(x2).cuda())()
    torch.cuda.synchronize()
    agree(hs.cpu().numpy(), oracle.recurrence_eval(group.desc(), [x2, a, h0])[0], 1e-4)


def test_no_steps_leaves_the_start(pkg, cuda, oracle):
    G = pkg.groups
    n = 70
    h0 = oracle.normal((n,), 50)
    got, want = run(pkg, cuda, oracle, G.gated_tanh_cell(n, 0), [np.zeros((0, n), np.float32), np.ones(n, np.float32), h0])
    assert got[0].shape == (0, n) and np.array_equal(got[1], h0) and np.array_equal(want[1], h0)


def test_refusals(pkg, cuda):
    G, L = pkg.groups, pkg.lib
    d = G.gated_tanh_cell(16, 4).desc()
    x = cuda.zeros(64, device="cuda")
    with pytest.raises(L.TB200Error) as e:
        L.recurrence_compiled(d, [x.data_ptr(), 0, x.data_ptr()], [x.data_ptr(), x.data_ptr()])
    assert e.value.status == -1
    d.body.outputs[0].ld = 8                       # rows overlap
    with pytest.raises(L.TB200Error) as e:
        L.recurrence_compiled(d, [x.data_ptr()] * 3, [x.data_ptr()] * 2)
    assert e.value.status == -2
