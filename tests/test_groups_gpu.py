"""Generic map -> fold row groups through the C ABI against the C oracle for groups (the reference's floor
over the same descriptor): the reference's programs spelled as terms, on the shapes its fold tests use
(test/cuda/folds.jl:16-25: 256x700, 9000x40, 100x3000, 512x300) and on ragged, tiny and long rows."""
import numpy as np
import pytest

from helpers import RTOL_F32

pytestmark = pytest.mark.gpu


def run_both(pkg, torch, oracle, group, inputs, wide=False, entry="generic"):
    """Returns (gpu outputs, oracle outputs) as numpy arrays (uint16 for BFloat16)."""
    L = pkg.lib
    d = group.desc()
    assert L.rowreduce_generic_check(d) == 0
    dev_in = [torch.from_numpy(np.ascontiguousarray(a).view(np.int16) if a.dtype == np.uint16 else np.ascontiguousarray(a)).cuda()
              for a in inputs]
    dev_out, ref_out = [], []
    for source, _, dtype, ld in group.outputs:
        shape = (group.rows, ld) if source == 0 else (group.rows,)
        host = np.zeros(shape, np.float32 if dtype == 0 else np.uint16)
        ref_out.append(host)
        dev_out.append(torch.zeros(shape, device="cuda", dtype=torch.float32 if dtype == 0 else torch.int16))
    run = L.rowreduce_generic if entry == "generic" else L.rowreduce_compiled
    run(d, [t.data_ptr() for t in dev_in], [t.data_ptr() for t in dev_out], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    oracle.group_eval(d, [np.ascontiguousarray(a) for a in inputs], ref_out, threads=8)
    got = [t.cpu().numpy().view(np.uint16) if t.dtype == torch.int16 else t.cpu().numpy() for t in dev_out]
    if not wide:
        return got, ref_out
    wide_out = [np.zeros_like(a) for a in ref_out]
    oracle.group_eval(d, [np.ascontiguousarray(a) for a in inputs], wide_out, threads=8, wide=True)
    return got, ref_out, wide_out


def agree(oracle, got, want, n, what="", wide=None):
    """Float32: within 1e-5 of the floor's result relative to the output's scale -- or, where the floor's own
    sequential Float32 sums have drifted further than that from the Float64 evaluation (long rows), no
    further from Float64 than twice the floor's distance."""
    if got.dtype == np.uint16:
        g, w = oracle.from_bf16(got).astype(np.float64), oracle.from_bf16(want).astype(np.float64)
        assert np.isfinite(g).all(), what
        assert np.abs(g - w).max() <= 2.0 ** -7 * np.abs(w).max() + 1e-30, what   # one BFloat16 step at the largest value
        assert (got != want).mean() <= 0.02, what                                  # and nearly all bits equal
    else:
        g, w = got.astype(np.float64), want.astype(np.float64)
        assert np.isfinite(g).all(), what
        scale = max(np.abs(w).max(), 1e-30)
        if np.abs(g - w).max() <= RTOL_F32 * scale:
            return
        assert wide is not None, (what, np.abs(g - w).max() / scale)
        w64 = wide.astype(np.float64)
        assert np.abs(g - w64).max() <= max(RTOL_F32 * scale, 2 * np.abs(w - w64).max()), what


SHAPES = [(256, 700), (9000, 40), (100, 3000), (512, 300), (1, 5), (3, 7), (4096, 64), (70001, 3), (33, 1000)]


ENTRIES = ["generic", "compiled"]   # the term interpreter; the group's own NVRTC-compiled kernel


@pytest.mark.parametrize("entry", ENTRIES)
@pytest.mark.parametrize("eltype", ["Float32", "BFloat16"])
@pytest.mark.parametrize("n,rows", SHAPES)
def test_programs_as_groups(pkg, cuda, oracle, n, rows, eltype, entry):
    G = pkg.groups
    cast = (lambda a: a) if eltype == "Float32" else oracle.to_bf16
    x = cast((oracle.normal((rows, n), n + rows) * 2).astype(np.float32))
    w = cast(oracle.normal((n,), n + 1))
    b = cast(oracle.normal((n,), n + 2))
    g2 = cast(oracle.normal((rows, n), n + 3))
    for name, group, inputs in (
        ("softmax", G.softmax(n, rows, eltype), [x]),
        ("log_softmax", G.log_softmax(n, rows, eltype), [x]),
        ("layernorm", G.layernorm(n, rows, eltype), [x, w, b]),
        ("layernorm two-pass", G.layernorm(n, rows, eltype, two_pass=True), [x, w, b]),
        ("rmsnorm", G.rmsnorm(n, rows, eltype), [x, w]),
        ("softmax pullback", G.softmax_pullback(n, rows, eltype), [x, g2]),
    ):
        got, want, wide = run_both(pkg, cuda, oracle, group, inputs, wide=True, entry=entry)
        for a, r, w64 in zip(got, want, wide):
            agree(oracle, a, r, n, f"{name} {n}x{rows} {eltype} {entry}", w64)


def test_against_the_named_kernels(pkg, cuda, oracle):
    """The generic softmax and LayerNorm against the library's own named entries on the same data."""
    torch, L, G = cuda, pkg.lib, pkg.groups
    n, rows = 4096, 300
    x = torch.randn(rows, n, device="cuda") * 3
    w, b = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    y_named, y_gen = torch.empty_like(x), torch.empty_like(x)
    lse_named, lse_gen = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    need = L.rowop_workspace_bytes(L.SOFTMAX_FWD, n, rows, L.F32)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    L.softmax_fwd(x.data_ptr(), y_named.data_ptr(), lse_named.data_ptr(), n, rows, n, L.F32, L.F32, ws.data_ptr(), need, stream)
    for run in (L.rowreduce_generic, L.rowreduce_compiled):
        y_gen.zero_()
        run(G.softmax(n, rows).desc(), [x.data_ptr()], [y_gen.data_ptr(), lse_gen.data_ptr()], stream)
        assert (y_named - y_gen).abs().max().item() <= 1e-5 * y_named.abs().max().item()
        assert (lse_named - lse_gen).abs().max().item() <= 1e-5 * lse_named.abs().max().item()
    need = L.rowop_workspace_bytes(L.LAYERNORM_FWD, n, rows, L.F32)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    L.layernorm_fwd(x.data_ptr(), w.data_ptr(), b.data_ptr(), y_named.data_ptr(), 0, 0, 1e-5, n, rows, n, L.F32,
                    ws.data_ptr(), need, stream)
    for run in (L.rowreduce_generic, L.rowreduce_compiled):
        y_gen.zero_()
        run(G.layernorm(n, rows).desc(), [x.data_ptr(), w.data_ptr(), b.data_ptr()], [y_gen.data_ptr()], stream)
        assert (y_named - y_gen).abs().max().item() <= 2e-5 * y_named.abs().max().item()


@pytest.mark.parametrize("entry", ENTRIES)
def test_strided_rows_statistics_and_saved_inputs(pkg, cuda, oracle, entry):
    """Rows at a pitch that is not a multiple of four (scalar accesses), four statistics in one sweep, and a
    per-row input: the softmax pullback from x and the saved log-sum-exp, y recomputed as exp(x - lse)."""
    G = pkg.groups
    n, rows, ld = 77, 50, 83
    x = np.zeros((rows, ld), np.float32)
    x[:, :n] = 1.0 + 0.02 * oracle.normal((rows, n), 61)
    g = G.Group(n, rows)
    xi = g.load(g.input("full", "Float32", ld=ld))
    for kind in ("max", "min", "sum", "prod"):
        g.output_stat(g.fold(kind, xi))
    got, want = run_both(pkg, cuda, oracle, g, [x], entry=entry)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    assert np.abs(got[2] - want[2]).max() <= 1e-5 * n
    assert np.abs(got[3] / want[3] - 1).max() <= 1e-5

    n, rows = 1000, 41
    xs = oracle.normal((rows, n), 62) * 2
    lse = oracle.softmax_fwd_f64(xs)[1].astype(np.float32)
    dy = oracle.normal((rows, n), 63)
    g = G.Group(n, rows)
    xi, li, di = g.load(g.input()), g.load(g.input("per_row")), g.load(g.input())
    y = g.exp(g.sub(xi, li))
    t = g.mul(di, y)
    s = g.fold("sum", t)
    g.output(g.sub(t, g.mul(y, g.stat(s))))
    got, want = run_both(pkg, cuda, oracle, g, [xs, lse, dy], entry=entry)
    agree(oracle, got[0], want[0], n, "pullback from saved lse")
    want64 = oracle.softmax_bwd_f64(oracle.softmax_fwd_f64(xs)[0], dy)
    assert np.abs(got[0] - want64).max() <= 2e-5 * np.abs(want64).max()


def test_empty_and_refused(pkg, cuda):
    L, G = pkg.lib, pkg.groups
    L.rowreduce_generic(G.softmax(0, 5).desc(), [0], [0, 0])       # nothing to do, nothing touched
    L.rowreduce_generic(G.softmax(5, 0).desc(), [0], [0, 0])
    for run in (L.rowreduce_generic, L.rowreduce_compiled):
        run(G.softmax(0, 5).desc(), [0], [0, 0])
        with pytest.raises(L.TB200Error) as e:
            run(G.softmax(8, 2).desc(), [0], [0, 0])
        assert e.value.status == -1


def test_through_the_generator(pkg, cuda, oracle):
    """claims -> build_claim -> launch() -> repoint -> launch(), the way Tempest's cover drives an Implementation."""
    torch, I, G = cuda, pkg.implement, pkg.groups
    n, rows = 515, 64
    g = G.rmsnorm(n, rows)
    gen, target = I.B200Generator(), I.Target()
    claims = gen.claims(target, g)
    assert [c.compiled for c in claims] == [True, False]
    x, w = torch.randn(rows, n, device="cuda"), torch.randn(n, device="cuda")
    want = np.zeros((rows, n), np.float32)
    oracle.group_eval(g.desc(), [x.cpu().numpy(), w.cpu().numpy()], [want])
    for claim in claims:
        y, y2 = torch.zeros_like(x), torch.zeros_like(x)
        launch, text = gen.build_claim(claim, target, g, {0: x, 1: w, 2: y})
        assert ("compiled" in text) == claim.compiled
        launch()
        launch.repoint(2, y2)()
        torch.cuda.synchronize()
        assert np.abs(y.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
        assert torch.equal(y, y2)


# ---- folds over the other axis ---------------------------------------------------------------------------

def run_columns(pkg, torch, oracle, group, inputs):
    L = pkg.lib
    d = group.desc()
    dev_in = [torch.from_numpy(np.ascontiguousarray(a).view(np.int16) if a.dtype == np.uint16 else np.ascontiguousarray(a)).cuda()
              for a in inputs]
    dev_out = [torch.zeros(group.n, device="cuda", dtype=torch.float32 if dtype == 0 else torch.int16)
               for _, _, dtype, _ in group.outputs]
    need = L.colreduce_workspace_bytes(d)
    ws = torch.empty(max(need, 16), device="cuda", dtype=torch.uint8)
    L.colreduce_compiled(d, [t.data_ptr() for t in dev_in], [t.data_ptr() for t in dev_out], ws.data_ptr(), need,
                         torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    got = [t.cpu().numpy().view(np.uint16) if t.dtype == torch.int16 else t.cpu().numpy() for t in dev_out]
    return got, oracle.group_eval_cols(d, inputs), oracle.group_eval_cols(d, inputs, wide=True)


def agree_columns(oracle, got, floor, wide, scale):
    """Float32 outputs: within 1e-5 of the Float64 evaluation relative to `scale` (the size of what was summed),
    or no further from it than twice the sequential Float32 floor is; BFloat16 outputs: one rounding on top."""
    for g, f, w in zip(got, floor, wide):
        if g.dtype == np.uint16:
            g, f, w = (oracle.from_bf16(a).astype(np.float64) for a in (g, f, w))
            assert (np.abs(g - w) <= 2.0 ** -7 * np.maximum(np.abs(w), scale * 1e-2) + 1e-30).all()
        else:
            g, f, w = (a.astype(np.float64) for a in (g, f, w))
            assert (np.abs(g - w) <= np.maximum(1e-5 * scale, 2.0 * np.abs(f - w)) + 1e-30).all()


@pytest.mark.parametrize("rows,n", [(700, 256), (40, 9000), (3000, 100), (300, 512), (1, 5), (4099, 33)])
@pytest.mark.parametrize("eltype", ["Float32", "BFloat16"])
def test_column_groups(pkg, cuda, oracle, rows, n, eltype):
    """The bias gradient, LayerNorm's weight gradients and per-column extrema against the oracle's sequential
    fold over the rows, on the transposes of the reference's fold shapes (test/cuda/folds.jl:16-25)."""
    G = pkg.groups
    cast = (lambda a: oracle.to_bf16(a)) if eltype == "BFloat16" else (lambda a: a)
    x, dy = oracle.normal((rows, n), 11 + n), oracle.normal((rows, n), 12 + n)
    mean = x.mean(axis=1).astype(np.float32)
    rstd = (1.0 / np.sqrt(x.var(axis=1) + 1e-5)).astype(np.float32)
    root = float(np.sqrt(rows))
    got, floor, wide = run_columns(pkg, cuda, oracle, G.bias_gradient(n, rows, eltype), [cast(dy)])
    agree_columns(oracle, got, floor, wide, root)
    got, floor, wide = run_columns(pkg, cuda, oracle, G.layernorm_weight_gradients(n, rows, eltype),
                                   [cast(x), cast(dy), mean, rstd])
    agree_columns(oracle, got, floor, wide, root)
    got, floor, wide = run_columns(pkg, cuda, oracle, G.column_extrema(n, rows, eltype), [cast(x)])
    assert np.array_equal(got[0], floor[0]) and np.array_equal(got[1], floor[1])   # extrema are exact
    agree_columns(oracle, got[2:], floor[2:], wide[2:], float(rows))


@pytest.mark.parametrize("rows,n", [(700, 256), (40, 9000), (3000, 100), (1, 5), (4099, 33)])
@pytest.mark.parametrize("eltype", ["Float32", "BFloat16"])
def test_relative_folds_over_the_rows(pkg, cuda, oracle, rows, n, eltype):
    """The log-sum-exp and the mean / variance states carried over the other axis (partial states per row slab,
    merged in a fixed order: ext/cuTileExt/emit.jl:729-753, build.jl:654-696) against the oracle's sequential fold
    over the rows and the Float64 closed forms, on the transposes of the reference's fold shapes."""
    G = pkg.groups
    x = (3.0 * oracle.normal((rows, n), 31 + n)).astype(np.float32)
    xin = oracle.to_bf16(x) if eltype == "BFloat16" else x
    xf = (oracle.from_bf16(xin) if eltype == "BFloat16" else x).astype(np.float64)
    got, floor, wide = run_columns(pkg, cuda, oracle, G.column_statistics(n, rows, eltype), [xin])
    m = xf.max(axis=0)
    lse = m + np.log(np.exp(xf - m).sum(axis=0))
    for g, want in zip(got, (lse, xf.mean(axis=0), xf.var(axis=0))):
        assert np.isfinite(g).all()
        assert np.abs(g - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    for g, w in zip(got, wide):
        assert np.abs(g.astype(np.float64) - w).max() <= 2e-5 * max(1.0, np.abs(w).max())
    # twice the same bits: slabs merge in a fixed order
    again, _, _ = run_columns(pkg, cuda, oracle, G.column_statistics(n, rows, eltype), [xin])
    assert all(np.array_equal(a, b) for a, b in zip(got, again))


def test_column_groups_agree_with_the_named_kernels(pkg, cuda, oracle):
    """dgamma and dbeta of the generated column group against the named LayerNorm backward on the same operands,
    and a group over no rows gives every fold's identity."""
    torch, L, G = cuda, pkg.lib, pkg.groups
    rows, n = 512, 1024
    x, dy, w = oracle.normal((rows, n), 1), oracle.normal((rows, n), 2), oracle.normal((n,), 3)
    y, mean, rstd = oracle.layernorm_fwd(x, w, np.zeros(n, np.float32))
    got, _, _ = run_columns(pkg, torch, oracle, G.layernorm_weight_gradients(n, rows), [x, dy, mean, rstd])
    _, dw, db = oracle.layernorm_bwd_f64(x, w, dy)
    assert np.abs(got[0] - dw).max() <= 1e-5 * np.sqrt(rows) * 4 and np.abs(got[1] - db).max() <= 1e-5 * np.sqrt(rows) * 4
    g = G.column_extrema(8, 0)
    d = g.desc()
    outs = [torch.zeros(8, device="cuda") for _ in range(3)]
    need = L.colreduce_workspace_bytes(d)
    ws = torch.empty(max(need, 16), device="cuda", dtype=torch.uint8)
    L.colreduce_compiled(d, [ws.data_ptr()], [o.data_ptr() for o in outs], ws.data_ptr(), need)
    torch.cuda.synchronize()
    assert torch.isinf(outs[0]).all() and (outs[0] < 0).all() and (outs[1] > 0).all() and (outs[2] == 0).all()
    with pytest.raises(L.TB200Error) as e:   # no workspace
        L.colreduce_compiled(G.bias_gradient(8, 4).desc(), [ws.data_ptr()], [outs[0].data_ptr()], 0, 0)
    assert e.value.status == -5


def test_column_group_through_the_generator(pkg, cuda, oracle):
    """A group marked `across` is claimed as a column group: two launches, scratch from the executable's
    resources, repointable like any other launch."""
    torch, I, G = cuda, pkg.implement, pkg.groups
    n, rows = 300, 1000
    g = G.bias_gradient(n, rows)
    gen, target = I.B200Generator(), I.Target()
    (claim,) = gen.claims(target, g)
    assert isinstance(claim, I.ColumnClaim)
    (work,) = gen.estimate(claim, target, g)
    assert work.launches == 2 and work.bytes == n * rows * 4 + n * 4
    x = torch.randn(rows, n, device="cuda")
    db, db2 = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    launch, text = gen.build_claim(claim, target, g, {0: x, 1: db})
    assert "columns" in text
    launch()
    launch.repoint(1, db2)()
    torch.cuda.synchronize()
    want = x.double().sum(dim=0)
    assert (db.double() - want).abs().max().item() <= 1e-5 * rows ** 0.5 * 4
    assert torch.equal(db, db2)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("heads,kv_heads,batch,S,D", [(2, 2, 1, 200, 128), (4, 2, 2, 133, 128), (3, 1, 3, 70, 32)])
def test_attention_group_through_the_generic_door(pkg, cuda, oracle, causal, heads, kv_heads, batch, S, D):
    """The attention group, spelled as terms (recomputed scores, the mask as a select on two positions, log-sum-exp,
    the weights' sum of the value rows), offered to the generator, claimed as attention and run: against the
    Float64 restatement of test/fixtures/operations.jl:21-76 (shapes of test/cuda/attention.jl:10-16)."""
    torch, I, G = cuda, pkg.implement, pkg.groups
    q = oracle.to_bf16(oracle.normal((batch, S, heads, D), 51))
    k = oracle.to_bf16(oracle.normal((batch, S, kv_heads, D), 52))
    v = oracle.to_bf16(oracle.normal((batch, S, kv_heads, D), 53))
    to = lambda a: torch.from_numpy(a).view(torch.bfloat16).cuda()   # noqa: E731
    qd, kd, vd = to(q), to(k), to(v)
    o = torch.full_like(qd, float("nan"))
    lse = torch.full((batch, S, heads), float("nan"), device="cuda")
    group = G.attention(S, S, D, causal)
    gen, target = I.B200Generator(), I.Target()
    (claim,) = gen.claims(target, group)
    assert isinstance(claim, I.AttentionClaim)
    launch, _ = gen.build_claim(claim, target, group, {"inputs": [qd, kd, vd], "outputs": [o, lse], "outer": (heads, kv_heads, batch)})
    launch()
    torch.cuda.synchronize()
    assert pkg.lib.attention_device_error() == 0
    o64, lse64 = oracle.attention_f64(q, k, v, causal)
    got = o.float().cpu().numpy()
    assert np.abs(got - o64).max() <= 2e-2
    assert np.abs(lse.cpu().numpy() - lse64).max() <= 1e-3
