"""Chunked gated DeltaNet forward through the C ABI against the rule applied token by token in
Float64 -- the yardstick the reference's own example uses (examples/deltanet.jl:89-101, 112-124:
largest difference relative to the largest reference value)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run(pkg, torch, q, k, v, a, beta):
    L = pkg.lib
    Hn, T, dk = q.shape
    dv = v.shape[2]
    to = lambda x: torch.from_numpy(np.ascontiguousarray(x)).view(torch.bfloat16).cuda()  # noqa: E731
    qd, kd, vd = to(q), to(k), to(v)
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(beta).cuda()
    o = torch.full((Hn, dv, T), float("nan"), device="cuda", dtype=torch.bfloat16)
    desc = L.deltanet_desc(Hn, T, dk, dv)
    need = L.deltanet_workspace_bytes(desc)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    L.deltanet_fwd(desc, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ad.data_ptr(), bd.data_ptr(), o.data_ptr(),
                   ws.data_ptr(), need, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return o.float().cpu().numpy()


@pytest.mark.parametrize("heads,T", [(1, 64), (2, 256), (3, 1024), (2, 4096)])
def test_forward_against_the_token_rule(pkg, cuda, oracle, heads, T):
    q, k, v, a, beta = oracle.deltanet_inputs(heads, T, 128, 128, 100 + T)
    got = run(pkg, cuda, q, k, v, a, beta)
    want = oracle.deltanet_sequential(q, k, v, a, beta, threads=4)
    assert np.isfinite(got).all()
    rel = np.abs(got - want).max() / np.abs(want).max()
    assert rel <= 2e-2, rel                      # BFloat16 results against the Float64 rule
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)


def test_example_distribution(pkg, cuda, oracle):
    """The example's own inputs (examples/deltanet.jl:104-111): unit keys, gates in (0.88, 0.98)."""
    T, H, d = 1024, 2, 128
    w = lambda n, s: np.sin(s * np.arange(1, n + 1, dtype=np.float64))  # noqa: E731
    unit = lambda x: x / np.sqrt((x * x).sum(axis=-1, keepdims=True))   # noqa: E731
    # Julia (d, T, H) column-major filled from a vector = memory [H][T][d]
    q = unit(w(d * T * H, 0.37).reshape(H, T, d)) / np.sqrt(d)
    k = unit(w(d * T * H, 0.53).reshape(H, T, d))
    v = w(d * T * H, 0.71).reshape(H, T, d)
    a = (-0.05 * (1.5 + w(T * H, 0.13).reshape(H, T))).astype(np.float32)
    beta = (1.0 / (1.0 + np.exp(-w(T * H, 0.29).reshape(H, T)))).astype(np.float32)
    qb, kb, vb = (oracle.to_bf16(x.astype(np.float32)) for x in (q, k, v))
    got = run(pkg, cuda, qb, kb, vb, a, beta)
    want = oracle.deltanet_sequential(qb, kb, vb, a, beta, threads=2)
    assert np.abs(got - want).max() / np.abs(want).max() <= 2e-2


def run_bwd(pkg, torch, q, k, v, a, beta, dout_bits):
    L = pkg.lib
    Hn, T, dk = q.shape
    dv = v.shape[2]
    to = lambda x: torch.from_numpy(np.ascontiguousarray(x)).view(torch.bfloat16).cuda()  # noqa: E731
    qd, kd, vd, dod = to(q), to(k), to(v), to(dout_bits)
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(beta).cuda()
    nan = lambda *shape, dtype: torch.full(shape, float("nan"), device="cuda", dtype=dtype)  # noqa: E731
    dq, dk_, dv_ = (nan(Hn, T, n, dtype=torch.bfloat16) for n in (dk, dk, dv))
    da, db = nan(Hn, T, dtype=torch.float32), nan(Hn, T, dtype=torch.float32)
    desc = L.deltanet_desc(Hn, T, dk, dv)
    need = L.deltanet_bwd_workspace_bytes(desc)
    assert need > L.deltanet_workspace_bytes(desc)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    L.deltanet_bwd(desc, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ad.data_ptr(), bd.data_ptr(), dod.data_ptr(),
                   dq.data_ptr(), dk_.data_ptr(), dv_.data_ptr(), da.data_ptr(), db.data_ptr(), ws.data_ptr(), need,
                   torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return [x.float().cpu().numpy().astype(np.float64) for x in (dq, dk_, dv_, da, db)]


@pytest.mark.parametrize("heads,T", [(1, 64), (2, 192), (1, 512)])
def test_pullback_against_the_token_rule(pkg, cuda, oracle, heads, T):
    """BFloat16 gradients against the Float64 pullback of the token rule: largest difference relative
    to the largest reference value, the example's yardstick (examples/deltanet.jl:112-124)."""
    q, k, v, a, beta = oracle.deltanet_inputs(heads, T, 128, 128, 300 + T)
    dout_bits = oracle.to_bf16(oracle.normal((heads, 128, T), 299 + T))
    dout = oracle.from_bf16(dout_bits).astype(np.float64)
    got = run_bwd(pkg, cuda, q, k, v, a, beta, dout_bits)
    want = oracle.deltanet_sequential_bwd(q, k, v, a, beta, dout)
    for name, g, w in zip(("dq", "dk", "dv", "da", "dbeta"), got, want):
        assert np.isfinite(g).all(), name
        rel = np.abs(g - w).max() / np.abs(w).max()
        assert rel <= 2e-2, (name, rel)
        assert np.linalg.norm(g - w) <= 1e-2 * np.linalg.norm(w), name


def test_pullback_is_linear_in_the_cotangent(pkg, cuda, oracle):
    """At a size the oracle cannot reach: the pullback of (d1 + d2) equals the sum of the pullbacks, and
    a zero cotangent gives zero gradients."""
    heads, T = 2, 2048
    q, k, v, a, beta = oracle.deltanet_inputs(heads, T, 128, 128, 900)
    d1 = oracle.from_bf16(oracle.to_bf16(oracle.normal((heads, 128, T), 901)))
    d2 = oracle.from_bf16(oracle.to_bf16(oracle.normal((heads, 128, T), 902)))
    both = oracle.to_bf16((d1 + d2).astype(np.float32))
    ga = run_bwd(pkg, cuda, q, k, v, a, beta, oracle.to_bf16(d1))
    gb = run_bwd(pkg, cuda, q, k, v, a, beta, oracle.to_bf16(d2))
    gs = run_bwd(pkg, cuda, q, k, v, a, beta, both)
    for x, y, z in zip(ga, gb, gs):
        assert np.abs(x + y - z).max() <= 3e-2 * np.abs(z).max()
    for g in run_bwd(pkg, cuda, q, k, v, a, beta, np.zeros((heads, 128, T), np.uint16)):
        assert (g == 0).all()


def test_config_length_against_the_token_rule(pkg, cuda, oracle):
    """The benchmark's sequence length, T = 8192 (128 chained chunks): forward of two sequences and the
    pullback of one against the Float64 token rule."""
    heads, T = 2, 8192
    q, k, v, a, beta = oracle.deltanet_inputs(heads, T, 128, 128, 8192)
    got = run(pkg, cuda, q, k, v, a, beta)
    want = oracle.deltanet_sequential(q, k, v, a, beta, threads=2)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)
    one = slice(0, 1)
    dout_bits = oracle.to_bf16(oracle.normal((1, 128, T), 8193))
    dout = oracle.from_bf16(dout_bits).astype(np.float64)
    grads = run_bwd(pkg, cuda, q[one], k[one], v[one], a[one], beta[one], dout_bits)
    wants = oracle.deltanet_sequential_bwd(q[one], k[one], v[one], a[one], beta[one], dout)
    for name, g, w in zip(("dq", "dk", "dv", "da", "dbeta"), grads, wants):
        assert np.isfinite(g).all(), name
        rel = np.abs(g - w).max() / np.abs(w).max()
        assert rel <= 2e-2, (name, rel)
        assert np.linalg.norm(g - w) <= 1e-2 * np.linalg.norm(w), name


def test_config_launch_of_64_sequences(pkg, cuda, oracle):
    """The whole benchmark launch (B * H = 64 sequences of 8192, forward and pullback): every result finite,
    and two sampled sequences bit-equal to the same sequences run alone (sequences are independent, and
    the kernels' order of summation does not depend on how many there are)."""
    torch, L = cuda, pkg.lib
    Hn, T = 64, 8192
    g = torch.Generator(device="cuda").manual_seed(64)
    unit = lambda x: torch.nn.functional.normalize(x, dim=-1)   # noqa: E731
    q = unit(torch.randn(Hn, T, 128, device="cuda", generator=g)).bfloat16()
    k = unit(torch.randn(Hn, T, 128, device="cuda", generator=g)).bfloat16()
    v = torch.randn(Hn, T, 128, device="cuda", generator=g).bfloat16()
    a = -torch.nn.functional.softplus(torch.randn(Hn, T, device="cuda", generator=g))
    beta = torch.sigmoid(torch.randn(Hn, T, device="cuda", generator=g))
    dout = torch.randn(Hn, 128, T, device="cuda", generator=g).bfloat16()
    stream = torch.cuda.current_stream().cuda_stream

    def both(sel):
        qs, ks, vs, as_, bs, ds = (x[sel].contiguous() for x in (q, k, v, a, beta, dout))
        n = qs.shape[0]
        desc = L.deltanet_desc(n, T)
        o = torch.full((n, 128, T), float("nan"), device="cuda", dtype=torch.bfloat16)
        need = L.deltanet_workspace_bytes(desc)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        L.deltanet_fwd(desc, qs.data_ptr(), ks.data_ptr(), vs.data_ptr(), as_.data_ptr(), bs.data_ptr(), o.data_ptr(),
                       ws.data_ptr(), need, stream)
        del ws
        dq, dk, dv = (torch.full((n, T, 128), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(3))
        da, db = (torch.full((n, T), float("nan"), device="cuda") for _ in range(2))
        need = L.deltanet_bwd_workspace_bytes(desc)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        L.deltanet_bwd(desc, qs.data_ptr(), ks.data_ptr(), vs.data_ptr(), as_.data_ptr(), bs.data_ptr(), ds.data_ptr(),
                       dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), da.data_ptr(), db.data_ptr(), ws.data_ptr(), need, stream)
        torch.cuda.synchronize()
        return o, dq, dk, dv, da, db

    whole = both(slice(0, Hn))
    for t in whole:
        assert torch.isfinite(t.float()).all()
    for h in (5, 63):
        alone = both(slice(h, h + 1))
        for w, s in zip(whole, alone):
            assert torch.equal(w[h], s[0])


def test_bounded_waits_report_nothing(pkg, cuda):
    """The scans wait for their tiles on mbarriers, with a limit; after every launch of this file none has given up."""
    assert pkg.lib.deltanet_device_error() == 0


def test_refuses_other_geometries(pkg, cuda):
    L = pkg.lib
    x = cuda.zeros(64, device="cuda")
    for desc in (L.deltanet_desc(1, 100), L.deltanet_desc(1, 128, dk=64), L.deltanet_desc(1, 128, chunk=32)):
        with pytest.raises(L.TB200Error) as e:
            L.deltanet_fwd(desc, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                           x.data_ptr(), 1 << 20)
        assert e.value.status == -7


def test_pullback_refuses_what_it_cannot_run(pkg, cuda):
    L = pkg.lib
    x = cuda.zeros(1 << 16, device="cuda")
    p = x.data_ptr()
    args = [p] * 11
    with pytest.raises(L.TB200Error) as e:   # other geometries
        L.deltanet_bwd(L.deltanet_desc(1, 128, dk=64), *args, p, 1 << 30)
    assert e.value.status == -7
    d = L.deltanet_desc(1, 128)
    need = L.deltanet_bwd_workspace_bytes(d)
    assert need == L.deltanet_workspace_bytes(d) + 128 * 1920   # what the launches hand each other, BFloat16
    with pytest.raises(L.TB200Error) as e:   # a workspace that is too small
        L.deltanet_bwd(d, *args, p, need - 1)
    assert e.value.status == -5
    with pytest.raises(L.TB200Error) as e:   # a missing gradient array
        L.deltanet_bwd(d, *([p] * 10), 0, p, need)
    assert e.value.status == -1
    L.deltanet_bwd(L.deltanet_desc(0, 128), *args, 0, 0)   # nothing to do
