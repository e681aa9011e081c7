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


def test_refuses_other_geometries(pkg, cuda):
    L = pkg.lib
    x = cuda.zeros(64, device="cuda")
    for desc in (L.deltanet_desc(1, 100), L.deltanet_desc(1, 128, dk=64), L.deltanet_desc(1, 128, chunk=32)):
        with pytest.raises(L.TB200Error) as e:
            L.deltanet_fwd(desc, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                           x.data_ptr(), 1 << 20)
        assert e.value.status == -7
