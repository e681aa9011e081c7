"""Attention through the C ABI against the CPU oracle (the reference's attention program restated,
test/fixtures/operations.jl:21-76): causal and not, grouped heads, sequence lengths that are not a
multiple of the tile (the reference's own geometries use 70, 133, 200 positions,
test/cuda/attention.jl:10-16), and the benchmark geometry on its 1/8 sub-batch against sampled
oracle rows and a plain Float32 PyTorch restatement."""
import numpy as np
import pytest

from helpers import ATOL_BF16, RTOL_F32

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16).cuda()


def host(torch, t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def run_fwd(pkg, torch, q, k, v, causal, want_lse=True):
    L = pkg.lib
    B, S, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    qd, kd, vd = dev(torch, q), dev(torch, k), dev(torch, v)
    o = torch.full_like(qd, float("nan"))
    lse = torch.full((B, S, H), float("nan"), device="cuda") if want_lse else None
    desc = L.attn_desc(B, H, S, Skv, D, causal, kv_heads=Hkv)
    L.attention_fwd(desc, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr() if want_lse else 0,
                    torch.cuda.current_stream().cuda_stream)
    assert L.attention_device_error() == 0
    return host(torch, o), (lse.cpu().numpy() if want_lse else None)


# (batch, heads, kv_heads, positions)
GEOMETRIES = [(1, 2, 2, 128), (1, 2, 1, 256), (2, 3, 3, 200), (1, 1, 1, 70), (1, 4, 2, 384), (1, 2, 2, 133), (2, 2, 2, 640)]


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,H,Hkv,S", GEOMETRIES)
def test_forward_against_oracle(pkg, cuda, oracle, B, H, Hkv, S, causal):
    D = 128
    q = oracle.to_bf16(oracle.normal((B, S, H, D), 1 + S))
    k = oracle.to_bf16(oracle.normal((B, S, Hkv, D), 2 + S))
    v = oracle.to_bf16(oracle.normal((B, S, Hkv, D), 3 + S))
    o, lse = run_fwd(pkg, cuda, q, k, v, causal)
    # the Float32 CPU reference (weights kept in Float32) and the variant that rounds the weights as the GPU does
    o_ref, lse_ref = oracle.attention_fwd(q, k, v, causal, threads=8)
    err = np.abs(oracle.from_bf16(o) - oracle.from_bf16(o_ref)).max()
    assert err <= ATOL_BF16, err
    assert np.abs(lse - lse_ref).max() <= 2e-5 * max(1.0, np.abs(lse_ref).max())
    o64, lse64 = oracle.attention_f64(q, k, v, causal)
    assert np.abs(oracle.from_bf16(o) - o64).max() <= ATOL_BF16
    assert np.abs(lse - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())


def test_forward_without_lse_and_peaked_scores(pkg, cuda, oracle):
    """No log-sum-exp requested; and scores whose maximum keeps growing along the keys, which is what
    makes the kernel rescale its accumulator."""
    B, S, H, D = 1, 512, 2, 128
    q = oracle.normal((B, S, H, D), 11)
    k = oracle.normal((B, S, H, D), 12)
    k = k * (1.0 + np.arange(S, dtype=np.float32)[None, :, None, None] / 64.0)   # later keys score higher
    v = oracle.normal((B, S, H, D), 13)
    qb, kb, vb = (oracle.to_bf16(a) for a in (q, k, v))
    o, _ = run_fwd(pkg, cuda, qb, kb, vb, False, want_lse=False)
    o64, _ = oracle.attention_f64(qb, kb, vb, False)
    assert np.abs(oracle.from_bf16(o) - o64).max() <= ATOL_BF16
    o, lse = run_fwd(pkg, cuda, qb, kb, vb, True)
    o64, lse64 = oracle.attention_f64(qb, kb, vb, True)
    assert np.abs(oracle.from_bf16(o) - o64).max() <= ATOL_BF16
    assert np.abs(lse - lse64).max() <= 2e-5 * np.abs(lse64).max()


def test_forward_refuses_what_it_does_not_compute(pkg, cuda):
    L, torch = pkg.lib, cuda
    x = torch.zeros(1, 128, 2, 512, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(L.TB200Error) as e:   # head dimensions over 256
        L.attention_fwd(L.attn_desc(1, 2, 128, 128, 512, True), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr())
    assert e.value.status == -7
    with pytest.raises(L.TB200Error) as e:   # causal needs as many queries as keys (operations.jl:40-41)
        L.attention_fwd(L.attn_desc(1, 2, 128, 256, 128, True), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr())
    assert e.value.status == -2


# (head dimension, heads, kv heads, positions, batch): the reference's own geometries
# (test/cuda/attention.jl:10-16) and a few more head dimensions, all on the CUDA-core path
OTHER_DIMS = [(16, 2, 2, 200, 2), (16, 4, 2, 200, 2), (32, 3, 1, 70, 3), (8, 1, 1, 133, 1), (64, 4, 2, 256, 1),
              (40, 2, 1, 97, 1), (256, 2, 2, 160, 1)]


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D,H,Hkv,S,B", OTHER_DIMS)
def test_other_head_dimensions(pkg, cuda, oracle, D, H, Hkv, S, B, causal):
    q = oracle.to_bf16(oracle.normal((B, S, H, D), 41 + S))
    k = oracle.to_bf16(oracle.normal((B, S, Hkv, D), 42 + S))
    v = oracle.to_bf16(oracle.normal((B, S, Hkv, D), 43 + S))
    g = oracle.to_bf16(oracle.normal((B, S, H, D), 44 + S))
    dq, dk, dv, o, lse = run_bwd(pkg, cuda, q, k, v, g, causal)
    o64, lse64, dq64, dk64, dv64 = oracle.attention_f64(q, k, v, causal, dout=g)
    assert np.abs(oracle.from_bf16(o) - o64).max() <= ATOL_BF16
    assert np.abs(lse - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())
    o_ref, lse_ref = oracle.attention_fwd(q, k, v, causal, threads=4)
    assert np.abs(oracle.from_bf16(o) - oracle.from_bf16(o_ref)).max() <= ATOL_BF16
    assert np.abs(lse - lse_ref).max() <= 2e-5 * max(1.0, np.abs(lse_ref).max())
    close_grad(oracle, dq, dq64, "dq")
    close_grad(oracle, dk, dk64, "dk")
    close_grad(oracle, dv, dv64, "dv")


def test_more_keys_than_queries(pkg, cuda, oracle):
    """Cross attention (not causal): 70 queries over 333 keys, head dimension 32."""
    B, Sq, Sk, H, D = 2, 70, 333, 2, 32
    q = oracle.to_bf16(oracle.normal((B, Sq, H, D), 51))
    k = oracle.to_bf16(oracle.normal((B, Sk, H, D), 52))
    v = oracle.to_bf16(oracle.normal((B, Sk, H, D), 53))
    o, lse = run_fwd(pkg, cuda, q, k, v, False)
    o64, lse64 = oracle.attention_f64(q, k, v, False)
    assert np.abs(oracle.from_bf16(o) - o64).max() <= ATOL_BF16
    assert np.abs(lse - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())


def doc_starts(lengths):
    """0-based start of each position's document (test/cuda/attention.jl:232, 1-based there)."""
    out, at = [], 0
    for n in lengths:
        out += [at] * n
        at += n
    return np.array(out, np.int32)


@pytest.mark.parametrize("D", [16, 128])
def test_packed_documents(pkg, cuda, oracle, D):
    """The reference's packed-documents program (test/cuda/attention.jl:217-246): 300 positions, 2 heads, 2
    sequences of documents [90, 1, 130, 40, 39] and [7, 200, 93]; then one document a sequence and one a
    position; forward and pullback."""
    torch, L = cuda, pkg.lib
    B, S, H = 2, 300, 2
    q, k, v, g = (oracle.to_bf16(oracle.normal((B, S, H, D), 61 + i)) for i in range(4))
    qd, kd, vd, gd = (dev(torch, a) for a in (q, k, v, g))
    desc = L.attn_desc(B, H, S, S, D, True, scale=0.25)
    for start in (np.stack([doc_starts([90, 1, 130, 40, 39]), doc_starts([7, 200, 93])]),
                  np.zeros((B, S), np.int32), np.tile(np.arange(S, dtype=np.int32), (B, 1))):
        sd = torch.from_numpy(start).cuda()
        mask = L.attn_mask(doc_start=sd.data_ptr())
        o, lse = torch.full_like(qd, float("nan")), torch.full((B, S, H), float("nan"), device="cuda")
        dq, dk, dv = (torch.full_like(t, float("nan")) for t in (qd, kd, vd))
        L.attention_fwd_masked(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr())
        L.attention_bwd_masked(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                               gd.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr())
        torch.cuda.synchronize()
        o64, lse64, dq64, dk64, dv64 = oracle.attention_f64(q, k, v, True, scale=0.25, dout=g, doc_start=start)
        assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16
        assert np.abs(lse.cpu().numpy() - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())
        close_grad(oracle, host(torch, dq), dq64, "dq")
        close_grad(oracle, host(torch, dk), dk64, "dk")
        close_grad(oracle, host(torch, dv), dv64, "dv")


@pytest.mark.parametrize("D", [16, 128])
def test_decode_up_to_lengths(pkg, cuda, oracle, D):
    """The reference's decode program (test/cuda/attention.jl:248-275): one query per head, 8 query heads over
    2 key heads, a cache (features, positions, key heads, sequences) of 200 positions read up to a length the
    device holds; another set of lengths is the same launch.  128 features: the tensor-core kernel."""
    torch, L = cuda, pkg.lib
    B, H, Hkv, N = 3, 8, 2, 200
    q = oracle.to_bf16(oracle.normal((B, 1, H, D), 71))
    kc = oracle.to_bf16(oracle.normal((B, Hkv, N, D), 72))     # the cache's memory order
    vc = oracle.to_bf16(oracle.normal((B, Hkv, N, D), 73))
    qd, kd, vd = dev(torch, q), dev(torch, kc), dev(torch, vc)
    desc = L.attn_desc(B, H, 1, N, D, False, scale=0.25, kv_heads=Hkv)
    k_std, v_std = kc.transpose(0, 2, 1, 3), vc.transpose(0, 2, 1, 3)   # [B][N][Hkv][D] for the yardstick
    for lengths in ([37, 200, 1], [200, 5, 64]):
        ld = torch.tensor(lengths, dtype=torch.int32, device="cuda")
        mask = L.attn_mask(kv_len=ld.data_ptr(), kv_stride=(Hkv * N * D, D, N * D))
        o, lse = torch.full_like(qd, float("nan")), torch.full((B, 1, H), float("nan"), device="cuda")
        L.attention_fwd_masked(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr())
        torch.cuda.synchronize()
        o64, lse64 = oracle.attention_f64(q, k_std, v_std, False, scale=0.25, kv_len=np.array(lengths))
        assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16
        assert np.abs(lse.cpu().numpy() - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())
    # a length of zero: nothing to attend to
    ld = torch.tensor([0, 3, 0], dtype=torch.int32, device="cuda")
    mask = L.attn_mask(kv_len=ld.data_ptr(), kv_stride=(Hkv * N * D, D, N * D))
    o, lse = torch.full_like(qd, float("nan")), torch.full((B, 1, H), float("nan"), device="cuda")
    L.attention_fwd_masked(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr())
    assert (o[0] == 0).all() and torch.isinf(lse[0]).all() and torch.isfinite(lse[1]).all()


def test_masks_on_the_tensor_core_forward(pkg, cuda, oracle):
    """128 features: the masked forward runs on the tensor cores.  Documents longer and shorter than a tile of 128
    (whole key tiles before a document's start are skipped, the tile the start falls in is masked row by row);
    starts that are not sorted (every tile's range is found from all its queries' starts); lengths over several key
    tiles with grouped heads and more keys than queries; the pair of outputs agrees with the CUDA-core kernels'."""
    torch, L = cuda, pkg.lib
    D = 128
    B, S, H = 2, 1000, 2
    q, k, v = (oracle.to_bf16(oracle.normal((B, S, H, D), 81 + i)) for i in range(3))
    qd, kd, vd = (dev(torch, a) for a in (q, k, v))
    desc = L.attn_desc(B, H, S, S, D, True, scale=0.1)
    rng = np.random.default_rng(5)
    unsorted = np.minimum(rng.integers(0, S, (B, S)), np.arange(S)[None, :]).astype(np.int32)
    for start in (np.stack([doc_starts([300, 500, 200]), doc_starts([129, 1, 126, 744])]), unsorted):
        sd = torch.from_numpy(start).cuda()
        mask = L.attn_mask(doc_start=sd.data_ptr())
        o, lse = torch.full_like(qd, float("nan")), torch.full((B, S, H), float("nan"), device="cuda")
        L.attention_fwd_masked(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr())
        torch.cuda.synchronize()
        assert L.attention_device_error() == 0
        o64, lse64 = oracle.attention_f64(q, k, v, True, scale=0.1, doc_start=start)
        assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16
        assert np.abs(lse.cpu().numpy() - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())
    # lengths: 200 queries against up to 700 keys, 4 query heads over 2 key heads, one sequence with no key at all
    Bq, M, N, Hq, Hkv = 3, 200, 700, 4, 2
    q = oracle.to_bf16(oracle.normal((Bq, M, Hq, D), 91))
    k, v = (oracle.to_bf16(oracle.normal((Bq, N, Hkv, D), 92 + i)) for i in range(2))
    qd, kd, vd = (dev(torch, a) for a in (q, k, v))
    lengths = [513, 0, 90]
    ld = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    desc = L.attn_desc(Bq, Hq, M, N, D, False, scale=0.1, kv_heads=Hkv)
    o, lse = torch.full_like(qd, float("nan")), torch.full((Bq, M, Hq), float("nan"), device="cuda")
    L.attention_fwd_masked(desc, L.attn_mask(kv_len=ld.data_ptr()), qd.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                           o.data_ptr(), lse.data_ptr())
    torch.cuda.synchronize()
    assert L.attention_device_error() == 0
    o64, lse64 = oracle.attention_f64(q, k, v, False, scale=0.1, kv_len=np.array(lengths))
    assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16
    assert (o[1] == 0).all() and torch.isinf(lse[1]).all()
    fin = np.isfinite(lse64)
    assert np.abs(lse.cpu().numpy()[fin] - lse64[fin]).max() <= 2e-5 * max(1.0, np.abs(lse64[fin]).max())


@pytest.mark.parametrize("deterministic", [0, 1])
def test_masked_pullback_on_the_tensor_cores(pkg, cuda, oracle, deterministic):
    """128 features: packed documents (sorted starts, and starts that are not), then lengths with grouped heads and
    more keys than queries (one sequence with no key: zero gradients), forward and pullback on the tensor cores, both
    forms of the pullback, against the Float64 yardstick."""
    torch, L = cuda, pkg.lib
    D = 128
    B, S, H = 2, 300, 2
    q, k, v, g = (oracle.to_bf16(oracle.normal((B, S, H, D), 101 + i)) for i in range(4))
    qd, kd, vd, gd = (dev(torch, a) for a in (q, k, v, g))
    desc = L.attn_desc(B, H, S, S, D, True, scale=0.1, deterministic=deterministic)
    need = L.attention_bwd_masked_workspace_bytes(desc)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    rng = np.random.default_rng(6)
    unsorted = np.minimum(rng.integers(0, S, (B, S)), np.arange(S)[None, :]).astype(np.int32)
    for start in (np.stack([doc_starts([90, 1, 130, 40, 39]), doc_starts([7, 200, 93])]), unsorted):
        sd = torch.from_numpy(start).cuda()
        mask = L.attn_mask(doc_start=sd.data_ptr())
        o, lse = torch.full_like(qd, float("nan")), torch.full((B, S, H), float("nan"), device="cuda")
        dq, dk, dv = (torch.full_like(t, float("nan")) for t in (qd, kd, vd))
        L.attention_fwd_masked(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr())
        L.attention_bwd_masked_ws(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                  gd.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need)
        torch.cuda.synchronize()
        assert L.attention_bwd_device_error() == 0
        o64, lse64, dq64, dk64, dv64 = oracle.attention_f64(q, k, v, True, scale=0.1, dout=g, doc_start=start)
        close_grad(oracle, host(torch, dq), dq64, "dq")
        close_grad(oracle, host(torch, dk), dk64, "dk")
        close_grad(oracle, host(torch, dv), dv64, "dv")
    Bq, M, N, Hq, Hkv = 3, 200, 700, 4, 2
    q, g = (oracle.to_bf16(oracle.normal((Bq, M, Hq, D), 111 + i)) for i in range(2))
    k, v = (oracle.to_bf16(oracle.normal((Bq, N, Hkv, D), 113 + i)) for i in range(2))
    qd, kd, vd, gd = (dev(torch, a) for a in (q, k, v, g))
    lengths = [513, 0, 90]
    ld = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    mask = L.attn_mask(kv_len=ld.data_ptr())
    desc = L.attn_desc(Bq, Hq, M, N, D, False, scale=0.1, kv_heads=Hkv, deterministic=deterministic)
    need = L.attention_bwd_masked_workspace_bytes(desc)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    o, lse = torch.full_like(qd, float("nan")), torch.full((Bq, M, Hq), float("nan"), device="cuda")
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (qd, kd, vd))
    L.attention_fwd_masked(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr())
    L.attention_bwd_masked_ws(desc, mask, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                              gd.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need)
    torch.cuda.synchronize()
    assert L.attention_bwd_device_error() == 0
    o64, lse64, dq64, dk64, dv64 = oracle.attention_f64(q, k, v, False, scale=0.1, dout=g, kv_len=np.array(lengths))
    close_grad(oracle, host(torch, dq), dq64, "dq")
    close_grad(oracle, host(torch, dk), dk64, "dk")
    close_grad(oracle, host(torch, dv), dv64, "dv")
    assert (dq[1] == 0).all() and (dk[1] == 0).all() and (dv[1] == 0).all()
    # strides the tensor-core path does not take: refused, the CUDA-core entry remains
    with pytest.raises(L.TB200Error) as e:
        L.attention_bwd_masked_ws(desc, L.attn_mask(kv_len=ld.data_ptr(), kv_stride=(Hkv * N * D, D, N * D)), qd.data_ptr(),
                                  kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), gd.data_ptr(), dq.data_ptr(),
                                  dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need)
    assert e.value.status == -7


@pytest.mark.parametrize("dqk,dv", [(24, 16), (16, 24), (128, 64), (192, 128)])
def test_values_with_features_of_their_own(pkg, cuda, oracle, dqk, dv):
    """Values with other features than the queries and keys, as multi-head latent attention's (the reference's
    test/cuda/attention.jl:150-177: (24, 16) and (16, 24), 2 heads, 70 positions, 2 sequences, causal; here also
    128-feature keys with 64-feature values, and 192 with 128): forward and pullback, each gradient over its own
    features, against the Float64 yardstick; grouped heads in the last case."""
    torch, L = cuda, pkg.lib
    B, S, H = 2, 70, 2
    Hkv = 1 if dqk == 192 else H
    q = oracle.to_bf16(0.5 * oracle.normal((B, S, H, dqk), 121))
    k = oracle.to_bf16(0.5 * oracle.normal((B, S, Hkv, dqk), 122))
    v = oracle.to_bf16(oracle.normal((B, S, Hkv, dv), 123))
    g = oracle.to_bf16(oracle.normal((B, S, H, dv), 124))
    qd, kd, vd, gd = (dev(torch, a) for a in (q, k, v, g))
    desc = L.attn_desc(B, H, S, S, dqk, True, scale=0.25, kv_heads=Hkv, value_dim=dv)
    o, lse = torch.full((B, S, H, dv), float("nan"), device="cuda", dtype=torch.bfloat16), torch.full((B, S, H), float("nan"), device="cuda")
    L.attention_fwd(desc, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr())
    need = L.attention_bwd_workspace_bytes(desc)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    dq, dk, dvv = torch.full_like(qd, float("nan")), torch.full_like(kd, float("nan")), torch.full_like(vd, float("nan"))
    L.attention_bwd(desc, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), gd.data_ptr(),
                    dq.data_ptr(), dk.data_ptr(), dvv.data_ptr(), ws.data_ptr(), need)
    torch.cuda.synchronize()
    o64, lse64, dq64, dk64, dv64 = oracle.attention_f64(q, k, v, True, scale=0.25, dout=g)
    assert o64.shape == (B, S, H, dv) and dv64.shape == (B, S, Hkv, dv)
    assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16
    assert np.abs(lse.cpu().numpy() - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())
    close_grad(oracle, host(torch, dq), dq64, "dq")
    close_grad(oracle, host(torch, dk), dk64, "dk")
    close_grad(oracle, host(torch, dvv), dv64, "dv")
    # the masked entries take them as dense arrays only
    with pytest.raises(L.TB200Error) as e:
        L.attention_fwd_masked(desc, L.attn_mask(kv_stride=(Hkv * S * dqk, dqk, S * dqk)), qd.data_ptr(), kd.data_ptr(),
                               vd.data_ptr(), o.data_ptr(), lse.data_ptr())
    assert e.value.status == -7


def test_masked_attention_through_the_plugin_mirror(pkg, cuda, oracle):
    """Binding -> supports -> build -> launch for packed documents, forward with its log-sum-exp and the pullback
    (tensor cores at 128 features, scratch from the executable's resources), and a decode-like forward with lengths."""
    torch, I = cuda, pkg.implement
    lib, target = I.B200Kernels(), I.Target()
    D, H, S, B = 128, 2, 300, 2
    q, k, v, g = (oracle.to_bf16(oracle.normal((B, S, H, D), 131 + i)) for i in range(4))
    qd, kd, vd, gd = (dev(torch, a) for a in (q, k, v, g))
    start = np.stack([doc_starts([90, 1, 130, 40, 39]), doc_starts([7, 200, 93])])
    sd = torch.from_numpy(start).cuda()
    o, lse = torch.empty_like(qd), torch.empty(B, S, H, device="cuda")
    dq, dk, dv = (torch.empty_like(qd) for _ in range(3))
    e = {"d": D, "h": H, "hk": H, "m": S, "n": S, "b": B, "one": 1}
    heads = lambda t, val: I.dense_heads(t, "BFloat16", D, H, S, B, val)  # noqa: E731
    arrays = {"q": heads(qd, 1), "k": heads(kd, 2), "v": heads(vd, 3), "o": heads(o, 4),
              "lse": I.Strided("Float32", 0, (1, H, S, B), (1, 1, H, H * S), lse, 5),
              "start": I.Strided("Int32", 0, (S, B), (1, S), sd, 6)}
    fwd = I.Binding("attention_causal_documents_lse", e, arrays)
    assert lib.supports(target, fwd)
    launch, note = lib.build(target, fwd)
    assert "packed documents" in note
    launch()
    res = I.Resources()
    bwd = I.Binding("attention_causal_documents_pullback", e, dict(arrays, g=heads(gd, 7), dq=heads(dq, 8), dk=heads(dk, 9),
                                                                  dv=heads(dv, 10)))
    assert lib.supports(target, bwd)
    launch, _ = lib.build(target, bwd, res)
    assert launch.workspace is not None and res.bytes >= pkg.lib.attention_bwd_masked_workspace_bytes(launch.desc)
    launch()
    torch.cuda.synchronize()
    assert pkg.lib.attention_device_error() == 0 and pkg.lib.attention_bwd_device_error() == 0
    o64, lse64, dq64, dk64, dv64 = oracle.attention_f64(q, k, v, True, dout=g, doc_start=start)
    assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16
    assert np.abs(lse.cpu().numpy() - lse64).max() <= 2e-5 * max(1.0, np.abs(lse64).max())
    close_grad(oracle, host(torch, dq), dq64, "dq")
    close_grad(oracle, host(torch, dk), dk64, "dk")
    close_grad(oracle, host(torch, dv), dv64, "dv")
    lengths = torch.tensor([17, 300], dtype=torch.int32, device="cuda")
    dec = I.Binding("attention_lengths", e, {"q": heads(qd, 1), "k": heads(kd, 2), "v": heads(vd, 3), "o": heads(o, 4),
                                             "lengths": I.dense_vector(lengths, "Int32", B, 11)})
    assert lib.supports(target, dec)
    launch, _ = lib.build(target, dec)
    launch()
    torch.cuda.synchronize()
    o64, _ = oracle.attention_f64(q, k, v, False, kv_len=np.array([17, 300]))
    assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16


def test_masked_entries_refuse_bad_requests(pkg, cuda):
    L, torch = pkg.lib, cuda
    x = torch.zeros(4096, device="cuda", dtype=torch.bfloat16)
    p = x.data_ptr()
    mask = L.attn_mask()
    with pytest.raises(L.TB200Error) as e:
        L.attention_fwd_masked(L.attn_desc(1, 2, 8, 8, 512, False), mask, p, p, p, p)
    assert e.value.status == -7
    with pytest.raises(L.TB200Error) as e:
        L.attention_fwd_masked(L.attn_desc(1, 2, 8, 8, 16, False), mask, p, 0, p, p)
    assert e.value.status == -1
    with pytest.raises(L.TB200Error) as e:   # causal needs as many queries as keys
        L.attention_fwd_masked(L.attn_desc(1, 2, 8, 16, 16, True), mask, p, p, p, p)
    assert e.value.status == -2
    with pytest.raises(L.TB200Error) as e:
        L.attention_bwd_masked(L.attn_desc(1, 2, 8, 8, 16, False), mask, p, p, p, p, 0, p, p, p, p)
    assert e.value.status == -1
    L.attention_fwd_masked(L.attn_desc(0, 2, 8, 8, 16, False), mask, 0, 0, 0, 0)   # an empty batch


def torch_reference(torch, q, k, v, causal, dout=None):
    """Plain Float32 PyTorch restatement on the device, one head at a time."""
    B, S, H, D = q.shape
    qf, kf, vf = q.float().requires_grad_(dout is not None), k.float().requires_grad_(dout is not None), \
        v.float().requires_grad_(dout is not None)
    s = torch.einsum("bmhd,bnhd->bhmn", qf, kf) * (D ** -0.5)
    if causal:
        mask = torch.ones(S, S, device="cuda", dtype=torch.bool).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("bhmn,bnhd->bmhd", torch.exp(s - lse[..., None]), vf)
    if dout is None:
        return o, lse.permute(0, 2, 1)
    o.backward(dout.float())
    return o.detach(), lse.permute(0, 2, 1).detach(), qf.grad, kf.grad, vf.grad


def test_forward_benchmark_geometry(pkg, cuda, oracle):
    """B=8, H=32, S=4096, D=128 causal on its 1/8 sub-batch: sampled query rows against the oracle, and
    4 heads in full against the Float32 restatement."""
    torch, L = cuda, pkg.lib
    torch.backends.cuda.matmul.allow_tf32 = False
    B, S, H, D = 1, 4096, 32, 128
    g = torch.Generator(device="cuda").manual_seed(20261125 + 4)
    q, k, v = (torch.randn(B, S, H, D, device="cuda", generator=g).bfloat16() for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty(B, S, H, device="cuda")
    L.attention_fwd(L.attn_desc(B, H, S, S, D, True), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                    lse.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert L.attention_device_error() == 0
    qh, kh, vh = host(torch, q), host(torch, k), host(torch, v)
    fn = oracle.load().oracle_attention_fwd_rows
    o_ref = np.zeros_like(qh)
    lse_ref = np.zeros((B, S, H), np.float32)
    import ctypes
    rows = [(0, 4), (1000, 1003), (2047, 2050), (4092, 4096)]
    for h in (0, 13, 31):
        for m0, m1 in rows:
            fn(oracle._ptr(qh), oracle._ptr(kh), oracle._ptr(vh), oracle._ptr(o_ref), oracle._ptr(lse_ref),
               ctypes.c_int(B), ctypes.c_int(H), ctypes.c_int(H), ctypes.c_int(S), ctypes.c_int(S), ctypes.c_int(D),
               ctypes.c_int(1), ctypes.c_float(D ** -0.5), ctypes.c_int(0), ctypes.c_int(h), ctypes.c_int(m0),
               ctypes.c_int(m1), ctypes.c_int(0))
            got = oracle.from_bf16(host(torch, o)[0, m0:m1, h])
            assert np.abs(got - oracle.from_bf16(o_ref[0, m0:m1, h])).max() <= ATOL_BF16
            assert np.abs(lse.cpu().numpy()[0, m0:m1, h] - lse_ref[0, m0:m1, h]).max() <= 2e-5 * 10
    hs = slice(8, 12)
    o32, lse32 = torch_reference(torch, q[:, :, hs], k[:, :, hs], v[:, :, hs], True)
    assert (o[:, :, hs].float() - o32).abs().max().item() <= ATOL_BF16
    assert (lse[:, :, hs] - lse32).abs().max().item() <= 1e-4


def run_bwd(pkg, torch, q, k, v, dout, causal, deterministic=False):
    L = pkg.lib
    B, S, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    qd, kd, vd, gd = dev(torch, q), dev(torch, k), dev(torch, v), dev(torch, dout)
    o = torch.empty_like(qd)
    lse = torch.empty(B, S, H, device="cuda")
    desc = L.attn_desc(B, H, S, Skv, D, causal, kv_heads=Hkv, deterministic=deterministic)
    stream = torch.cuda.current_stream().cuda_stream
    L.attention_fwd(desc, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), stream)
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (qd, kd, vd))
    need = L.attention_bwd_workspace_bytes(desc)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    L.attention_bwd(desc, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), gd.data_ptr(),
                    dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need, stream)
    assert L.attention_device_error() == 0 and L.attention_bwd_device_error() == 0
    return host(torch, dq), host(torch, dk), host(torch, dv), host(torch, o), lse.cpu().numpy()


MAX_ABS_REACHED = {}   # per gradient, the largest plain max-abs difference any case reached (printed by the last test)


def close_grad(oracle, got_bits, want, what):
    """2e-2 max-abs against the Float32 CPU reference, relative to the gradient's own scale
    (gradients of N(0,1) data reach tens), and 1e-2 in norm."""
    got = oracle.from_bf16(got_bits).astype(np.float64)
    want = np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    scale = max(1.0, np.abs(want).max())
    worst = np.abs(got - want).max()
    # the plain max-abs reached is part of the message either way: 2e-2 holds as it stands while the gradient's
    # values stay below ~2.5 (one BFloat16 ulp of a value in [4, 8) is already 3e-2)
    assert worst <= ATOL_BF16 * scale, f"{what}: max-abs {worst:.3e} at gradient scale {scale:.2f} (bound {ATOL_BF16 * scale:.3e})"
    MAX_ABS_REACHED[what] = max(MAX_ABS_REACHED.get(what, 0.0), float(worst))
    # (a gradient that is exactly zero in exact arithmetic -- a query that sees only itself -- comes out as
    # rounding noise: allow 1e-5 per element on top)
    assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want) + 1e-5 * np.sqrt(want.size), what


@pytest.mark.parametrize("deterministic", [False, True])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,H,Hkv,S", GEOMETRIES)
def test_backward_against_oracle(pkg, cuda, oracle, B, H, Hkv, S, causal, deterministic):
    D = 128
    q = oracle.to_bf16(oracle.normal((B, S, H, D), 21 + S))
    k = oracle.to_bf16(oracle.normal((B, S, Hkv, D), 22 + S))
    v = oracle.to_bf16(oracle.normal((B, S, Hkv, D), 23 + S))
    g = oracle.to_bf16(oracle.normal((B, S, H, D), 24 + S))
    dq, dk, dv, o, lse = run_bwd(pkg, cuda, q, k, v, g, causal, deterministic)
    # the oracle's pullback from the same saved output and log-sum-exp the kernel read
    dq_ref, dk_ref, dv_ref = oracle.attention_bwd(q, k, v, o, lse, g, causal, threads=8)
    close_grad(oracle, dq, oracle.from_bf16(dq_ref), "dq")
    close_grad(oracle, dk, oracle.from_bf16(dk_ref), "dk")
    close_grad(oracle, dv, oracle.from_bf16(dv_ref), "dv")
    _, _, dq64, dk64, dv64 = oracle.attention_f64(q, k, v, causal, dout=g)
    close_grad(oracle, dq, dq64, "dq vs Float64")
    close_grad(oracle, dk, dk64, "dk vs Float64")
    close_grad(oracle, dv, dv64, "dv vs Float64")


def test_backward_repeats_bit_for_bit(pkg, cuda, oracle):
    """The deterministic form repeats bit for bit.  The default form adds each key tile's dQ contribution into a
    Float32 accumulator in whatever order the tiles finish: its dK and dV repeat bit for bit, its dQ to the
    rounding of a Float32 sum (at most one BFloat16 ulp after the final rounding), and the two forms agree
    likewise."""
    B, S, H, D = 1, 640, 4, 128
    q, k, v, g = (oracle.to_bf16(oracle.normal((B, S, H if i != 1 and i != 2 else 2, D), 31 + i)) for i in range(4))
    first = run_bwd(pkg, cuda, q, k, v, g, True, deterministic=True)
    again = run_bwd(pkg, cuda, q, k, v, g, True, deterministic=True)
    for a, b in zip(first[:3], again[:3]):
        assert np.array_equal(a, b)
    one = run_bwd(pkg, cuda, q, k, v, g, True)
    two = run_bwd(pkg, cuda, q, k, v, g, True)
    assert np.array_equal(one[1], two[1]) and np.array_equal(one[2], two[2])
    assert np.array_equal(one[1], first[1]) and np.array_equal(one[2], first[2])    # dK, dV: the same products
    fa, fb = (oracle.from_bf16(x[0]).astype(np.float64) for x in (one, two))
    assert (np.abs(fa - fb) <= 2.0 ** -7 * np.abs(fb) + 1e-3).all()
    # against the deterministic form's dQ, whose kernel keeps P in Float32 where this one rounds it first:
    # the two agree as each agrees with the oracle
    fd = oracle.from_bf16(first[0]).astype(np.float64)
    assert np.abs(fa - fd).max() <= ATOL_BF16 * max(1.0, np.abs(fd).max())
    assert np.linalg.norm(fa - fd) <= 1e-2 * np.linalg.norm(fd)


@pytest.mark.parametrize("deterministic", [False, True])
def test_backward_benchmark_geometry(pkg, cuda, deterministic):
    """S=4096, D=128 causal, 4 heads of the 1/8 sub-batch against the Float32 PyTorch restatement."""
    torch, L = cuda, pkg.lib
    torch.backends.cuda.matmul.allow_tf32 = False
    B, S, H, D = 1, 4096, 4, 128
    gen = torch.Generator(device="cuda").manual_seed(20261125 + 5)
    q, k, v, g = (torch.randn(B, S, H, D, device="cuda", generator=gen).bfloat16() for _ in range(4))
    o, lse = torch.empty_like(q), torch.empty(B, S, H, device="cuda")
    desc = L.attn_desc(B, H, S, S, D, True, deterministic=deterministic)
    stream = torch.cuda.current_stream().cuda_stream
    L.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), stream)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    need = L.attention_bwd_workspace_bytes(desc)
    assert (need > 4 * 2 * B * H * S + 1024) == (not deterministic)    # the Float32 dq accumulator of the default form
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    L.attention_bwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), g.data_ptr(),
                    dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need, stream)
    assert L.attention_device_error() == 0 and L.attention_bwd_device_error() == 0
    _, _, dq32, dk32, dv32 = torch_reference(torch, q, k, v, True, dout=g)
    for got, want, name in ((dq, dq32, "dq"), (dk, dk32, "dk"), (dv, dv32, "dv")):
        err = (got.float() - want).abs().max().item()
        scale = max(1.0, want.abs().max().item())
        assert err <= ATOL_BF16 * scale, (name, err, scale)
        assert ((got.float() - want).norm() / want.norm()).item() <= 1e-2, name
    print("largest plain max-abs differences reached by the gradient cases:", MAX_ABS_REACHED)


def test_tuner_picks_a_backward_form(pkg, cuda):
    """tb200_attention_bwd_tune times both forms and answers 0 or 1; dq, dk, dv hold the pullback either way; other
    head dimensions have one schedule."""
    torch, L = cuda, pkg.lib
    B, S, H, D = 1, 1024, 4, 128
    q, k, v, g = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(4))
    o, lse = torch.empty_like(q), torch.empty(B, S, H, device="cuda")
    desc = L.attn_desc(B, H, S, S, D, True)
    L.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr())
    need = L.attention_bwd_workspace_bytes(desc)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    grads = [torch.full_like(q, float("nan")) for _ in range(3)]
    form = L.attention_bwd_tune(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), g.data_ptr(),
                                *(t.data_ptr() for t in grads), ws.data_ptr(), need)
    assert form in (0, 1)
    _, _, dq32, dk32, dv32 = torch_reference(torch, q, k, v, True, dout=g)
    for got, want in zip(grads, (dq32, dk32, dv32)):
        assert (got.float() - want).abs().max().item() <= ATOL_BF16 * max(1.0, want.abs().max().item())
    assert L.attention_bwd_device_error() == 0
    small = L.attn_desc(1, 2, 64, 64, 32, True)
    x = torch.randn(1, 64, 2, 32, device="cuda").bfloat16()
    o2, lse2 = torch.empty_like(x), torch.empty(1, 64, 2, device="cuda")
    L.attention_fwd(small, x.data_ptr(), x.data_ptr(), x.data_ptr(), o2.data_ptr(), lse2.data_ptr())
    need2 = L.attention_bwd_workspace_bytes(small)
    ws2 = torch.empty(max(need2, 16), dtype=torch.uint8, device="cuda")
    outs = [torch.empty_like(x) for _ in range(3)]
    assert L.attention_bwd_tune(small, x.data_ptr(), x.data_ptr(), x.data_ptr(), o2.data_ptr(), lse2.data_ptr(), x.data_ptr(),
                                *(t.data_ptr() for t in outs), ws2.data_ptr(), need2) == 1
