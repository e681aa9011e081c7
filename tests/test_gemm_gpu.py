"""Products with fused epilogues through the C ABI against the CPU oracle:
the reference's product tests' shapes (test/cuda/products.jl:9-64: 96x80 * 80x112
with a GELU epilogue, split-K 64x3000 * 3000x48, layouts NN/TN/NT/TT, BFloat16
with a cast in the epilogue), ragged edges, both tile variants, and the
benchmark's layer shapes against a plain Float32 matmul of the same inputs."""
import numpy as np
import pytest

from helpers import ATOL_BF16, RTOL_F32, agree

pytestmark = pytest.mark.gpu


def dev(torch, a):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.view(torch.bfloat16) if a.dtype == np.uint16 else t).cuda()


def host(torch, t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.cpu().numpy()


def operands(oracle, M, N, K, a_mn, b_mn, seed, bf16):
    A = oracle.normal((K, M) if a_mn else (M, K), seed)
    B = oracle.normal((K, N) if b_mn else (N, K), seed + 1)
    if bf16:
        A, B = oracle.to_bf16(A), oracle.to_bf16(B)
    return A, B


def close_bf16(oracle, got_bits, want_f32, k):
    """2e-2 max-abs against the Float32 CPU reference, scaled by the product's
    magnitude sqrt(K) for N(0,1) factors (the tolerance is stated for O(1) results)."""
    got = oracle.from_bf16(got_bits).astype(np.float64)
    want = np.asarray(want_f32, np.float64)
    scale = max(1.0, np.abs(want).max())
    worst = np.abs(got - want).max()
    assert worst <= ATOL_BF16 * scale, f"max-abs {worst:.3e} vs {ATOL_BF16 * scale:.3e}"


LAYOUTS = [(False, False), (False, True), (True, False), (True, True)]
SHAPES = [(96, 112, 80), (128, 256, 64), (200, 136, 200), (64, 48, 3000), (256, 512, 320), (8, 8, 8), (130, 264, 72)]


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_bf16_tensor_core_product(pkg, cuda, oracle, M, N, K, a_mn, b_mn):
    L = pkg.lib
    A, B = operands(oracle, M, N, K, a_mn, b_mn, 1000 + M + K, True)
    want = oracle.gemm(A, B, M=M, N=N, K=K, a_km=a_mn, b_kn=b_mn, want_pre=True)[1]
    Ad, Bd = dev(cuda, A), dev(cuda, B)
    for tile_n, direct in ((128, False), (256, False), (256, True), (512, False), (512, True)):
        C = cuda.full((M, N), float("nan"), device="cuda", dtype=cuda.bfloat16)
        L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn),
               tile_n=tile_n, direct_epilogue=direct, stream=cuda.cuda.current_stream().cuda_stream)
        assert L.device_error() == 0
        close_bf16(oracle, host(cuda, C), want, K)
        # and Float32 output of the same accumulators: tight, the only difference is summation order
        C32 = cuda.empty((M, N), device="cuda")
        L.gemm(Ad.data_ptr(), Bd.data_ptr(), C32.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn),
               out_dtype=L.F32, tile_n=tile_n, direct_epilogue=direct)
        assert L.device_error() == 0
        agree(C32.cpu().numpy(), want, 1e-5)


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
def test_generic_kernel_float32(pkg, cuda, oracle, a_mn, b_mn):
    L = pkg.lib
    M, N, K = 96, 112, 80
    A, B = operands(oracle, M, N, K, a_mn, b_mn, 7, False)
    Ad, Bd = dev(cuda, A), dev(cuda, B)
    C = cuda.empty((M, N), device="cuda")
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn),
           in_dtype=L.F32)
    agree(C.cpu().numpy(), oracle.gemm(A, B, M=M, N=N, K=K, a_km=a_mn, b_kn=b_mn), RTOL_F32)
    # odd sizes and leading dimensions, BFloat16 through the generic kernel
    M, N, K = 33, 45, 51
    A, B = operands(oracle, M, N, K, a_mn, b_mn, 9, True)
    C = cuda.empty((M, N), device="cuda", dtype=cuda.bfloat16)
    Ad, Bd = dev(cuda, A), dev(cuda, B)
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn))
    close_bf16(oracle, host(cuda, C), oracle.gemm(A, B, M=M, N=N, K=K, a_km=a_mn, b_kn=b_mn, want_pre=True)[1], K)


@pytest.mark.parametrize("force_simt,direct,tile_n", [(False, False, 0), (False, True, 0), (True, False, 0),
                                                      (False, False, 512), (False, True, 512)])
def test_epilogues(pkg, cuda, oracle, force_simt, direct, tile_n):
    """tile_n 512: the same epilogues behind tiles of 256 x 256 computed by pairs of CTAs (300 rows: one whole pair
    tile and a ragged one)."""
    L = pkg.lib
    M, N, K = (300, 264, 96) if tile_n else (200, 136, 96)
    A, B = operands(oracle, M, N, K, False, True, 21, True)
    A = oracle.to_bf16(oracle.from_bf16(A) * 0.1)
    bias = oracle.to_bf16(oracle.normal((N,), 23))
    Ad, Bd, bd = dev(cuda, A), dev(cuda, B), dev(cuda, bias)
    acc = oracle.gemm(A, B, M=M, N=N, K=K, want_pre=True)[1]
    pre = acc + oracle.from_bf16(bias)
    run = dict(a_layout=L.K_MAJOR, b_layout=L.MN_MAJOR, force_simt=force_simt, direct_epilogue=direct, tile_n=tile_n)

    def call(**kw):
        C = cuda.empty((M, N), device="cuda", dtype=cuda.bfloat16)
        L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, **run, **kw)
        assert L.device_error() == 0
        return C

    close_bf16(oracle, host(cuda, call(epilogue=L.EPI_BIAS, bias=bd.data_ptr())), pre, K)
    Z = cuda.empty((M, N), device="cuda", dtype=cuda.bfloat16)
    got = call(epilogue=L.EPI_BIAS_GELU, bias=bd.data_ptr(), aux_out=Z.data_ptr())
    gelu = np.vectorize(oracle.gelu_tanh)(pre)
    close_bf16(oracle, host(cuda, got), gelu, K)
    close_bf16(oracle, host(cuda, Z), pre, K)
    close_bf16(oracle, host(cuda, call(epilogue=L.EPI_BIAS_TANH, bias=bd.data_ptr())), np.tanh(pre), K)
    aux = oracle.to_bf16(oracle.normal((M, N), 29))
    auxd = dev(cuda, aux)
    grad = np.vectorize(oracle.gelu_tanh_grad)(oracle.from_bf16(aux))
    close_bf16(oracle, host(cuda, call(epilogue=L.EPI_MUL_GELU_GRAD, aux=auxd.data_ptr())), acc * grad, K)
    t = np.tanh(oracle.from_bf16(aux))
    tb = oracle.to_bf16(t.astype(np.float32))
    tbd = dev(cuda, tb)
    close_bf16(oracle, host(cuda, call(epilogue=L.EPI_MUL_TANH_GRAD, aux=tbd.data_ptr())),
               acc * (1 - oracle.from_bf16(tb) ** 2), K)
    # accumulate into an existing array, scaled: D .+ alpha * A*B (ext/cuBLASExt.jl:25-29), in place
    D = dev(cuda, aux).clone()
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), D.data_ptr(), M, N, K, **run, epilogue=L.EPI_AXPY, aux=D.data_ptr(),
           alpha=-0.5)
    assert L.device_error() == 0
    close_bf16(oracle, host(cuda, D), oracle.from_bf16(aux) - 0.5 * acc, K)


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [
    (8192, 4096, 1024, False, True),    # layer 1 forward
    (2048, 4096, 4096, False, False),   # dX
    (4096, 4096, 2048, True, True),     # dW over a quarter of the batch
    (1024, 1024, 4096, False, True),    # last layer, narrow tiles
])
def test_layer_shapes_against_float32_matmul(pkg, cuda, M, N, K, a_mn, b_mn):
    """The benchmark's products, too large for the scalar oracle: compared with a plain
    Float32 matmul of the same BFloat16 inputs (cuBLAS, TF32 off) and by linearity."""
    torch, L = cuda, pkg.lib
    torch.backends.cuda.matmul.allow_tf32 = False
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    A = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).bfloat16()
    B = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).bfloat16()
    Af = (A.float().t() if a_mn else A.float())
    Bf = (B.float() if b_mn else B.float().t())
    want = Af @ Bf
    C = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn))
    assert L.device_error() == 0
    err = (C.float() - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= 2e-2 * scale, (err, scale)
    rel = ((C.float() - want).norm() / want.norm()).item()
    assert rel < 4e-3, rel   # BFloat16 rounding of the result alone is 2^-9 relative
    C32 = torch.empty((M, N), device="cuda")
    L.gemm(A.data_ptr(), B.data_ptr(), C32.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn),
           out_dtype=L.F32)
    assert L.device_error() == 0
    assert ((C32 - want).norm() / want.norm()).item() < 2e-5


def test_pointwise_and_folds(pkg, cuda, oracle):
    torch, L = cuda, pkg.lib
    stream = torch.cuda.current_stream().cuda_stream
    ws_bytes = L.squared_error_workspace_bytes()
    ws = torch.zeros(ws_bytes, device="cuda", dtype=torch.uint8)
    for count, dt in ((64 * 16, torch.float32), (1000003, torch.float32), (8192 * 1024, torch.bfloat16), (77, torch.bfloat16)):
        g = torch.Generator(device="cuda").manual_seed(count)
        a = torch.randn(count, device="cuda", generator=g).to(dt)
        b = torch.randn(count, device="cuda", generator=g).to(dt)
        grad = torch.empty_like(a)
        loss = torch.zeros(1, device="cuda")
        code = L.F32 if dt == torch.float32 else L.BF16
        for _ in range(2):   # the ticket is left ready for the next call
            L.squared_error(a.data_ptr(), b.data_ptr(), grad.data_ptr(), loss.data_ptr(), count, 0.25, 0.5, False,
                            code, ws.data_ptr(), ws_bytes, stream)
            d = a.double() - b.double()
            assert abs(loss.item() - 0.25 * (d * d).sum().item()) <= 1e-5 * 0.25 * (d * d).sum().item()
            tol = 1e-6 if dt == torch.float32 else 2e-2
            assert (grad.double() - d).abs().max().item() <= tol * max(1.0, d.abs().max().item())
        # the README's sum(abs2, tanh(z)) and its pullback 2y(1 - y^2)
        y = torch.tanh(a.float()).to(dt)
        L.squared_error(y.data_ptr(), 0, grad.data_ptr(), loss.data_ptr(), count, 1.0, 1.0, True, code,
                        ws.data_ptr(), ws_bytes, stream)
        yd = y.double()
        assert abs(loss.item() - (yd * yd).sum().item()) <= 1e-5 * (yd * yd).sum().item()
        assert (grad.double() - 2 * yd * (1 - yd * yd)).abs().max().item() <= (1e-6 if dt == torch.float32 else 1e-2)
    # column sums: the bias gradient
    for rows, n, dt in ((8192, 4096, torch.bfloat16), (100, 33, torch.float32), (1, 8, torch.bfloat16), (5000, 1024, torch.float32)):
        x = torch.randn(rows, n, device="cuda").to(dt)
        out = torch.empty(n, device="cuda", dtype=dt)
        need = L.colsum_workspace_bytes(rows, n)
        cws = torch.empty(max(need, 16), device="cuda", dtype=torch.uint8)
        L.colsum(x.data_ptr(), out.data_ptr(), rows, n, n, 1.0, L.F32 if dt == torch.float32 else L.BF16,
                 cws.data_ptr(), need, stream)
        want = x.double().sum(dim=0)
        tol = 1e-5 if dt == torch.float32 else 2 ** -8
        # a sum that cancels is judged against the size of what was summed (the column's 2-norm), not its result
        scale = torch.maximum(want.abs(), x.double().norm(dim=0)).clamp(min=1.0)
        assert ((out.double() - want).abs() <= tol * scale * 2).all()
    # y += alpha x
    for count in (8, 1003, 4096 * 4096):
        yv = torch.randn(count, device="cuda").bfloat16()
        xv = torch.randn(count, device="cuda").bfloat16()
        want = (yv.float() - 0.125 * xv.float()).bfloat16()
        L.axpy(yv.data_ptr(), xv.data_ptr(), -0.125, count, L.BF16, L.BF16, stream)
        assert torch.equal(yv, want)


def test_readme_loss_and_gradient(pkg, cuda, oracle):
    """loss(w,b,x) = sum(abs2, tanh.(w'x .+ b)), w 32x64, b 64, x 32x16, Float32 (README.md:15):
    the loss and (dw, db, dx) through the C ABI against the oracle's restatement."""
    torch, L = cuda, pkg.lib
    stream = torch.cuda.current_stream().cuda_stream
    I, J, N = 32, 64, 16
    w, b, x = oracle.normal((J, I), 20261126), oracle.normal((J,), 20261127), oracle.normal((N, I), 20261128)
    loss_ref, dw_ref, db_ref, dx_ref = oracle.readme_loss_grad(w, b, x)
    wd, bd, xd = dev(torch, w), dev(torch, b), dev(torch, x)
    y = torch.empty(N, J, device="cuda")
    gz = torch.empty(N, J, device="cuda")
    dw, db, dx = torch.empty(J, I, device="cuda"), torch.empty(J, device="cuda"), torch.empty(N, I, device="cuda")
    loss = torch.zeros(1, device="cuda")
    ws_bytes = L.squared_error_workspace_bytes()
    ws = torch.zeros(ws_bytes, device="cuda", dtype=torch.uint8)
    f32 = dict(in_dtype=L.F32, stream=stream)
    # y[n][j] = tanh(sum_i x[n][i] w[j][i] + b[j])
    L.gemm(xd.data_ptr(), wd.data_ptr(), y.data_ptr(), N, J, I, a_layout=L.K_MAJOR, b_layout=L.K_MAJOR,
           epilogue=L.EPI_BIAS_TANH, bias=bd.data_ptr(), **f32)
    L.squared_error(y.data_ptr(), 0, gz.data_ptr(), loss.data_ptr(), N * J, 1.0, 1.0, True, L.F32, ws.data_ptr(),
                    ws_bytes, stream)
    # dw[j][i] = sum_n gz[n][j] x[n][i];  dx[n][i] = sum_j gz[n][j] w[j][i];  db[j] = sum_n gz[n][j]
    L.gemm(gz.data_ptr(), xd.data_ptr(), dw.data_ptr(), J, I, N, a_layout=L.MN_MAJOR, b_layout=L.MN_MAJOR, **f32)
    L.gemm(gz.data_ptr(), wd.data_ptr(), dx.data_ptr(), N, I, J, a_layout=L.K_MAJOR, b_layout=L.MN_MAJOR, **f32)
    need = L.colsum_workspace_bytes(N, J)
    cws = torch.empty(max(need, 16), device="cuda", dtype=torch.uint8)
    L.colsum(gz.data_ptr(), db.data_ptr(), N, J, J, 1.0, L.F32, cws.data_ptr(), need, stream)
    torch.cuda.synchronize()
    assert abs(loss.item() - loss_ref) <= RTOL_F32 * abs(loss_ref)
    agree(dw.cpu().numpy(), dw_ref, RTOL_F32)
    agree(db.cpu().numpy(), db_ref, RTOL_F32)
    agree(dx.cpu().numpy(), dx_ref, RTOL_F32)


def test_mlp_step_against_oracle(pkg, cuda, oracle):
    """A small MLP step (same structure as the benchmark's: GELU(tanh) between layers, bias, MSE,
    SGD) against the oracle's restatement: loss, every layer's pullback, gradients and the update."""
    torch = cuda
    sizes, batch, rate = (64, 128, 96, 32), 48, 1e-3
    ws = [oracle.to_bf16(0.2 * oracle.normal((sizes[i], sizes[i + 1]), 50 + i)) for i in range(3)]
    bs = [oracle.to_bf16(0.1 * oracle.normal((sizes[i + 1],), 60 + i)) for i in range(3)]
    x = oracle.to_bf16(oracle.normal((batch, sizes[0]), 70))
    y = oracle.to_bf16(oracle.normal((batch, sizes[-1]), 71))
    loss_ref, dz_ref, dw_ref, db_ref, w_ref, b_ref, a_ref, z_ref = oracle.mlp_step(ws, bs, x, y, rate)
    for fuse in (False, True):
        step = pkg.mlp.MLPStep(torch, sizes, batch, rate, weights=[dev(torch, w) for w in ws],
                               biases=[dev(torch, b) for b in bs], fuse_update=fuse)
        loss = step.step(dev(torch, x), dev(torch, y))
        torch.cuda.synchronize()
        assert pkg.lib.device_error() == 0
        assert abs(loss.item() - loss_ref) <= 2e-3 * abs(loss_ref)
        for i in range(3):
            close_bf16(oracle, host(torch, step.a[i + 1]), oracle.from_bf16(a_ref[i + 1]), sizes[i])
            close_bf16(oracle, host(torch, step.dz[i]), oracle.from_bf16(dz_ref[i]), 1)
            ref = oracle.from_bf16(dz_ref[i])
            assert np.linalg.norm(oracle.from_bf16(host(torch, step.dz[i])) - ref) <= 1e-2 * np.linalg.norm(ref)
            close_bf16(oracle, host(torch, step.w[i]), oracle.from_bf16(w_ref[i]), 1)
            close_bf16(oracle, host(torch, step.b[i]), oracle.from_bf16(b_ref[i]), 1)
            got_db = oracle.from_bf16(host(torch, step.db[i]))
            assert np.abs(got_db - db_ref[i]).max() <= 2e-2 * max(1.0, np.abs(db_ref[i]).max())
            if not fuse:
                got = oracle.from_bf16(host(torch, step.dw[i]))
                rel = np.linalg.norm(got - dw_ref[i]) / np.linalg.norm(dw_ref[i])
                assert rel < 5e-3, rel


def test_mlp_step_replayed_from_stretch_graphs(pkg, cuda, oracle):
    """The data-parallel form of the step (unfused updates) replayed from one CUDA graph per stretch between two
    gradient exchanges leaves the same bits as the same steps launched kernel by kernel."""
    torch = cuda
    sizes, batch, rate = (64, 128, 96, 32), 48, 1e-3
    ws = [oracle.to_bf16(0.2 * oracle.normal((sizes[i], sizes[i + 1]), 50 + i)) for i in range(3)]
    bs = [oracle.to_bf16(0.1 * oracle.normal((sizes[i + 1],), 60 + i)) for i in range(3)]
    x, y = dev(torch, oracle.to_bf16(oracle.normal((batch, sizes[0]), 70))), dev(torch, oracle.to_bf16(oracle.normal((batch, sizes[-1]), 71)))
    make = lambda: pkg.mlp.MLPStep(torch, sizes, batch, rate, weights=[dev(torch, w) for w in ws],
                                   biases=[dev(torch, b) for b in bs], fuse_update=False)
    eager, graphed = make(), make()
    for _ in range(3):
        eager.step(x, y)
    replay = graphed.capture_segments(x, y)   # runs the step once itself
    replay()
    loss = replay()
    torch.cuda.synchronize()
    assert pkg.lib.device_error() == 0
    assert loss.item() == eager.loss.item()
    for i in range(3):
        assert torch.equal(graphed.w[i], eager.w[i]) and torch.equal(graphed.b[i], eager.b[i])
    with pytest.raises(ValueError):
        pkg.mlp.MLPStep(torch, sizes, batch, rate, fuse_update=True).capture_segments(x, y)


def test_products_and_attention_through_the_plugin_mirror(pkg, cuda, oracle):
    """Binding -> supports -> build -> launch for a product template and an attention template, with the
    arrays described as Tempest describes them (column-major `Strided` views)."""
    torch, I = cuda, pkg.implement
    lib, target = I.B200Kernels(), I.Target()
    m, k, n = 96, 64, 40   # w (m, k), x (k, n): memory w [k][m], x [n][k], y [n][m]
    w = oracle.to_bf16(0.2 * oracle.normal((k, m), 3))
    x = oracle.to_bf16(oracle.normal((n, k), 4))
    b = oracle.to_bf16(oracle.normal((m,), 5))
    wd, xd, bd = dev(torch, w), dev(torch, x), dev(torch, b)
    y = torch.empty(n, m, device="cuda", dtype=torch.bfloat16)
    bind = I.Binding("linear_bias_gelu", {"m": m, "k": k, "n": n},
                     {"w": I.dense_matrix(wd, "BFloat16", m, k, 1), "x": I.dense_matrix(xd, "BFloat16", k, n, 2),
                      "b": I.dense_vector(bd, "BFloat16", m, 3), "y": I.dense_matrix(y, "BFloat16", m, n, 4)})
    assert lib.supports(target, bind)
    launch, description = lib.build(target, bind)
    assert "linear_bias_gelu" in description
    launch()
    torch.cuda.synchronize()
    want = oracle.gemm(x, w, bias=b, M=n, N=m, K=k, a_km=False, b_kn=True, epilogue=2, want_pre=True)[1]
    want = np.vectorize(oracle.gelu_tanh)(want)
    close_bf16(oracle, host(torch, y), want, k)
    # attention, causal, with its log-sum-exp, then its pullback through the same mirror
    B, S, H, D = 1, 200, 2, 128
    q, kk, v, g = (oracle.to_bf16(oracle.normal((B, S, H, D), 10 + i)) for i in range(4))
    qd, kd, vd, gd = (dev(torch, a) for a in (q, kk, v, g))
    o, lse = torch.empty_like(qd), torch.empty(B, S, H, device="cuda")
    e = {"d": D, "h": H, "hk": H, "m": S, "n": S, "b": B, "one": 1}
    heads = lambda t, val: I.dense_heads(t, "BFloat16", D, H, S, B, val)  # noqa: E731
    fwd = I.Binding("attention_causal_lse", e, {"q": heads(qd, 1), "k": heads(kd, 2), "v": heads(vd, 3), "o": heads(o, 4),
                                                "lse": I.Strided("Float32", 0, (1, H, S, B), (1, 1, H, H * S), lse, 5)})
    assert lib.supports(target, fwd)
    launch, _ = lib.build(target, fwd)
    launch()
    dq, dk, dv = (torch.empty_like(qd) for _ in range(3))
    bwd = I.Binding("attention_causal_pullback", e, dict(fwd.arrays, g=heads(gd, 6), dq=heads(dq, 7), dk=heads(dk, 8),
                                                         dv=heads(dv, 9)))
    assert lib.supports(target, bwd)
    launch, _ = lib.build(target, bwd)
    launch()
    torch.cuda.synchronize()
    assert pkg.lib.attention_device_error() == 0 and pkg.lib.attention_bwd_device_error() == 0
    o64, lse64, dq64, dk64, dv64 = oracle.attention_f64(q, kk, v, True, dout=g)
    assert np.abs(oracle.from_bf16(host(torch, o)) - o64).max() <= ATOL_BF16
    assert np.abs(lse.cpu().numpy() - lse64).max() <= 1e-4
    for got, want in ((dq, dq64), (dk, dk64), (dv, dv64)):
        gotf = oracle.from_bf16(host(torch, got))
        assert np.abs(gotf - want).max() <= ATOL_BF16 * max(1.0, np.abs(want).max())


def test_builds_keep_their_measured_picks_in_the_tuning_record(pkg, cuda, oracle, tmp_path, monkeypatch):
    """With a tuning record the mirror's `build` measures a product's variants once, keeps the pick in the record's
    file, and a later session (a new record on the same file) builds the same launch without measuring."""
    torch, I, T = cuda, pkg.implement, pkg.tuning
    m, k, n = 512, 256, 1024
    w = (0.1 * torch.randn(k, m, device="cuda")).bfloat16()
    x = torch.randn(n, k, device="cuda").bfloat16()
    y = torch.empty(n, m, device="cuda", dtype=torch.bfloat16)
    bind = I.Binding("linear", {"m": m, "k": k, "n": n},
                     {"w": I.dense_matrix(w, "BFloat16", m, k, 1), "x": I.dense_matrix(x, "BFloat16", k, n, 2),
                      "y": I.dense_matrix(y, "BFloat16", m, n, 4)})
    record = T.TuningRecord(torch.cuda.get_device_name(0), str(tmp_path))
    launch, note = I.B200Kernels(record=record).build(I.Target(), bind)
    assert "variants measured" in note and launch.pick["tile_n"] in (128, 256, 512) and record.written == 1
    y.zero_()
    launch()
    torch.cuda.synchronize()
    want = x.float() @ w.float()
    assert (y.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    later = T.TuningRecord(torch.cuda.get_device_name(0), str(tmp_path))
    monkeypatch.setattr(pkg.lib, "gemm_tune_desc", lambda *a, **k: (_ for _ in ()).throw(AssertionError("measured again")))
    launch2, note2 = I.B200Kernels(record=later).build(I.Target(), bind)
    assert "from the tuning record" in note2 and launch2.pick == launch.pick and later.written == 0
    y.zero_()
    launch2()
    torch.cuda.synchronize()
    assert (y.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()


def test_tune_returns_a_variant_and_leaves_the_product(pkg, cuda, oracle):
    """tb200_gemm_tune times the 128- and 256-wide tiles and the 256 x 256 tiles of CTA pairs (512) on the operands,
    returns one of them, and C holds the product; where there is nothing to choose it answers without measuring."""
    torch, L = cuda, pkg.lib
    M, N, K = 512, 1024, 256
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(K, N, device="cuda").bfloat16()
    C = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    width = L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, tune=True)
    assert width in (128, 256, 512)
    want = A.float() @ B.float()
    assert (C.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    C2 = torch.zeros_like(C)
    L.gemm(A.data_ptr(), B.data_ptr(), C2.data_ptr(), M, N, K, tile_n=width)
    assert torch.equal(C, C2)
    narrow = torch.zeros(M, 64, device="cuda", dtype=torch.bfloat16)
    assert L.gemm(A.data_ptr(), B.data_ptr(), narrow.data_ptr(), M, 64, K, ldb=N, tune=True) == 128
    with pytest.raises(L.TB200Error):
        L.gemm(0, B.data_ptr(), C.data_ptr(), M, N, K, tune=True)


def test_products_alike_through_the_plugin_mirror(pkg, cuda, oracle):
    """Several plain products of one shape built as one launch (the reference's `Products`), and moved to other
    buffers through `repoint` (which rewrites the arrays of addresses on the stream)."""
    torch, I = cuda, pkg.implement
    lib, target = I.B200Kernels(), I.Target()
    m, k, n, count = 64, 128, 64, 9
    ws = [oracle.to_bf16(0.2 * oracle.normal((k, m), 30 + i)) for i in range(count)]
    xs = [oracle.to_bf16(oracle.normal((n, k), 50 + i)) for i in range(count)]
    wd, xd = [dev(torch, w) for w in ws], [dev(torch, x) for x in xs]
    ys = [torch.full((n, m), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(count)]
    binds = [I.Binding("linear", {"m": m, "k": k, "n": n},
                       {"w": I.dense_matrix(wd[i], "BFloat16", m, k, 10 * i + 1), "x": I.dense_matrix(xd[i], "BFloat16", k, n, 10 * i + 2),
                        "y": I.dense_matrix(ys[i], "BFloat16", m, n, 10 * i + 3)}) for i in range(count)]
    launch, description = lib.build_alike(target, binds)
    assert "9 products alike" in description and launch.repoints()
    launch()
    torch.cuda.synchronize()
    for i in range(count):
        want = oracle.gemm(xs[i], ws[i], M=n, N=m, K=k, a_km=False, b_kn=True, want_pre=True)[1]
        close_bf16(oracle, host(torch, ys[i]), want, k)
    # the fourth product's input moves to another buffer
    moved = dev(torch, xs[0])
    launch.repoint(10 * 3 + 2, moved)
    ys[3].fill_(float("nan"))
    launch()
    torch.cuda.synchronize()
    want = oracle.gemm(xs[0], ws[3], M=n, N=m, K=k, a_km=False, b_kn=True, want_pre=True)[1]
    close_bf16(oracle, host(torch, ys[3]), want, k)
    with pytest.raises(ValueError):
        lib.build_alike(target, binds[:2] + [I.Binding("linear", {"m": m, "k": k, "n": 32}, binds[0].arrays)])
