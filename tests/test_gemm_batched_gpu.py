"""Batches of products, split sums, Float16 operands, prepared launches and the failure path of the
tensor-core product, through the C ABI against the CPU oracle.

Shapes follow the reference's product tests (test/cuda/products.jl): the batch `contract(A, B, (1,2,4),
(2,3,4), (1,3,4))` with A (32, 24, 5), B (24, 40, 5) (:46-57), the long sum 64x3000 * 3000x48 that must
split among blocks (:36-43), 96x80 * 80x112 (:10), and Float16 factors accumulating in Float32 with one
rounding (:25-30, tolerance eps(Float16) norm-wise)."""
import numpy as np
import pytest

from helpers import ATOL_BF16, agree
from test_gemm_gpu import close_bf16, dev, host, operands

pytestmark = pytest.mark.gpu


def batch_operands(oracle, batch, M, N, K, a_mn, b_mn, seed, share_b=False):
    As, Bs = [], []
    for i in range(batch):
        A, B = operands(oracle, M, N, K, a_mn, b_mn, seed + 2 * i, True)
        As.append(A)
        Bs.append(Bs[0] if (share_b and i) else B)
    return np.stack(As), np.stack(Bs)


@pytest.mark.parametrize("batch,M,N,K,a_mn,b_mn", [
    (5, 32, 40, 24, True, True),       # the reference's batched contract: Julia (m,k,b) x (k,n,b) column-major
    (5, 32, 40, 24, False, True),
    (3, 200, 136, 96, False, False),
    (7, 64, 64, 128, True, False),     # the per-chunk products of the delta rule: many small alike products
    (2, 256, 512, 320, False, True),
])
def test_batched_products(pkg, cuda, oracle, batch, M, N, K, a_mn, b_mn):
    torch, L = cuda, pkg.lib
    A, B = batch_operands(oracle, batch, M, N, K, a_mn, b_mn, 4000 + M + K)
    want = np.stack([oracle.gemm(A[i], B[i], M=M, N=N, K=K, a_km=a_mn, b_kn=b_mn, want_pre=True)[1]
                     for i in range(batch)])
    Ad, Bd = dev(torch, A), dev(torch, B)
    for force_simt, direct, tile_n in ((False, False, 0), (False, True, 0), (True, False, 0), (False, False, 512)):
        C = torch.full((batch, M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn),
               batch=batch, force_simt=force_simt, direct_epilogue=direct, tile_n=tile_n)
        assert L.device_error() == 0
        close_bf16(oracle, host(torch, C), want, K)
        C32 = torch.full((batch, M, N), float("nan"), device="cuda")
        L.gemm(Ad.data_ptr(), Bd.data_ptr(), C32.data_ptr(), M, N, K, a_layout=int(a_mn), b_layout=int(b_mn),
               batch=batch, out_dtype=L.F32, force_simt=force_simt, direct_epilogue=direct, tile_n=tile_n)
        assert L.device_error() == 0
        agree(C32.cpu().numpy(), want, 1e-5)


def test_batch_with_a_shared_weight_padded_members_and_bias(pkg, cuda, oracle):
    """Members at strides larger than their size (views into a bigger array), one B for every member
    (stride 0), a bias per member, the activation epilogue keeping what it saw."""
    torch, L = cuda, pkg.lib
    batch, M, N, K = 4, 72, 136, 64
    A, B = batch_operands(oracle, batch, M, N, K, False, True, 77, share_b=True)
    A = oracle.to_bf16(0.2 * oracle.from_bf16(A))
    bias = oracle.to_bf16(oracle.normal((batch, N), 78))
    pad_a, pad_c = M * K + 64, M * N + 256
    Abuf = torch.zeros(batch * pad_a, device="cuda", dtype=torch.bfloat16)
    for i in range(batch):
        Abuf[i * pad_a: i * pad_a + M * K] = dev(torch, A[i]).reshape(-1)
    Bd, bd = dev(torch, B[0]), dev(torch, bias)
    pre = np.stack([oracle.gemm(A[i], B[0], M=M, N=N, K=K, want_pre=True)[1] + oracle.from_bf16(bias[i])
                    for i in range(batch)])
    for direct in (False, True):
        Cbuf = torch.full((batch * pad_c,), float("nan"), device="cuda", dtype=torch.bfloat16)
        Zbuf = torch.full((batch * pad_c,), float("nan"), device="cuda", dtype=torch.bfloat16)
        L.gemm(Abuf.data_ptr(), Bd.data_ptr(), Cbuf.data_ptr(), M, N, K, batch=batch, stride_a=pad_a, stride_b=0,
               stride_c=pad_c, stride_bias=N, stride_aux_out=pad_c, epilogue=L.EPI_BIAS_GELU, bias=bd.data_ptr(),
               aux_out=Zbuf.data_ptr(), direct_epilogue=direct)
        assert L.device_error() == 0
        got = torch.stack([Cbuf[i * pad_c: i * pad_c + M * N].view(M, N) for i in range(batch)])
        saw = torch.stack([Zbuf[i * pad_c: i * pad_c + M * N].view(M, N) for i in range(batch)])
        close_bf16(oracle, host(torch, got), np.vectorize(oracle.gelu_tanh)(pre), K)
        close_bf16(oracle, host(torch, saw), pre, K)
        # the padding between members is untouched
        assert torch.isnan(Cbuf[M * N: pad_c].float()).all()
    # members that would overlap are refused
    with pytest.raises(L.TB200Error) as e:
        L.gemm(Abuf.data_ptr(), Bd.data_ptr(), Cbuf.data_ptr(), M, N, K, batch=batch, stride_a=pad_a, stride_b=0,
               stride_c=M * N - 1)
    assert e.value.status == -2


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(64, 48, 3000, False, True), (64, 48, 3000, True, False),
                                             (96, 112, 80, False, True), (130, 72, 4100, False, False)])
def test_split_sums(pkg, cuda, oracle, M, N, K, a_mn, b_mn):
    """The reference's split-K case and neighbours: the split result equals the unsplit one to Float32
    rounding, both match the oracle, every epilogue survives the merge, and a missing workspace falls back."""
    torch, L = cuda, pkg.lib
    A, B = operands(oracle, M, N, K, a_mn, b_mn, 5000 + K, True)
    A = oracle.to_bf16(0.05 * oracle.from_bf16(A))
    want = oracle.gemm(A, B, M=M, N=N, K=K, a_km=a_mn, b_kn=b_mn, want_pre=True)[1]
    Ad, Bd = dev(torch, A), dev(torch, B)
    lay = dict(a_layout=int(a_mn), b_layout=int(b_mn))
    auto = L.gemm_desc(M, N, K, **lay)
    need_auto = L.gemm_workspace_bytes(auto)
    assert (need_auto > 0) == (K >= 512)          # a long sum over a small output splits by itself
    for split in (0, 4, 16):
        d = L.gemm_desc(M, N, K, split_k=split, **lay)
        need = L.gemm_workspace_bytes(d)
        ws = torch.full((max(need, 16),), 255, device="cuda", dtype=torch.uint8)
        for direct in (False, True):
            C32 = torch.full((M, N), float("nan"), device="cuda")
            L.gemm(Ad.data_ptr(), Bd.data_ptr(), C32.data_ptr(), M, N, K, out_dtype=L.F32, split_k=split,
                   workspace=ws.data_ptr(), workspace_bytes=need, direct_epilogue=direct, **lay)
            assert L.device_error() == 0
            agree(C32.cpu().numpy(), want, 1e-5)
    # epilogues through the merge
    bias = oracle.to_bf16(oracle.normal((N,), 3))
    aux = oracle.to_bf16(oracle.normal((M, N), 4))
    bd, xd = dev(torch, bias), dev(torch, aux)
    d = L.gemm_desc(M, N, K, split_k=8, **lay)
    need = L.gemm_workspace_bytes(d)
    ws = torch.empty(max(need, 16), device="cuda", dtype=torch.uint8)
    run = dict(split_k=8, workspace=ws.data_ptr(), workspace_bytes=need, **lay)
    C = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    Z = torch.empty_like(C)
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, epilogue=L.EPI_BIAS_GELU, bias=bd.data_ptr(),
           aux_out=Z.data_ptr(), **run)
    pre = want + oracle.from_bf16(bias)
    close_bf16(oracle, host(torch, C), np.vectorize(oracle.gelu_tanh)(pre), 1)
    close_bf16(oracle, host(torch, Z), pre, 1)
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, epilogue=L.EPI_MUL_GELU_GRAD, aux=xd.data_ptr(), **run)
    close_bf16(oracle, host(torch, C), want * np.vectorize(oracle.gelu_tanh_grad)(oracle.from_bf16(aux)), 1)
    D = xd.clone()
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), D.data_ptr(), M, N, K, epilogue=L.EPI_AXPY, aux=D.data_ptr(), alpha=-0.5, **run)
    close_bf16(oracle, host(torch, D), oracle.from_bf16(aux) - 0.5 * want, 1)
    assert L.device_error() == 0
    # asked to split but given no workspace: the product still runs, unsplit
    C32 = torch.empty((M, N), device="cuda")
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), C32.data_ptr(), M, N, K, out_dtype=L.F32, split_k=8, **lay)
    agree(C32.cpu().numpy(), want, 1e-5)


def test_split_sum_of_a_batch(pkg, cuda, oracle):
    torch, L = cuda, pkg.lib
    batch, M, N, K = 3, 64, 64, 2048
    A, B = batch_operands(oracle, batch, M, N, K, False, True, 91)
    A = oracle.to_bf16(0.05 * oracle.from_bf16(A))
    want = np.stack([oracle.gemm(A[i], B[i], M=M, N=N, K=K, want_pre=True)[1] for i in range(batch)])
    d = L.gemm_desc(M, N, K, batch=batch)
    need = L.gemm_workspace_bytes(d)
    assert need > 0
    ws = torch.empty(need, device="cuda", dtype=torch.uint8)
    C32 = torch.empty((batch, M, N), device="cuda")
    Ad, Bd = dev(torch, A), dev(torch, B)
    L.gemm(Ad.data_ptr(), Bd.data_ptr(), C32.data_ptr(), M, N, K, batch=batch, out_dtype=L.F32,
           workspace=ws.data_ptr(), workspace_bytes=need)
    assert L.device_error() == 0
    agree(C32.cpu().numpy(), want, 1e-5)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (False, False), (True, True)])
def test_float16_operands(pkg, cuda, oracle, a_mn, b_mn):
    """Half factors accumulate in Float32 and round once (test/cuda/products.jl:25-30: 64x48 * 48x32,
    rtol eps(Float16)); also a shape that fills several tiles, with a bias and with a Float32 result."""
    torch, L = cuda, pkg.lib
    for M, N, K, scale in ((64, 32, 48, 0.1), (200, 264, 136, 0.1)):
        A = (scale * oracle.normal((K, M) if a_mn else (M, K), 600 + M)).astype(np.float16)
        B = oracle.normal((K, N) if b_mn else (N, K), 601 + M).astype(np.float16)
        bias = oracle.normal((N,), 602).astype(np.float16)
        Af = (A.T if a_mn else A).astype(np.float32)
        Bf = (B if b_mn else B.T).astype(np.float32)
        want = oracle.gemm(np.ascontiguousarray(Af), np.ascontiguousarray(Bf), M=M, N=N, K=K)   # Float32, sequential sums
        Ad, Bd, bd = (torch.from_numpy(x).cuda() for x in (A, B, bias))
        lay = dict(a_layout=int(a_mn), b_layout=int(b_mn), in_dtype=L.F16)
        for force_simt, direct in ((False, False), (False, True), (True, False)):
            C = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
            L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, force_simt=force_simt, direct_epilogue=direct, **lay)
            assert L.device_error() == 0
            got = C.float().cpu().numpy().astype(np.float64)
            assert np.linalg.norm(got - want) <= 2.0 ** -10 * np.linalg.norm(want)
            assert np.abs(got - want).max() <= 2.0 ** -10 * max(1.0, np.abs(want).max())   # one rounding of the result
            C32 = torch.empty((M, N), device="cuda")
            L.gemm(Ad.data_ptr(), Bd.data_ptr(), C32.data_ptr(), M, N, K, out_dtype=L.F32, epilogue=L.EPI_BIAS,
                   bias=bd.data_ptr(), force_simt=force_simt, direct_epilogue=direct, **lay)
            assert L.device_error() == 0
            agree(C32.cpu().numpy(), want + bias.astype(np.float32), 1e-5)
            D = torch.from_numpy(np.ones((M, N), np.float16)).cuda()
            L.gemm(Ad.data_ptr(), Bd.data_ptr(), D.data_ptr(), M, N, K, epilogue=L.EPI_AXPY, aux=D.data_ptr(), alpha=0.5,
                   force_simt=force_simt, direct_epilogue=direct, **lay)
            assert np.abs(D.float().cpu().numpy() - (1 + 0.5 * want)).max() <= 2.0 ** -10 * max(1.0, np.abs(want).max())
    # a BFloat16 result of Float16 factors is not a thing the reference forms
    with pytest.raises(L.TB200Error) as e:
        L.gemm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K, out_dtype=L.BF16, **lay)
    assert e.value.status == -3


def test_prepared_launch_and_repoint(pkg, cuda, oracle):
    """A plan gives the bits of the per-call entry, launch after launch; repoint moves an operand (the new
    array's product appears, the old result array is left alone) and refuses an address that is aligned
    less than the plan was built for."""
    torch, L = cuda, pkg.lib
    stream = torch.cuda.current_stream().cuda_stream
    M, N, K = 256, 384, 192
    g = torch.Generator(device="cuda").manual_seed(5)
    A, A2 = (torch.randn(M, K, device="cuda", generator=g).bfloat16() for _ in range(2))
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g).bfloat16()
    C, C2, Z, want = (torch.zeros(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(4))
    opts = dict(epilogue=L.EPI_BIAS_GELU)
    L.gemm(A.data_ptr(), B.data_ptr(), want.data_ptr(), M, N, K, bias=bias.data_ptr(), aux_out=Z.data_ptr(), **opts)
    plan = L.GemmPlan(L.gemm_desc(M, N, K, **opts), A.data_ptr(), B.data_ptr(), C.data_ptr(), bias=bias.data_ptr(),
                      aux_out=Z.data_ptr())
    for _ in range(3):
        C.zero_()
        plan.launch(stream)
        assert torch.equal(C, want)
    L.gemm(A2.data_ptr(), B.data_ptr(), want.data_ptr(), M, N, K, bias=bias.data_ptr(), aux_out=Z.data_ptr(), **opts)
    kept = C.clone()
    plan.repoint(L.GEMM_A, A2.data_ptr()).repoint(L.GEMM_C, C2.data_ptr())
    plan.launch(stream)
    assert torch.equal(C2, want) and torch.equal(C, kept)
    with pytest.raises(L.TB200Error) as e:
        plan.repoint(L.GEMM_A, A2.data_ptr() + 2)      # two bytes in: no TMA descriptor for that
    assert e.value.status == -4
    plan.launch(stream)                                # and the plan still runs as before
    assert torch.equal(C2, want)
    with pytest.raises(L.TB200Error):
        plan.repoint(99, A.data_ptr())
    assert L.device_error() == 0
    plan.close()
    # a plan of the generic kernel (Float32), and one of nothing at all
    Af, Bf = torch.randn(33, 17, device="cuda"), torch.randn(17, 9, device="cuda")
    Cf = torch.empty(33, 9, device="cuda")
    p32 = L.GemmPlan(L.gemm_desc(33, 9, 17, in_dtype=L.F32), Af.data_ptr(), Bf.data_ptr(), Cf.data_ptr())
    p32.launch(stream)
    agree(Cf.cpu().numpy(), oracle.gemm(Af.cpu().numpy(), Bf.cpu().numpy(), M=33, N=9, K=17), 1e-5)
    L.GemmPlan(L.gemm_desc(0, 9, 17, in_dtype=L.F32), 0, 0, 0).launch(stream)
    with pytest.raises(L.TB200Error):
        L.GemmPlan(L.gemm_desc(8, 8, 8), 0, B.data_ptr(), C.data_ptr())


def test_a_plan_on_pairs_of_ctas_draws_its_tiles_from_the_counter(pkg, cuda):
    """More 256 x 256 tiles than pairs of SMs: the first CTA of a pair draws the tile and passes it to the second;
    launched several times (the counter is left ready), with an epilogue, and after a launch whose loads were
    withheld (every wait runs out, both CTAs of every pair leave together)."""
    torch, L = cuda, pkg.lib
    M, N, K = 4096, 4352, 192
    A = (0.1 * torch.randn(M, K, device="cuda")).bfloat16()
    B = torch.randn(K, N, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    C = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    want = A.float() @ B.float() + bias.float()
    plan = L.GemmPlan(L.gemm_desc(M, N, K, epilogue=L.EPI_BIAS, tile_n=512), A.data_ptr(), B.data_ptr(), C.data_ptr(),
                      bias=bias.data_ptr())
    for _ in range(3):
        C.zero_()
        plan.launch()
        assert (C.float() - want).abs().max().item() <= ATOL_BF16 * want.abs().max().item()
    assert L.device_error() == 0
    plan.close()
    plan = L.GemmPlan(L.gemm_desc(M, N, K, epilogue=L.EPI_BIAS, tile_n=512, debug=1), A.data_ptr(), B.data_ptr(),
                      C.data_ptr(), bias=bias.data_ptr())
    plan.launch()
    assert L.device_error() in (3, 4)
    plan.close()
    plan = L.GemmPlan(L.gemm_desc(M, N, K, epilogue=L.EPI_BIAS), A.data_ptr(), B.data_ptr(), C.data_ptr(),
                      bias=bias.data_ptr())       # the library's own choice: pairs here
    C.zero_()
    plan.launch()
    assert (C.float() - want).abs().max().item() <= ATOL_BF16 * want.abs().max().item()
    assert L.device_error() == 0
    plan.close()


def test_a_bounded_wait_runs_out_and_the_device_stays_usable(pkg, cuda):
    """The failure path of the tensor-core product: with the test hook set the loading thread withholds its
    tiles, so the consumers' waits find nothing; each wait gives up after its (shortened) limit, the kernel
    records a code and drains, the launch returns, the code shows in tb200_device_error / tb200_device_errors,
    and the next ordinary product is correct.  No fault, trap or endless loop is involved: a wait that
    nothing satisfies runs into its limit."""
    torch, L = cuda, pkg.lib
    M, N, K = 256, 256, 256
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(K, N, device="cuda").bfloat16()
    C = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    assert L.device_errors() == 0
    L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, debug=1)    # returns: the launch only enqueues
    torch.cuda.synchronize()                                              # and the kernel ends by itself
    code = L.device_error()
    assert code in (3, 4), code                # the MMA thread's or the epilogue's wait for operands gave up
    # the same with pairs of CTAs on a tile: both CTAs' waits run out, both reach the pair's closing barrier
    L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, debug=1, tile_n=512)
    torch.cuda.synchronize()
    assert L.device_error() in (3, 4)
    # a plan with more tiles than SMs draws them from a counter: same ending, and the counters are left ready
    big = 2048
    A2 = torch.randn(big, K, device="cuda").bfloat16()
    B2 = torch.randn(K, big, device="cuda").bfloat16()
    C2 = torch.zeros(big, big, device="cuda", dtype=torch.bfloat16)
    plan = L.GemmPlan(L.gemm_desc(big, big, K, debug=1), A2.data_ptr(), B2.data_ptr(), C2.data_ptr())
    plan.launch()
    assert L.device_error() in (3, 4)
    plan.close()
    plan = L.GemmPlan(L.gemm_desc(big, big, K), A2.data_ptr(), B2.data_ptr(), C2.data_ptr())
    for _ in range(3):
        C2.zero_()
        plan.launch()
        want2 = A2.float() @ B2.float()
        assert (C2.float() - want2).abs().max().item() <= ATOL_BF16 * want2.abs().max().item()
    assert L.device_error() == 0
    plan.close()
    assert L.device_error() == 0               # reading it cleared it
    L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, debug=1)
    with pytest.raises(L.TB200Error):
        L.check_device()
    assert L.device_errors() == 0
    # the context is intact: the same product without the hook is right
    L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K)
    assert L.device_error() == 0
    want = A.float() @ B.float()
    assert (C.float() - want).abs().max().item() <= ATOL_BF16 * want.abs().max().item()


def test_tune_desc_picks_among_every_variant(pkg, cuda, oracle):
    torch, L = cuda, pkg.lib
    M, N, K = 64, 48, 3000
    A, B = operands(oracle, M, N, K, False, True, 8, True)
    A = oracle.to_bf16(0.05 * oracle.from_bf16(A))
    Ad, Bd = dev(torch, A), dev(torch, B)
    C = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    d = L.gemm_desc(M, N, K)
    need = L.gemm_workspace_bytes(d)
    ws = torch.empty(need, device="cuda", dtype=torch.uint8)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    L.gemm_tune_desc(d, Ad.data_ptr(), Bd.data_ptr(), C.data_ptr())
    assert d.tile_n == 128 and d.split_k in (0, 1) and d.direct_epilogue in (0, 1)
    want = oracle.gemm(A, B, M=M, N=N, K=K, want_pre=True)[1]
    close_bf16(oracle, host(torch, C), want, 1)
    plan = L.GemmPlan(d, Ad.data_ptr(), Bd.data_ptr(), C.data_ptr())
    C.zero_()
    plan.launch()
    close_bf16(oracle, host(torch, C), want, 1)
    assert L.device_error() == 0


def test_update_of_views_that_start_at_odd_elements(pkg, cuda):
    """y += alpha x on views that are not 16-byte aligned (a bias gradient behind a weight gradient of odd
    size in one bucket) takes the element-wise path instead of being refused."""
    torch, L = cuda, pkg.lib
    base_y = torch.randn(5000, device="cuda").bfloat16()
    base_x = torch.randn(5000, device="cuda").bfloat16()
    for off_y, off_x, count in ((1, 0, 1003), (3, 5, 4096), (0, 7, 77), (21, 21, 1)):
        y, x = base_y.clone(), base_x
        want = y.clone()
        want[off_y: off_y + count] = (y[off_y: off_y + count].float() - 0.125 * x[off_x: off_x + count].float()).bfloat16()
        L.axpy(y.data_ptr() + 2 * off_y, x.data_ptr() + 2 * off_x, -0.125, count, L.BF16, L.BF16)
        assert torch.equal(y, want)
    with pytest.raises(L.TB200Error) as e:    # a Float32 array one byte off its element size
        L.axpy(base_y.data_ptr() + 1, base_x.data_ptr(), 1.0, 4, L.F32, L.BF16)
    assert e.value.status == -4


def test_mlp_step_with_odd_layer_sizes(pkg, cuda, oracle):
    """Layers whose weight count is not a multiple of 8 leave the bias gradient at an odd offset of the
    layer's bucket; the step must still run, fused and unfused, and match the oracle."""
    torch = cuda
    sizes, batch, rate = (10, 7, 3), 12, 1e-2
    ws = [oracle.to_bf16(0.5 * oracle.normal((sizes[i], sizes[i + 1]), 150 + i)) for i in range(2)]
    bs = [oracle.to_bf16(0.1 * oracle.normal((sizes[i + 1],), 160 + i)) for i in range(2)]
    x = oracle.to_bf16(oracle.normal((batch, sizes[0]), 170))
    y = oracle.to_bf16(oracle.normal((batch, sizes[-1]), 171))
    loss_ref, _, _, _, w_ref, b_ref, _, _ = oracle.mlp_step(ws, bs, x, y, rate)
    for fuse in (False, True):
        step = pkg.mlp.MLPStep(torch, sizes, batch, rate, weights=[dev(torch, w) for w in ws],
                               biases=[dev(torch, b) for b in bs], fuse_update=fuse)
        loss = step.step(dev(torch, x), dev(torch, y))
        step.check()
        assert abs(loss.item() - loss_ref) <= 2e-3 * abs(loss_ref)
        for i in range(2):
            close_bf16(oracle, host(torch, step.w[i]), oracle.from_bf16(w_ref[i]), 1)
            close_bf16(oracle, host(torch, step.b[i]), oracle.from_bf16(b_ref[i]), 1)


def test_layernorm_backward_without_eps_and_with_empty_row_slots(pkg, cuda, oracle):
    """eps = 0 and a row count that leaves some of a block's row slots empty: the empty slots must add
    nothing (not 0 * inf) to dgamma / dbeta."""
    torch, L = cuda, pkg.lib
    for rows, n in ((7, 256), (13, 64), (3, 1024), (5, 4096)):
        x = oracle.normal((rows, n), 40 + rows)
        g = oracle.normal((rows, n), 41 + rows)
        w = (1 + 0.1 * oracle.normal((n,), 42)).astype(np.float32)
        dx_ref, dw_ref, db_ref = oracle.layernorm_bwd(x, w, g, eps=0.0)
        xd, gd, wd = (torch.from_numpy(a).cuda() for a in (x, g, w))
        dx, dw, db = torch.empty_like(xd), torch.empty_like(wd), torch.empty_like(wd)
        need = L.rowop_workspace_bytes(L.LAYERNORM_BWD, n, rows, L.F32)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        L.layernorm_bwd(xd.data_ptr(), wd.data_ptr(), gd.data_ptr(), 0, 0, dx.data_ptr(), dw.data_ptr(), db.data_ptr(),
                        0.0, n, rows, n, L.F32, ws.data_ptr(), need)
        torch.cuda.synchronize()
        assert torch.isfinite(dw).all() and torch.isfinite(db).all() and torch.isfinite(dx).all()
        agree(dx.cpu().numpy(), dx_ref, 1e-5)
        agree(dw.cpu().numpy(), dw_ref, 1e-5)
        agree(db.cpu().numpy(), db_ref, 1e-5)


@pytest.mark.parametrize("count,M,N,K,a_mn,b_mn", [
    (37, 64, 64, 128, True, False),    # the delta rule's per-chunk products, scattered in memory
    (37, 64, 64, 128, False, True),
    (5, 50, 70, 100, False, False),    # extents that are not multiples of the tile, every layout
    (5, 50, 70, 100, True, True),
    (3, 130, 200, 72, True, False),
    (3, 130, 200, 72, False, True),
])
def test_products_by_arrays_of_addresses(pkg, cuda, oracle, count, M, N, K, a_mn, b_mn):
    """tb200_gemm_pointers (the reference's `Products`, ext/cuBLASExt.jl:273-306): members anywhere in memory, in any
    order, some off a 16-byte boundary; BFloat16 on the warp-level MMAs and on the generic kernel, Float32 results
    against the oracle's Float32 product."""
    torch, L = cuda, pkg.lib
    A, B = batch_operands(oracle, count, M, N, K, a_mn, b_mn, 9100 + M + K)
    want = np.stack([oracle.gemm(A[i], B[i], M=M, N=N, K=K, a_km=a_mn, b_kn=b_mn, want_pre=True)[1] for i in range(count)])
    # members laid out in reverse order with gaps; every third one starts two elements off alignment
    gap = 24
    a_len, b_len = A[0].size, B[0].size
    pool_a = torch.zeros(count * (a_len + gap) + 8, device="cuda", dtype=torch.bfloat16)
    pool_b = torch.zeros(count * (b_len + gap) + 8, device="cuda", dtype=torch.bfloat16)
    pool_c = torch.full((count * (M * N + gap) + 8,), float("nan"), device="cuda")
    pa, pb, pc, views = [], [], [], []
    for i in range(count):
        j = count - 1 - i
        off = 2 if i % 3 == 1 else 0
        va = pool_a[j * (a_len + gap) + off: j * (a_len + gap) + off + a_len]
        vb = pool_b[j * (b_len + gap) + off: j * (b_len + gap) + off + b_len]
        vc = pool_c[j * (M * N + gap): j * (M * N + gap) + M * N]
        va.copy_(dev(torch, A[i]).reshape(-1))
        vb.copy_(dev(torch, B[i]).reshape(-1))
        pa.append(va.data_ptr()); pb.append(vb.data_ptr()); pc.append(vc.data_ptr()); views.append(vc)
    ptrs = [torch.tensor(p, dtype=torch.int64, device="cuda") for p in (pa, pb, pc)]
    for force_simt in (False, True):
        pool_c.fill_(float("nan"))
        d = L.gemm_desc(M, N, K, a_layout=int(a_mn), b_layout=int(b_mn), out_dtype=L.F32, force_simt=force_simt)
        L.gemm_pointers(d, ptrs[0].data_ptr(), ptrs[1].data_ptr(), ptrs[2].data_ptr(), count)
        torch.cuda.synchronize()
        got = np.stack([v.view(M, N).cpu().numpy() for v in views])
        agree(got, want, 1e-5)
    # BFloat16 results, rounded once
    outs = torch.full((count, M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    pc16 = torch.tensor([outs[i].data_ptr() for i in range(count)], dtype=torch.int64, device="cuda")
    L.gemm_pointers(L.gemm_desc(M, N, K, a_layout=int(a_mn), b_layout=int(b_mn)), ptrs[0].data_ptr(), ptrs[1].data_ptr(),
                    pc16.data_ptr(), count)
    torch.cuda.synchronize()
    close_bf16(oracle, host(torch, outs), want, K)


def test_products_by_addresses_other_types_and_refusals(pkg, cuda, oracle):
    torch, L = cuda, pkg.lib
    count, M, N, K = 4, 40, 56, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    A32 = torch.randn(count, M, K, device="cuda", generator=g)
    B32 = torch.randn(count, N, K, device="cuda", generator=g)          # K-major B: [n][k]
    want = torch.einsum("bmk,bnk->bmn", A32.double(), B32.double())
    for dt, code, tol in ((torch.float32, L.F32, 1e-5), (torch.float16, L.F16, 2e-3)):
        Ad, Bd = A32.to(dt), B32.to(dt)
        ref = torch.einsum("bmk,bnk->bmn", Ad.double(), Bd.double())
        C = torch.full((count, M, N), float("nan"), device="cuda")
        mk = lambda t: torch.tensor([t[i].data_ptr() for i in range(count)], dtype=torch.int64, device="cuda")  # noqa: E731
        pa, pb, pc = mk(Ad), mk(Bd), mk(C)
        L.gemm_pointers(L.gemm_desc(M, N, K, a_layout=L.K_MAJOR, b_layout=L.K_MAJOR, in_dtype=code, out_dtype=L.F32),
                        pa.data_ptr(), pb.data_ptr(), pc.data_ptr(), count)
        torch.cuda.synchronize()
        assert ((C.double() - ref).norm() / ref.norm()).item() <= tol
    assert want.shape == (count, M, N)
    d = L.gemm_desc(M, N, K, epilogue=L.EPI_BIAS)
    with pytest.raises(L.TB200Error) as e:      # plain products only
        L.gemm_pointers(d, pa.data_ptr(), pb.data_ptr(), pc.data_ptr(), count)
    assert e.value.status == -7
    with pytest.raises(L.TB200Error) as e:      # a missing array
        L.gemm_pointers(L.gemm_desc(M, N, K), 0, pb.data_ptr(), pc.data_ptr(), count)
    assert e.value.status == -1
    L.gemm_pointers(L.gemm_desc(M, N, K), 0, 0, 0, 0)   # nothing to do
