"""The LayerNorm backward entry point that takes no workspace.

Some callers cannot bring scratch memory: every device buffer they own was
laid out before the kernels were picked, and nothing at call time can allocate
(or may touch the driver's allocator).  For them the library carries a fixed
8 MiB array and `tb200_layernorm_bwd_noalloc` uses it.  This file checks,
through the C ABI, that it returns what `tb200_layernorm_bwd` returns on two
calls in a row (the array keeps the first call's contents), that it refuses
rows beyond its stated limit, and that it works whether it is the first thing
the process runs or the last.  It is named to be collected after every other
test file.
"""
import numpy as np
import pytest

from helpers import RTOL_F32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("eltype", ["Float32", "BFloat16"])
def test_matches_the_workspace_entry_point_twice(pkg, cuda, eltype):
    torch, L = cuda, pkg.lib
    stream = torch.cuda.current_stream().cuda_stream
    dt = torch.float32 if eltype == "Float32" else torch.bfloat16
    code = L.F32 if eltype == "Float32" else L.BF16
    gen = torch.Generator(device="cuda").manual_seed(31)
    # two different shapes back to back: the second call finds the first one's partial sums in the array
    # (3000, 8192): more row groups than the built-in array has partial rows for, so the grid is cut to
    # what fits and each block walks more rows; `saved`: the forward's mean and rstd handed in
    for rows, n, saved in ((3000, 4096, False), (517, 1000, False), (64, 8192, True), (3000, 8192, False),
                           (3000, 4096, True)):
        x = torch.randn(rows, n, device="cuda", generator=gen).to(dt)
        g = torch.randn(rows, n, device="cuda", generator=gen).to(dt)
        w = (1 + 0.25 * torch.randn(n, device="cuda", generator=gen)).to(dt)
        mean = rstd = None
        if saved:
            mean = x.float().mean(dim=1)
            rstd = torch.rsqrt(x.float().var(dim=1, unbiased=False) + 1e-5)
        mp, rp = (mean.data_ptr(), rstd.data_ptr()) if saved else (0, 0)
        need = L.rowop_workspace_bytes(L.LAYERNORM_BWD, n, rows, code)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        dx0, dw0, db0 = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
        L.layernorm_bwd(x.data_ptr(), w.data_ptr(), g.data_ptr(), mp, rp, dx0.data_ptr(), dw0.data_ptr(),
                        db0.data_ptr(), 1e-5, n, rows, n, code, ws.data_ptr(), need, stream)
        for _ in range(2):
            dx1, dw1, db1 = torch.full_like(x, 7.0), torch.full_like(w, 7.0), torch.full_like(w, 7.0)
            L.layernorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), g.data_ptr(), mp, rp, dx1.data_ptr(), dw1.data_ptr(),
                                    db1.data_ptr(), 1e-5, n, rows, n, code, stream)
            torch.cuda.synchronize()
            # dx does not involve the scratch: identical where both entries run the same kernel (with saved
            # statistics the workspace entry has kernels of its own, whose row sums group differently: one
            # BFloat16 ulp, or Float32 rounding).  dgamma/dbeta: the same Float32 partial sums,
            # possibly grouped into fewer blocks, so equal to the tests' Float32 tolerance (one BFloat16
            # ulp where the result is rounded to BFloat16)
            if saved and eltype == "BFloat16":
                assert ((dx1.double() - dx0.double()).abs() <= 2 ** -7 * dx0.double().abs() + 2e-2).all()
            elif saved:
                assert ((dx1.double() - dx0.double()).abs() <= 1e-5 * dx0.double().abs() + 1e-5).all()
            else:
                assert torch.equal(dx1, dx0)
            for got, want in ((dw1, dw0), (db1, db0)):
                got, want = got.double(), want.double()
                if eltype == "Float32":
                    assert (got - want).norm() <= RTOL_F32 * want.norm()
                else:
                    assert ((got - want).abs() <= 2 ** -7 * want.abs() + 1e-4).all()


def test_refuses_rows_beyond_its_limit(pkg, cuda):
    torch, L = cuda, pkg.lib
    limit = L.layernorm_bwd_noalloc_max_row()
    assert limit == 8192
    n, rows = limit + 8, 4
    x = torch.randn(rows, n, device="cuda")
    w = torch.ones(n, device="cuda")
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    with pytest.raises(L.TB200Error) as e:
        L.layernorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), x.data_ptr(), 0, 0, dx.data_ptr(), dw.data_ptr(),
                                db.data_ptr(), 1e-5, n, rows, n, L.F32)
    assert e.value.status == -5
    # and the context is fine afterwards
    n = 256
    x = torch.randn(rows, n, device="cuda")
    w = torch.ones(n, device="cuda")
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    L.layernorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), x.data_ptr(), 0, 0, dx.data_ptr(), dw.data_ptr(),
                            db.data_ptr(), 1e-5, n, rows, n, L.F32)
    torch.cuda.synchronize()
    assert torch.isfinite(dx).all() and torch.isfinite(dw).all()


def test_rows_that_cannot_be_read_in_vectors(pkg, cuda):
    """Rows whose length or addresses rule out 128-bit accesses: up to 4096 elements they give the workspace
    entry's results; beyond that they do not fit one block's registers and are refused, as the header says."""
    torch, L = cuda, pkg.lib
    stream = torch.cuda.current_stream().cuda_stream
    rows, n = 40, 4001                                   # an odd length: one element at a time
    x, g = torch.randn(rows, n, device="cuda"), torch.randn(rows, n, device="cuda")
    w = 1 + 0.25 * torch.randn(n, device="cuda")
    need = L.rowop_workspace_bytes(L.LAYERNORM_BWD, n, rows, L.F32)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    dx0, dw0, db0 = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    L.layernorm_bwd(x.data_ptr(), w.data_ptr(), g.data_ptr(), 0, 0, dx0.data_ptr(), dw0.data_ptr(), db0.data_ptr(),
                    1e-5, n, rows, n, L.F32, ws.data_ptr(), need, stream)
    for _ in range(2):
        dx1, dw1, db1 = torch.full_like(x, 7.0), torch.full_like(w, 7.0), torch.full_like(w, 7.0)
        L.layernorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), g.data_ptr(), 0, 0, dx1.data_ptr(), dw1.data_ptr(),
                                db1.data_ptr(), 1e-5, n, rows, n, L.F32, stream)
        torch.cuda.synchronize()
        assert torch.equal(dx1, dx0)
        for got, want in ((dw1, dw0), (db1, db0)):
            assert (got.double() - want.double()).norm() <= RTOL_F32 * want.double().norm()
    n = 5001                                             # odd and longer than 4096: refused
    x = torch.randn(4, n, device="cuda")
    w = torch.ones(n, device="cuda")
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    with pytest.raises(L.TB200Error) as e:
        L.layernorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), x.data_ptr(), 0, 0, dx.data_ptr(), dw.data_ptr(),
                                db.data_ptr(), 1e-5, n, 4, n, L.F32)
    assert e.value.status == -5
    # an even length from an address that is not 16-byte aligned: same rule
    base = torch.randn(4 * 6000 + 1, device="cuda")
    with pytest.raises(L.TB200Error) as e:
        L.layernorm_bwd_noalloc(base.data_ptr() + 4, w.data_ptr(), x.data_ptr(), 0, 0, dx.data_ptr(), dw.data_ptr(),
                                db.data_ptr(), 1e-5, 5000, 4, 6000, L.F32)
    assert e.value.status == -5
