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
    for rows, n in ((3000, 4096), (517, 1000), (64, 8192), (3000, 4096)):
        x = torch.randn(rows, n, device="cuda", generator=gen).to(dt)
        g = torch.randn(rows, n, device="cuda", generator=gen).to(dt)
        w = (1 + 0.25 * torch.randn(n, device="cuda", generator=gen)).to(dt)
        need = L.rowop_workspace_bytes(L.LAYERNORM_BWD, n, rows, code)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        dx0, dw0, db0 = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
        L.layernorm_bwd(x.data_ptr(), w.data_ptr(), g.data_ptr(), 0, 0, dx0.data_ptr(), dw0.data_ptr(),
                        db0.data_ptr(), 1e-5, n, rows, n, code, ws.data_ptr(), need, stream)
        for _ in range(2):
            dx1, dw1, db1 = torch.full_like(x, 7.0), torch.full_like(w, 7.0), torch.full_like(w, 7.0)
            L.layernorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), g.data_ptr(), 0, 0, dx1.data_ptr(), dw1.data_ptr(),
                                    db1.data_ptr(), 1e-5, n, rows, n, code, stream)
            torch.cuda.synchronize()
            # dx does not involve the scratch: identical.  dgamma/dbeta: the same Float32 partial sums,
            # possibly grouped into fewer blocks, so equal to the tests' Float32 tolerance (one BFloat16
            # ulp where the result is rounded to BFloat16)
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
