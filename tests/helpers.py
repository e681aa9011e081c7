"""Shared pieces of the tests: tolerances as the reference states them, and the
glue that runs one template of the backend on numpy inputs through the
`implement` mirror (Binding -> build -> launch), i.e. through the C ABI."""
import numpy as np

# Float32 pointwise / reduction work: 1e-5 relative, measured as the reference's
# `agree` does (test/setup.jl:41-42): isapprox on the arrays' norms with
# atol = rtol * 1e-2 -- plus an elementwise bound so that no single element hides.
RTOL_F32 = 1.0e-5
# BFloat16 results against the Float32 CPU reference: 2e-2 max-abs, or one
# BFloat16 ulp of the reference value where that is larger (values >= 4).
ATOL_BF16 = 2.0e-2


def agree(got, want, rtol=RTOL_F32):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if got.size == 0:
        return
    assert np.isfinite(got).all() == np.isfinite(want).all()
    diff = np.linalg.norm(got - want)
    bound = max(rtol * 1.0e-2, rtol * max(np.linalg.norm(got), np.linalg.norm(want)))
    assert diff <= bound, f"norm of difference {diff:.3e} > {bound:.3e}"
    worst = np.abs(got - want).max()
    scale = max(np.abs(want).max(), 1e-30)
    assert worst <= 20 * rtol * scale, f"largest element difference {worst:.3e} vs scale {scale:.3e}"


def agree_bf16(got_bits, want_f32, oracle, atol=ATOL_BF16):
    got = oracle.from_bf16(got_bits).astype(np.float64)
    want = np.asarray(want_f32, np.float64)
    assert got.shape == want.shape
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
    tol = np.maximum(atol, ulp)
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{bad.sum()} elements beyond tolerance, worst {np.abs(got - want).max():.3e}"


class Runner:
    """Runs the backend's templates on numpy arrays, Julia layout: a Julia
    (n, rows) matrix is a numpy [rows][n] array."""

    def __init__(self, pkg, torch):
        self.pkg, self.torch = pkg, torch
        self.I = pkg.implement
        self.lib = self.I.B200Kernels()
        self.target = self.I.Target()
        self.resources = self.lib.resources(self.target)

    def dev(self, a):
        t = self.torch.from_numpy(np.ascontiguousarray(a))
        if a.dtype == np.uint16:
            t = t.view(self.torch.bfloat16)
        return t.cuda()

    def host(self, t):
        if t.dtype == self.torch.bfloat16:
            return t.view(self.torch.uint16).cpu().numpy() if hasattr(self.torch, "uint16") else \
                t.view(self.torch.int16).cpu().numpy().view(np.uint16)
        return t.cpu().numpy()

    @staticmethod
    def eltype(a):
        return "BFloat16" if a.dtype == np.uint16 else "Float32"

    def run(self, template, extents, arrays):
        b = self.I.Binding(template, extents, arrays)
        assert self.lib.supports(self.target, b)
        launch, description = self.lib.build(self.target, b, self.resources)
        launch()
        self.torch.cuda.synchronize()
        return launch, description

    def softmax(self, x, want_lse=True, stat="Float32"):
        rows, n = x.shape
        e = self.eltype(x)
        xd = self.dev(x)
        y = self.torch.empty_like(xd)
        arrays = {"x": self.I.dense_columns(xd, e, n, rows, 1), "y": self.I.dense_columns(y, e, n, rows, 2)}
        lse = None
        if want_lse:
            lse = self.torch.empty(rows, device="cuda",
                                   dtype=self.torch.float32 if stat == "Float32" else self.torch.bfloat16)
            arrays["lse"] = self.I.Strided(stat, 0, (1, rows), (1, 1), lse, 3)
        self.run("softmax_columns_lse" if want_lse else "softmax_columns", {"n": n, "rows": rows}, arrays)
        return self.host(y), (self.host(lse) if lse is not None else None)

    def softmax_pullback(self, y, g):
        rows, n = y.shape
        e = self.eltype(y)
        yd, gd = self.dev(y), self.dev(g)
        dx = self.torch.empty_like(yd)
        self.run("softmax_columns_pullback", {"n": n, "rows": rows},
                 {"y": self.I.dense_columns(yd, e, n, rows, 1), "g": self.I.dense_columns(gd, e, n, rows, 2),
                  "dx": self.I.dense_columns(dx, e, n, rows, 3)})
        return self.host(dx)

    def softmax_pullback_recomputed(self, x, lse, g):
        rows, n = x.shape
        e = self.eltype(x)
        xd, gd, ld = self.dev(x), self.dev(g), self.dev(lse)
        dx = self.torch.empty_like(xd)
        self.run("softmax_columns_pullback_recomputed", {"n": n, "rows": rows},
                 {"x": self.I.dense_columns(xd, e, n, rows, 1), "g": self.I.dense_columns(gd, e, n, rows, 2),
                  "lse": self.I.Strided("Float32", 0, (1, rows), (1, 1), ld, 4),
                  "dx": self.I.dense_columns(dx, e, n, rows, 3)})
        return self.host(dx)

    def layernorm(self, x, w, b=None, stats=False):
        rows, n = x.shape
        e = self.eltype(x)
        xd, wd = self.dev(x), self.dev(w)
        y = self.torch.empty_like(xd)
        arrays = {"x": self.I.dense_columns(xd, e, n, rows, 1), "w": self.I.dense_vector(wd, e, n, 2),
                  "y": self.I.dense_columns(y, e, n, rows, 3)}
        if b is not None:
            arrays["b"] = self.I.dense_vector(self.dev(b), e, n, 4)
        mean = rstd = None
        if stats:
            mean, rstd = self.torch.empty(rows, device="cuda"), self.torch.empty(rows, device="cuda")
            arrays["mean"] = self.I.Strided("Float32", 0, (1, rows), (1, 1), mean, 5)
            arrays["rstd"] = self.I.Strided("Float32", 0, (1, rows), (1, 1), rstd, 6)
        self.run("layernorm_bias" if b is not None else "layernorm", {"n": n, "rows": rows}, arrays)
        if stats:
            return self.host(y), self.host(mean), self.host(rstd)
        return self.host(y)

    def layernorm_pullback(self, x, w, g, mean=None, rstd=None):
        rows, n = x.shape
        e = self.eltype(x)
        xd, wd, gd = self.dev(x), self.dev(w), self.dev(g)
        dx, dw, db = self.torch.empty_like(xd), self.torch.empty_like(wd), self.torch.empty_like(wd)
        arrays = {"x": self.I.dense_columns(xd, e, n, rows, 1), "w": self.I.dense_vector(wd, e, n, 2),
                  "g": self.I.dense_columns(gd, e, n, rows, 3), "dx": self.I.dense_columns(dx, e, n, rows, 4),
                  "dw": self.I.dense_vector(dw, e, n, 5), "db": self.I.dense_vector(db, e, n, 6)}
        if mean is not None:
            arrays["mean"] = self.I.Strided("Float32", 0, (1, rows), (1, 1), self.dev(mean), 7)
            arrays["rstd"] = self.I.Strided("Float32", 0, (1, rows), (1, 1), self.dev(rstd), 8)
        self.run("layernorm_pullback", {"n": n, "rows": rows}, arrays)
        return self.host(dx), self.host(dw), self.host(db)
