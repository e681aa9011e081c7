"""The benchmark's MLP training step at its full size -- 4 Dense layers 1024 -> 4096 -> 4096 -> 4096 -> 1024,
GELU(tanh), bias, BFloat16, batch 8192, MSE, SGD 1e-3 (examples/mlp.jl:13-35 with test/fixtures/programs.jl:19) --
through the C ABI against the oracle's restatement of the same step from the same BFloat16 inputs: the loss,
every layer's activations and pullback, the bias and weight gradients and the updated parameters."""
import numpy as np
import pytest

from helpers import ATOL_BF16
from test_gemm_gpu import dev, host

pytestmark = pytest.mark.gpu

SIZES, BATCH, RATE = (1024, 4096, 4096, 4096, 1024), 8192, 1e-3


def inputs(oracle):
    rng = np.random.Generator(np.random.Philox(20261127))
    ws = []
    for i in range(4):
        fin, fout = SIZES[i], SIZES[i + 1]
        limit = (6.0 / (fin + fout)) ** 0.5                      # Glorot-uniform, stored [in][out]
        ws.append(oracle.to_bf16((rng.random((fin, fout), dtype=np.float32) * 2 - 1) * limit))
    # the benchmark starts from zero biases; small non-zero ones here so that a wrong bias path shows
    bs = [oracle.to_bf16(0.05 * oracle.normal((SIZES[i + 1],), 300 + i)) for i in range(4)]
    x = oracle.to_bf16(oracle.normal((BATCH, SIZES[0]), 310))
    y = oracle.to_bf16(oracle.normal((BATCH, SIZES[-1]), 311))
    return ws, bs, x, y


def close(oracle, got_bits, want, what, rel=1e-2):
    """BFloat16 result against the Float32 restatement: 2e-2 max-abs scaled by the array's magnitude where that
    exceeds 1, and 1e-2 norm-wise."""
    got = oracle.from_bf16(got_bits).astype(np.float64)
    want = np.asarray(want, np.float64)
    scale = max(1.0, np.abs(want).max())
    worst = np.abs(got - want).max()
    assert worst <= ATOL_BF16 * scale, f"{what}: max-abs {worst:.3e} vs {ATOL_BF16 * scale:.3e}"
    assert np.linalg.norm(got - want) <= rel * np.linalg.norm(want), what


def test_full_size_step(pkg, cuda, oracle):
    torch = cuda
    ws, bs, x, y = inputs(oracle)
    loss_ref, dz_ref, dw_ref, db_ref, w_ref, b_ref, a_ref, z_ref = oracle.mlp_step_blas(ws, bs, x, y, RATE)
    xd, yd = dev(torch, x), dev(torch, y)
    rows = np.array([0, 1, 777, 4095, 4096, 8191])
    for fuse in (True, False):
        step = pkg.mlp.MLPStep(torch, SIZES, BATCH, RATE, weights=[dev(torch, w) for w in ws],
                               biases=[dev(torch, b) for b in bs], fuse_update=fuse)
        loss = step.step(xd, yd)
        step.check()
        assert abs(loss.item() - loss_ref) <= 2e-3 * abs(loss_ref), (loss.item(), loss_ref)
        for i in range(4):
            fin, fout = SIZES[i], SIZES[i + 1]
            cols = np.array([0, 5, fout // 2, fout - 1])
            # the forward's activations and the value the activation saw: sampled rows, and whole-array norms
            a_got, a_want = host(torch, step.a[i + 1]), oracle.from_bf16(a_ref[i + 1])
            close(oracle, a_got[rows], a_want[rows], f"a[{i + 1}] rows")
            close(oracle, a_got, a_want, f"a[{i + 1}]")
            if step.z[i] is not None:
                close(oracle, host(torch, step.z[i])[rows], oracle.from_bf16(z_ref[i])[rows], f"z[{i}] rows")
            # the pullback dz: sampled rows and columns at its own scale (its values are ~1e-4), whole-array norm
            dz_got, dz_want = oracle.from_bf16(host(torch, step.dz[i])).astype(np.float64), oracle.from_bf16(dz_ref[i])
            scale = np.abs(dz_want).max()
            assert np.abs(dz_got[rows] - dz_want[rows]).max() <= ATOL_BF16 * scale, f"dz[{i}] rows"
            assert np.abs(dz_got[:, cols] - dz_want[:, cols]).max() <= ATOL_BF16 * scale, f"dz[{i}] columns"
            assert np.linalg.norm(dz_got - dz_want) <= 1e-2 * np.linalg.norm(dz_want), f"dz[{i}]"
            # the bias gradient, whole
            db_got = oracle.from_bf16(host(torch, step.db[i])).astype(np.float64)
            assert np.abs(db_got - db_ref[i]).max() <= ATOL_BF16 * max(np.abs(db_ref[i]).max(), 1e-30), f"db[{i}]"
            if not fuse:
                # the weight gradient as the data-parallel form keeps it (BFloat16, before any exchange)
                dw_got = oracle.from_bf16(host(torch, step.dw[i])).astype(np.float64)
                wrows = np.array([0, 3, fin // 2, fin - 1])
                scale = np.abs(dw_ref[i]).max()
                assert np.abs(dw_got[wrows] - dw_ref[i][wrows]).max() <= ATOL_BF16 * scale, f"dw[{i}] rows"
                assert np.abs(dw_got[:, cols] - dw_ref[i][:, cols]).max() <= ATOL_BF16 * scale, f"dw[{i}] columns"
                assert np.linalg.norm(dw_got - dw_ref[i]) <= 5e-3 * np.linalg.norm(dw_ref[i]), f"dw[{i}]"
            # the updated parameters: the step w - rate * dw is below one BFloat16 ulp of most weights, so they are
            # compared at the weight's own precision -- at most one BFloat16 ulp apart (or, for weights so close
            # to zero that the update itself decides their value, 2 % of the largest update) and almost
            # everywhere identical
            for name, got_t, want_bits, grad in (("w", step.w[i], w_ref[i], dw_ref[i]), ("b", step.b[i], b_ref[i], db_ref[i])):
                got_bits = host(torch, got_t)
                got, want = oracle.from_bf16(got_bits).astype(np.float64), oracle.from_bf16(want_bits).astype(np.float64)
                bound = 2.0 ** -7 * np.abs(want) + ATOL_BF16 * RATE * np.abs(grad).max()
                worst = (np.abs(got - want) - bound).max()
                assert worst <= 0, f"{name}[{i}] is {worst:.3e} beyond one BFloat16 ulp"
                # the fused update rounds w - rate * dw once; the unfused one rounds dw first, so a few more
                # weights land on the other side of a rounding boundary
                differing = (got_bits != want_bits).mean()
                assert differing <= (0.01 if fuse else 0.03), f"{name}[{i}]: {differing:.4f} of the entries differ"
        del step
