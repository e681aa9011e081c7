"""Host logic of the plugin mirror (no GPU): templates, supports, estimate, build errors."""
import pytest


@pytest.fixture()
def I(pkg):
    return pkg.implement


def binding(I, template="softmax_columns", n=4096, rows=8, eltype="Float32", **over):
    arrays = {"x": I.dense_columns(None, eltype, n, rows, 1), "y": I.dense_columns(None, eltype, n, rows, 2)}
    arrays.update(over)
    return I.Binding(template, {"n": n, "rows": rows}, arrays)


def test_templates_follow_the_target(I):
    lib = I.B200Kernels()
    names = [t.name for t in lib.templates(I.Target(online=True))]
    assert "softmax_columns" in names and "layernorm_pullback" in names
    # a target that keeps the two passes is offered no one-pass fold (ext/cuDNNExt.jl:60-62), only products and scans
    kept = [t.name for t in lib.templates(I.Target(online=False))]
    assert kept and all(n.startswith("linear") or "_dims" in n for n in kept)


def test_supports(I):
    lib, t = I.B200Kernels(), I.Target()
    assert lib.supports(t, binding(I))
    assert lib.supports(t, binding(I, eltype="BFloat16"))
    assert not lib.supports(t, binding(I, template="attention"))
    assert not lib.supports(t, binding(I, y=I.dense_columns(None, "BFloat16", 4096, 8, 2)))  # mixed types
    strided = I.Strided("Float32", 0, (4096, 8), (2, 8192), None, 2)
    assert not lib.supports(t, binding(I, y=strided))  # folded axis not contiguous
    other_ld = I.dense_columns(None, "Float32", 4096, 8, 2, ld=4100)
    assert not lib.supports(t, binding(I, y=other_ld))  # two leading dimensions
    both = binding(I, x=I.dense_columns(None, "Float32", 4096, 8, 1, ld=4100), y=other_ld)
    assert lib.supports(t, both)


def test_estimate_counts_algorithmic_bytes(I):
    lib, t = I.B200Kernels(), I.Target()
    (w,) = lib.estimate(t, binding(I, n=4096, rows=65536))
    assert w.bytes == 2 * 4096 * 65536 * 4 and w.launches == 1
    (w,) = lib.estimate(t, binding(I, template="softmax_columns_pullback", n=4096, rows=65536, eltype="BFloat16"))
    assert w.bytes == 3 * 4096 * 65536 * 2
    (w,) = lib.estimate(t, binding(I, n=40000, rows=4))
    assert w.launches == 2


def test_build_refuses_without_buffers(I):
    lib, t = I.B200Kernels(), I.Target()
    with pytest.raises(ValueError):
        lib.build(t, binding(I))
    with pytest.raises(ValueError):
        lib.build(t, binding(I, template="attention"))


def test_strided_pointer_and_repoint(I):
    s = I.Strided("BFloat16", 8, (16, 4), (1, 16), 4096, 3)
    assert s.pointer() == 4096 + 16
    b = I.Binding("softmax_columns", {"n": 16, "rows": 4}, {"x": s, "y": I.Strided("BFloat16", 0, (16, 4), (1, 16), 8192, 4)})
    launch = I.RowLaunch(b, 1e-5, None, 0)
    assert launch.repoints()
    launch.repoint(3, 65536)
    assert b.arrays["x"].pointer() == 65536 + 16 and b.arrays["y"].pointer() == 8192


def test_row_type_ignores_statistics_listed_first(I):
    """A Float32 statistic ahead of BFloat16 rows in the binding must not decide the kernels' element type
    (nor the workspace size or the byte count)."""
    rows, n = 8, 4096
    stat = lambda v: I.Strided("Float32", 0, (1, rows), (1, 1), 1 << 20, v)  # noqa: E731
    arrays = {"mean": stat(7), "rstd": stat(8)}
    for i, name in enumerate(("x", "g", "dx")):
        arrays[name] = I.dense_columns(4096 * (i + 1), "BFloat16", n, rows, i + 1)
    for i, name in enumerate(("w", "dw", "db")):
        arrays[name] = I.dense_vector(1 << 16, "BFloat16", n, 4 + i)
    b = I.Binding("layernorm_pullback", {"n": n, "rows": rows}, arrays)
    lib, t = I.B200Kernels(), I.Target()
    assert lib.supports(t, b)
    assert I.row_eltype(b) == "BFloat16"
    assert I.RowLaunch(b, 1e-5, None, 0).dtype == 1            # TB200_BF16
    (w,) = lib.estimate(t, b)
    assert w.bytes == 3 * n * rows * 2
    lse_first = I.Binding("softmax_columns_lse", {"n": n, "rows": rows},
                          {"lse": stat(3), "x": arrays["x"], "y": arrays["dx"]})
    assert I.RowLaunch(lse_first, 1e-5, None, 0).dtype == 1


def test_product_and_attention_templates(I):
    lib, t = I.B200Kernels(), I.Target()
    names = [x.name for x in lib.templates(t)]
    assert "linear_bias_gelu" in names and "attention_causal_lse" in names and "attention_causal_pullback" in names
    # products do not depend on the online rewrites; attention does
    off = [x.name for x in lib.templates(I.Target(online=False))]
    assert "linear" in off and not any(n.startswith("attention") for n in off)
    b = I.Binding("linear_bias_gelu", {"m": 4096, "k": 1024, "n": 8192},
                  {"w": I.dense_matrix(None, "BFloat16", 4096, 1024, 1), "x": I.dense_matrix(None, "BFloat16", 1024, 8192, 2),
                   "b": I.dense_vector(None, "BFloat16", 4096, 3), "y": I.dense_matrix(None, "BFloat16", 4096, 8192, 4)})
    assert lib.supports(t, b)
    (w,) = lib.estimate(t, b)
    assert w.flops == 2.0 * 4096 * 8192 * 1024
    # the rest of the cost statement (src/Compiler/Implement/Implement.jl:30-82): 8192 x 4096 results in 256 x 256
    # tiles by pairs of CTAs, each tile row fetching w again and each tile column x, 16 steps of 64 along k
    assert w.factor == "BFloat16" and w.blocks == 32 * 16 and w.steps == 16 and not w.split
    assert w.reread == 2 * (4096 * 1024 * 31 + 1024 * 8192 * 15)
    e = {"d": 128, "h": 32, "hk": 32, "m": 4096, "n": 4096, "b": 8}
    arrays = {n: I.dense_heads(None, "BFloat16", 128, 32, 4096, 8, i) for i, n in enumerate(("q", "k", "v", "o"))}
    a = I.Binding("attention_causal", e, arrays)
    assert lib.supports(t, a)
    (w,) = lib.estimate(t, a)
    assert abs(w.flops - 1.0995e12) / 1.0995e12 < 1e-3
    # the scores are a fold recomputed inside the products: half the flops; 32 query tiles x 32 heads x 8, each
    # sweeping on average half of the 32 key tiles
    assert w.recomputed == 0.5 * w.flops and w.blocks == 32 * 32 * 8 and w.steps == 16 and w.factor == "BFloat16"
    pull = I.Binding("attention_causal_pullback", e, arrays)
    (wp,) = lib.estimate(t, pull)
    assert wp.flops == 2.5 * w.flops and wp.passed == 2 * 4 * 128 * 32 * 4096 * 8 and wp.launches == 3
    # the forward builds without touching the device (addresses stand in for buffers); its description names the kernels
    at = lambda d: {n: I.dense_heads(4096 * (i + 1), "BFloat16", d, 32, 4096, 8, i) for i, n in enumerate(("q", "k", "v", "o"))}  # noqa: E731
    assert lib.build(t, I.Binding("attention_causal", e, at(128)))[1].endswith("tensor cores, two query tiles a block")
    assert lib.build(t, I.Binding("attention_causal", dict(e, d=64), at(64)))[1].endswith("CUDA-core kernels")
    assert lib.supports(t, I.Binding("attention_causal", dict(e, d=64), arrays))      # CUDA-core path
    assert not lib.supports(t, I.Binding("attention_causal", dict(e, d=512), arrays))
    assert not lib.supports(t, I.Binding("attention_causal", dict(e, n=2048), arrays))
    strided = dict(arrays, q=I.Strided("BFloat16", 0, (128, 32, 4096, 8), (1, 256, 8192, 1 << 25), None, 0))
    assert not lib.supports(t, I.Binding("attention_causal", e, strided))


def test_generator_claims_groups(pkg):
    """The `Implementation` door: claims, estimate and the descriptor checks, without a device."""
    I, G = pkg.implement, pkg.groups
    gen, t = I.B200Generator(), I.Target()
    g = G.layernorm(4096, 65536, "BFloat16", two_pass=True)
    claims = gen.claims(t, g)
    claim = claims[-1]                                   # the interpreter is always offered, last
    assert claim.threads == 256 and claim.phases == 3 and not claim.compiled
    assert all(c.compiled for c in claims[:-1])         # the compiled kernel first, when NVRTC is at hand
    (w,) = gen.estimate(claim, t, g)
    assert w.bytes == 2 * 4096 * 65536 * 2 + 2 * 4096 * 2 and w.launches == 1
    assert gen.claims(t, G.softmax(20, 3))[-1].threads == 8
    big = G.Group(8, 1)
    x = big.load(big.input())
    for _ in range(60):
        x = big.neg(x)
    big.output(x)
    assert gen.claims(t, big) == ()
    import pytest
    with pytest.raises(ValueError):
        gen.build_claim(None, t, big, {"inputs": [0], "outputs": [0]})
    launch, text = gen.build_claim(claim, t, g, {0: 16, 1: 32, 2: 48, 3: 64})
    assert launch.repoints() and "3 sweeps" in text
    launch.repoint(3, 128)
    assert launch.outputs == [(3, 128)] and launch.inputs[0] == (0, 16)
    # a group that folds the other axis: one claim, two launches, n values per fold
    cols = G.layernorm_weight_gradients(4096, 65536, "BFloat16")
    (cc,) = gen.claims(t, cols)
    assert isinstance(cc, I.ColumnClaim)
    (w,) = gen.estimate(cc, t, cols)
    assert w.launches == 2 and w.bytes == 2 * 4096 * 65536 * 2 + 2 * 65536 * 4 + 2 * 4096 * 2


def test_scan_templates(I):
    lib, t = I.B200Kernels(), I.Target()
    names = [x.name for x in lib.templates(t)]
    assert "cumsum_dims1" in names and "recurrence_dims2_reverse" in names and "running_variance_dims1" in names
    assert "cumsum_dims1" in [x.name for x in lib.templates(I.Target(online=False))]     # a scan needs no rewrite
    n, rows = 1000, 64
    arrays = {"x": I.dense_columns(None, "Float32", n, rows, 1), "y": I.dense_columns(None, "Float32", n, rows, 2)}
    b = I.Binding("cumsum_dims2", {"n": n, "rows": rows}, arrays)
    assert lib.supports(t, b)
    (w,) = lib.estimate(t, b)
    assert w.bytes == 2 * n * rows * 4 and w.blocks == 4
    # many rows: cut into slabs, two launches, the input read twice
    tall = I.Binding("cumsum_dims2", {"n": 4096, "rows": 16384}, {"x": I.dense_columns(None, "Float32", 4096, 16384, 1),
                                                                  "y": I.dense_columns(None, "Float32", 4096, 16384, 2)})
    (w,) = lib.estimate(t, tall)
    assert w.launches == 2 and w.reread == 4096 * 16384 * 4 and w.split
    assert not lib.supports(t, I.Binding("recurrence_dims1", {"n": n, "rows": rows}, arrays))   # the pairs' second array is missing
    assert not lib.supports(t, I.Binding("cumsum_dims3", {"n": n, "rows": rows}, arrays))
    launch = I.ScanLaunch(I.Binding("cummax_dims1_reverse", {"n": n, "rows": rows}, arrays))
    assert (launch.op, launch.across, launch.reverse) == (2, False, True)


def test_tuning_record_keeps_and_reads_back(pkg, tmp_path, monkeypatch):
    """The picks made while building launches, kept between sessions as the reference keeps its tuning record
    (src/Compiler/cover/record.jl:22-32, 60-80): a tab-separated file per device under TEMPEST_CACHE/tuning,
    appended to, the later line winning, a line cut short ignored."""
    T = pkg.tuning
    assert T.file_name("NVIDIA B200 (sm_100a)") == "NVIDIA_B200__sm_100a_"
    monkeypatch.delenv("TEMPEST_CACHE", raising=False)
    assert T.tuning_directory() is None
    nowhere = T.TuningRecord("NVIDIA B200")
    assert nowhere.path is None
    nowhere.keep("product", "k", {"tile_n": 512})
    assert nowhere.lookup("product", "k") == {"tile_n": 512}      # kept in memory, written nowhere
    monkeypatch.setenv("TEMPEST_CACHE", str(tmp_path))
    assert T.tuning_directory() == str(tmp_path / "tuning")
    r = T.TuningRecord("NVIDIA B200")
    assert r.path == str(tmp_path / "tuning" / "NVIDIA_B200.b200.tsv") and r.lookup("product", "a") is None
    key = r.key("linear_bias_gelu", 4096, 8192, 4096, "BFloat16")
    assert key == "linear_bias_gelu 4096 8192 4096 BFloat16"
    r.keep("product", key, {"tile_n": 256, "direct_epilogue": 0}, 0.21)
    r.keep("product", key, {"tile_n": 512, "direct_epilogue": 0}, 0.19)
    r.keep("attention_pullback", "x", {"deterministic": 1})
    with open(r.path, "a") as f:
        f.write("product\tcut short")
    again = T.TuningRecord("NVIDIA B200")
    assert again.lookup("product", key) == {"tile_n": 512, "direct_epilogue": 0}
    assert again.lookup("attention_pullback", "x") == {"deterministic": 1}
    assert again.lookup("product", "cut short") is None and again.written == 0
    other = T.TuningRecord("NVIDIA H100")                           # another device: another file
    assert other.lookup("product", key) is None


def test_masked_attention_templates(I):
    """Attention whose mask the device holds, as the reference's packed-documents and decode programs
    (test/cuda/attention.jl:217-275): offered on a target that allows one-pass folds, the mask array Int32 and dense."""
    lib, t = I.B200Kernels(), I.Target()
    names = [x.name for x in lib.templates(t)]
    for want in ("attention_causal_documents", "attention_causal_documents_lse", "attention_lengths_lse",
                 "attention_causal_documents_pullback", "attention_lengths_pullback"):
        assert want in names
    D, H, S, B = 128, 2, 300, 2
    heads = lambda v: I.dense_heads(None, "BFloat16", D, H, S, B, v)  # noqa: E731
    e = {"d": D, "h": H, "hk": H, "m": S, "n": S, "b": B, "one": 1}
    arrays = {"q": heads(1), "k": heads(2), "v": heads(3), "o": heads(4),
              "start": I.Strided("Int32", 0, (S, B), (1, S), None, 5)}
    assert lib.supports(t, I.Binding("attention_causal_documents", e, arrays))
    assert not lib.supports(t, I.Binding("attention_causal_documents", e, {k: v for k, v in arrays.items() if k != "start"}))
    assert not lib.supports(t, I.Binding("attention_causal_documents", e, dict(arrays, start=I.Strided("Float32", 0, (S, B), (1, S), None, 5))))
    assert not lib.supports(t, I.Binding("attention_lengths", e, arrays))       # the other mask's array
    lengths = dict({k: v for k, v in arrays.items() if k != "start"}, lengths=I.dense_vector(None, "Int32", B, 6))
    assert lib.supports(t, I.Binding("attention_lengths", e, lengths))


def test_tile_form_of_a_product(pkg):
    """Which tiles a product takes, decided on the host: pairs of CTAs on 256 x 256 tiles wherever there is at least
    one such tile per pair of SMs (148 SMs where no device answers), single-CTA tiles of 256 columns below that, of 128
    where the wide ones would fill less than half the device or the result is narrow; the descriptor can ask."""
    L = pkg.lib
    assert L.gemm_tile_form(L.gemm_desc(8192, 4096, 4096)) == 512          # 32 x 16 tiles for 74 pairs
    assert L.gemm_tile_form(L.gemm_desc(8192, 1024, 4096)) == 512          # 128 tiles
    assert L.gemm_tile_form(L.gemm_desc(2048, 2048, 256)) == 256           # 64 pair tiles: not one per pair of SMs
    assert L.gemm_tile_form(L.gemm_desc(1024, 1024, 4096)) == 128          # 32 wide tiles: under half the device
    assert L.gemm_tile_form(L.gemm_desc(4096, 128, 512)) == 128            # a narrow result
    assert L.gemm_tile_form(L.gemm_desc(8192, 4096, 4096, tile_n=-1)) == 256   # single-CTA tiles asked for
    assert L.gemm_tile_form(L.gemm_desc(8192, 4096, 4096, tile_n=128)) == 128
    assert L.gemm_tile_form(L.gemm_desc(512, 512, 64, tile_n=512)) == 512
    assert L.gemm_tile_form(L.gemm_desc(128, 512, 64, tile_n=512)) == 256  # one row of tiles: nothing to pair
    assert L.gemm_tile_form(L.gemm_desc(64, 2048, 2048, batch=64)) == 256  # a batch of short products: one row of tiles each, nothing to pair
    assert L.gemm_tile_form(L.gemm_desc(0, 512, 64)) == 0


def test_the_rest_of_the_protocol(pkg):
    """What the cover asks of an implementation before it offers it a group
    (src/Compiler/Implement/Implement.jl:85-214), each answer checked against the default's meaning."""
    I, G = pkg.implement, pkg.groups
    gen, lib, t = I.B200Generator(), I.B200Kernels(), I.Target()
    assert gen.package_of() == lib.package_of() == "tempest_b200"       # one line of the rates file for both doors
    assert gen.loaded() and lib.loaded()
    assert isinstance(gen.resources(t), I.Resources) and gen.resources(t) is not gen.resources(t)
    assert gen.candidates(t, plan=None) == []
    assert gen.recomputes_folds(t)
    g = G.softmax(4096, 8)
    claim = gen.claims(t, g)[-1]
    name = gen.record_name(claim)
    assert name.startswith("B200Generator RowClaim(") and name == gen.record_name(gen.claims(t, G.softmax(4096, 8))[-1])
    # scalar functions: by name, or as a term of a group
    assert gen.lowers(t, "tanh") and gen.lowers(t, "fma") and not gen.lowers(t, "erf") and not gen.lowers(t, "load")
    assert all(gen.lowers(t, i, g) for i in range(len(g.terms)))


def test_which_kernels_compute_an_attention(pkg):
    """tb200_attention_form: the entries' own routing as host arithmetic -- the benchmark's geometry goes to the
    tensor cores in every direction, the reference's small test geometries to the CUDA cores."""
    L = pkg.lib
    bench = L.attn_desc(8, 32, 4096, 4096, 128, True)
    assert L.attention_form(bench) == L.ATTN_FORM_TWO_TILES
    assert L.attention_form(bench, masked=True) == L.ATTN_FORM_TILE          # device-held masks: one tile a block
    assert L.attention_form(bench, pullback=True) == L.ATTN_FORM_ONE_KERNEL  # the reference's default, not deterministic
    det = L.attn_desc(8, 32, 4096, 4096, 128, True, deterministic=True)
    assert L.attention_form(det, pullback=True) == L.ATTN_FORM_TWO_KERNELS
    assert L.attention_form(L.attn_desc(1, 32, 128, 8192, 128, False, kv_heads=8)) == L.ATTN_FORM_TILE   # decode over a cache
    for d, h, kv, s, b in ((16, 2, 2, 200, 2), (16, 4, 2, 200, 2), (32, 3, 1, 70, 3), (8, 1, 1, 133, 1)):
        small = L.attn_desc(b, h, s, s, d, True, kv_heads=kv)                # test/cuda/attention.jl:10-16
        assert L.attention_form(small) == L.attention_form(small, pullback=True) == L.ATTN_FORM_CUDA_CORES
    assert L.attention_form(L.attn_desc(1, 4, 64, 64, 128, False, value_dim=64)) == L.ATTN_FORM_CUDA_CORES
    import pytest
    with pytest.raises(L.TB200Error):
        L.attention_form(L.attn_desc(1, 3, 64, 64, 128, False, kv_heads=2))  # heads not a multiple of key heads
