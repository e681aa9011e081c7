"""Groups the library recognises by the structure of their terms and hands to a kernel of their own (no GPU needed
for the recognition)."""


def test_attention_group_is_described_and_routed(pkg):
    """The attention group of the reference's plans -- scores as a Recomputed sum over the features, the causal mask as
    a select on two positions, the log-sum-exp, and the weights' sum of the value rows -- is a descriptor the library
    recognises by its terms; the row interpreter and generator decline it; near misses are not taken for it."""
    G, L, I = pkg.groups, pkg.lib, pkg.implement
    for causal in (False, True):
        g = G.attention(200, 200, 128, causal)
        d = g.desc()
        assert L.group_route(d) == (L.ROUTE_ATTENTION_CAUSAL if causal else L.ROUTE_ATTENTION)
        assert L.rowreduce_generic_check(d) == -7 and L.rowreduce_compile(d) != 0
        (claim,) = I.B200Generator().claims(I.Target(), g)
        assert isinstance(claim, I.AttentionClaim) and claim.causal == causal
        (w,) = I.B200Generator().estimate(claim, I.Target(), g)
        assert w.flops == 4.0 * 128 * 200 * 200 * (0.5 if causal else 1.0)
        launch, text = I.B200Generator().build_claim(claim, I.Target(), g, {0: 16, 1: 32, 2: 48, 3: 64, 4: 80, "outer": (4, 2, 3)})
        assert "attention" in text and launch.outer == (4, 2, 3) and launch.repoints()
    assert L.group_route(G.softmax(64, 8).desc()) == L.ROUTE_NONE
    # the weights must be exp(scores - stat(lse)) of the same scores the log-sum-exp folds
    g = G.Group(64, 64)
    q, k, v = g.input("row_vectors", "BFloat16", ld=128), g.input("along_vectors", "BFloat16", ld=128), g.input("along_vectors", "BFloat16", ld=128)
    s = g.mul(g.lit(0.1), g.recomputed(q, k, 128))
    other = g.mul(g.lit(0.2), g.recomputed(q, k, 128))
    lse = g.fold("logsumexp", s)
    g.output_stat(g.fold("weighted", g.exp(g.sub(other, g.stat(lse))), payload=v), "BFloat16")
    assert L.group_route(g.desc()) == L.ROUTE_NONE
    # a mask the other way round (keys after the query) is not the causal program
    g = G.Group(64, 64)
    q, k, v = g.input("row_vectors", "BFloat16", ld=128), g.input("along_vectors", "BFloat16", ld=128), g.input("along_vectors", "BFloat16", ld=128)
    s = g.mul(g.lit(0.1), g.recomputed(q, k, 128))
    s = g.select(g.add(g.sub(g.index(), g.row_index()), g.lit(0.5)), s, g.lit(float("-inf")))
    lse = g.fold("logsumexp", s)
    g.output_stat(g.fold("weighted", g.exp(g.sub(s, g.stat(lse))), payload=v), "BFloat16")
    assert L.group_route(g.desc()) == L.ROUTE_NONE
