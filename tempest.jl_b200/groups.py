"""Row groups as data: the host-side picture of what Tempest hands a backend.

Tempest's planner gives every backend a `GroupView` (src/Compiler/Implement/groups.jl:106-125): the kind of
the group, its domain, its terms (`IR/terms.jl:12-87`: Load, Lit, Ix, Apply, Stat, Cast) and its folds
(`IR/folds.jl`).  `Group` builds the cut of that view this library runs -- a (n, rows) domain whose first,
contiguous axis is folded -- and turns it into the `tb200_group_desc` of include/tempest_b200.h.  The
spellings at the bottom are the reference's own test programs (test/fixtures/programs.jl:7-19,
test/cuda/folds.jl:10-14) written as terms; the named kernels compute the first three faster.
"""
from . import lib as L

OPS = {"load": 0, "lit": 1, "index": 2, "stat": 3, "stat2": 4, "add": 5, "sub": 6, "mul": 7, "div": 8, "max": 9,
       "min": 10, "neg": 11, "exp": 12, "log": 13, "tanh": 14, "sqrt": 15, "rsqrt": 16, "abs": 17, "abs2": 18,
       "recip": 19, "sigmoid": 20, "fma": 21, "select": 22, "round_bf16": 23, "recomputed": 24, "row_index": 25, "state": 26}
ARITY = {**{k: 0 for k in ("load", "lit", "index", "stat", "stat2", "recomputed", "row_index", "state")},
         **{k: 2 for k in ("add", "sub", "mul", "div", "max", "min")},
         **{k: 1 for k in ("neg", "exp", "log", "tanh", "sqrt", "rsqrt", "abs", "abs2", "recip", "sigmoid", "round_bf16")},
         "fma": 3, "select": 3}
FOLDS = {"sum": 0, "max": 1, "min": 2, "prod": 3, "logsumexp": 4, "meanvar": 5, "weighted": 6}
SHAPES = {"full": 0, "along": 1, "per_row": 2, "scalar": 3, "row_vectors": 4, "along_vectors": 5}
DTYPES = {"Float32": L.F32, "BFloat16": L.BF16}


class Group:
    """A map -> fold group over (n, rows).  Methods return the index of the term / fold / input they add."""

    def __init__(self, n, rows, across=False):
        """`across`: the folds run over the rows (the other axis) and each yields `n` values -- the groups of
        `lib.colreduce_compiled`; otherwise along each row, one value per row."""
        self.n, self.rows, self.across = int(n), int(rows), bool(across)
        self.inputs, self.terms, self.folds, self.outputs = [], [], [], []
        self._level = []   # first phase in which a term can be evaluated

    # ---- leaves
    def input(self, shape="full", eltype="Float32", ld=None):
        self.inputs.append((SHAPES[shape], DTYPES[eltype], int(ld if ld is not None else self.n)))
        return len(self.inputs) - 1

    def _term(self, op, a=0, b=0, c=0, imm=0.0, level=0):
        self.terms.append((OPS[op], int(a), int(b), int(c), float(imm)))
        self._level.append(level)
        return len(self.terms) - 1

    def load(self, inp):
        return self._term("load", inp)

    def lit(self, x):
        return self._term("lit", imm=x)

    def index(self):
        return self._term("index")

    def row_index(self):
        """The row's own position (with `index` under a `select`: a mask on two positions)."""
        return self._term("row_index")

    def recomputed(self, per_row, along, extent):
        """sum over e < extent of X[row][e] * Y[i][e]: a fold formed where it is read (`Recomputed`,
        src/Compiler/IR/terms.jl:69-87); X an input of shape "row_vectors", Y one of shape "along_vectors"."""
        return self._term("recomputed", per_row, along, extent)

    def stat(self, fold, second=False):
        return self._term("stat2" if second else "stat", fold, level=self.folds[fold][2] + 1)

    # ---- Apply nodes
    def apply(self, op, *args):
        assert len(args) == ARITY[op], (op, args)
        padded = list(args) + [0] * (3 - len(args))
        return self._term(op, *padded, level=max(self._level[a] for a in args))

    def __getattr__(self, op):
        if op in ARITY and ARITY[op] > 0:
            return lambda *args: self.apply(op, *args)
        raise AttributeError(op)

    # ---- folds and outputs
    def fold(self, kind, term, payload=0):
        """The fold runs in the first phase in which its term is known (a term that reads a statistic waits
        for that statistic's phase to finish).  `payload`: the input of value rows a "weighted" fold sums."""
        self.folds.append((FOLDS[kind], int(term), self._level[term], int(payload)))
        return len(self.folds) - 1

    def output(self, term, eltype="Float32", ld=None):
        self.outputs.append((0, int(term), DTYPES[eltype], int(ld if ld is not None else self.n)))
        return len(self.outputs) - 1

    def output_stat(self, fold, eltype="Float32", second=False):
        self.outputs.append((2 if second else 1, int(fold), DTYPES[eltype], 0))
        return len(self.outputs) - 1

    # ---- the C descriptor
    def desc(self):
        if (len(self.inputs) > L.GROUP_MAX_INPUTS or len(self.terms) > L.GROUP_MAX_TERMS or
                len(self.folds) > L.GROUP_MAX_FOLDS or len(self.outputs) > L.GROUP_MAX_OUTPUTS):
            raise ValueError("group too large for one descriptor")
        d = L.GroupDesc()
        d.n, d.rows = self.n, self.rows
        d.n_inputs, d.n_terms, d.n_folds, d.n_outputs = (len(self.inputs), len(self.terms), len(self.folds),
                                                         len(self.outputs))
        for i, (shape, dtype, ld) in enumerate(self.inputs):
            d.inputs[i].shape, d.inputs[i].dtype, d.inputs[i].ld = shape, dtype, ld
        for i, (op, a, b, c, imm) in enumerate(self.terms):
            t = d.terms[i]
            t.op, t.a, t.b, t.c, t.imm = op, a, b, c, imm
        for i, (kind, term, phase, payload) in enumerate(self.folds):
            d.folds[i].kind, d.folds[i].term, d.folds[i].phase, d.folds[i].payload = kind, term, phase, payload
        for i, (source, index, dtype, ld) in enumerate(self.outputs):
            o = d.outputs[i]
            o.source, o.index, o.dtype, o.ld = source, index, dtype, ld
        return d

    def bytes(self):
        """Algorithmic bytes: every input once, every output once (the `bytes` of a GroupView)."""
        size = {L.F32: 4, L.BF16: 2}
        extent = {0: self.n * self.rows, 1: self.n, 2: self.rows, 3: 1}
        total = sum(extent[shape] * size[dtype] for shape, dtype, _ in self.inputs)
        per_fold = self.n if self.across else self.rows
        total += sum((self.n * self.rows if source == 0 else per_fold) * size[dtype]
                     for source, _, dtype, _ in self.outputs)
        return total


class Recurrence(Group):
    """A recurrence whose step is a map, over (n, steps): `n` positions that do not interact, stepping along the
    other axis with states carried from step to step (the `:recurrence` groups of
    src/Compiler/Implement/groups.jl:29-47 whose members are computed element by element).  States are declared
    first (`state(start)`, started from an input of shape "along" or "scalar"), read with `carried(k)`, and given
    their value after the step with `carry(k, term)`; every state is assigned at once from the values before the step."""

    kind = "recurrence"

    def __init__(self, n, steps, reverse=False):
        super().__init__(n, steps)
        self.reverse = bool(reverse)
        self.states = []   # [start input, next term]

    def state(self, start):
        self.states.append([int(start), -1])
        return len(self.states) - 1

    def carried(self, k):
        """The state's value before this step."""
        return self._term("state", k)

    def step_index(self):
        return self._term("row_index")

    def carry(self, k, term):
        self.states[k][1] = int(term)

    def output_state(self, k, eltype="Float32"):
        """State k as the steps leave it: n values."""
        self.outputs.append((3, int(k), DTYPES[eltype], 0))
        return len(self.outputs) - 1

    def bytes(self):
        size = {L.F32: 4, L.BF16: 2}
        extent = {0: self.n * self.rows, 1: self.n, 2: self.rows, 3: 1}
        total = sum(extent[shape] * size[dtype] for shape, dtype, _ in self.inputs)
        return total + sum((self.n * self.rows if source == 0 else self.n) * size[dtype]
                           for source, _, dtype, _ in self.outputs)

    def desc(self):
        if not self.states or any(nxt < 0 for _, nxt in self.states) or len(self.states) > 4:
            raise ValueError("a recurrence has one to four states, each carried from a term")
        r = L.RecurrenceDesc()
        r.body = super().desc()
        r.n_states = len(self.states)
        for k, (start, nxt) in enumerate(self.states):
            r.states[k].start, r.states[k].next = start, nxt
        r.reverse = int(self.reverse)
        return r


def gated_tanh_cell(n, steps, eltype="Float32", reverse=False):
    """h = tanh.(a .* h .+ x) at every step, h stored: the map part of the reference's `cell`
    (test/runtime/recurrences.jl:14) with a per-position gate in place of the matrix."""
    g = Recurrence(n, steps, reverse)
    x, a, h0 = g.input("full", eltype), g.input("along", eltype), g.input("along", eltype)
    h = g.state(h0)
    new = g.tanh(g.fma(g.load(a), g.carried(h), g.load(x)))
    g.carry(h, new)
    g.output(new, eltype)
    g.output_state(h, eltype)
    return g


def second_order(n, steps, eltype="Float32"):
    """(y, last) -> (tanh.(1.5 .* y .- 0.5 .* last .+ x), y): two states assigned at once, the second lagging the first
    (test/runtime/recurrences.jl:195)."""
    g = Recurrence(n, steps)
    x, a, b = g.input("full", eltype), g.input("along", eltype), g.input("along", eltype)
    y, last = g.state(a), g.state(b)
    new = g.tanh(g.add(g.sub(g.mul(g.lit(1.5), g.carried(y)), g.mul(g.lit(0.5), g.carried(last))), g.load(x)))
    g.carry(y, new)
    g.carry(last, g.carried(y))
    g.output(new, eltype)
    g.output_state(y, eltype)
    g.output_state(last, eltype)
    return g


def decayed_sum(n, steps, eltype="Float32"):
    """s = s .* 0.5 .+ abs2.(x) with a scalar start: the map form of the reference's `run`
    (test/runtime/recurrences.jl:15), only the last state kept."""
    g = Recurrence(n, steps)
    x, s0 = g.input("full", eltype), g.input("scalar", eltype)
    s = g.state(s0)
    g.carry(s, g.fma(g.carried(s), g.lit(0.5), g.abs2(g.load(x))))
    g.output_state(s, eltype)
    return g


# ---- the reference's programs as groups -------------------------------------------------------------------

def softmax(n, rows, eltype="Float32"):
    """exp.(x .- logsumexp(x; dims=1))  (test/fixtures/programs.jl:8)."""
    g = Group(n, rows)
    x = g.load(g.input("full", eltype))
    lse = g.fold("logsumexp", x)
    g.output(g.exp(g.sub(x, g.stat(lse))), eltype)
    g.output_stat(lse)
    return g


def log_softmax(n, rows, eltype="Float32"):
    g = Group(n, rows)
    x = g.load(g.input("full", eltype))
    lse = g.fold("logsumexp", x)
    g.output(g.sub(x, g.stat(lse)), eltype)
    return g


def softmax_pullback(n, rows, eltype="Float32"):
    """t = g .* y;  t .- y .* sum(t; dims=1)."""
    g = Group(n, rows)
    y = g.load(g.input("full", eltype))
    dy = g.load(g.input("full", eltype))
    t = g.mul(dy, y)
    s = g.fold("sum", t)
    g.output(g.sub(t, g.mul(y, g.stat(s))), eltype)
    return g


def layernorm(n, rows, eltype="Float32", eps=1.0e-5, two_pass=False):
    """(x .- m) ./ sqrt.(v .+ eps) .* w .+ b  (test/fixtures/programs.jl:13-17).  `two_pass` spells the variance
    as the reference's source does -- sum(abs2, x .- m) / n, a fold that waits for the mean -- instead of the
    one-pass Welford state its rewrite produces (src/Compiler/plan/rewrites.jl:29-44)."""
    g = Group(n, rows)
    x = g.load(g.input("full", eltype))
    w = g.load(g.input("along", eltype))
    b = g.load(g.input("along", eltype))
    if two_pass:
        s = g.fold("sum", x)
        mean = g.mul(g.stat(s), g.lit(1.0 / n))
        centred = g.sub(x, mean)
        q = g.fold("sum", g.abs2(centred))
        var = g.mul(g.stat(q), g.lit(1.0 / n))
    else:
        mv = g.fold("meanvar", x)
        centred = g.sub(x, g.stat(mv))
        var = g.stat(mv, second=True)
    rstd = g.rsqrt(g.add(var, g.lit(eps)))
    g.output(g.fma(g.mul(centred, rstd), w, b), eltype)
    return g


def rmsnorm(n, rows, eltype="Float32", eps=1.0e-6):
    """x ./ sqrt.(sum(abs2, x; dims=1) ./ n .+ eps) .* w  (test/cuda/folds.jl:10-14)."""
    g = Group(n, rows)
    x = g.load(g.input("full", eltype))
    w = g.load(g.input("along", eltype))
    q = g.fold("sum", g.abs2(x))
    scale = g.rsqrt(g.fma(g.stat(q), g.lit(1.0 / n), g.lit(eps)))
    g.output(g.mul(g.mul(x, scale), w), eltype)
    return g


def attention(keys, queries, features, causal, scale=None, lse=True):
    """The attention group of the reference's plans at one (head, batch) (test/fixtures/operations.jl:21-76 as the
    planner groups it, src/Compiler/Implement/groups.jl:106-125): over the keys of each query row fold the pair
    (score, value row) -- scores recomputed over the features and, when causal, masked to the keys up to the
    query's own position; their log-sum-exp shares the sweep; the output is the weights' sum of the value rows.
    Not a row fold of scalars: `lib.group_route` recognises it and `lib.group_attention` runs it."""
    g = Group(keys, queries)
    q = g.input("row_vectors", "BFloat16", ld=features)
    k = g.input("along_vectors", "BFloat16", ld=features)
    v = g.input("along_vectors", "BFloat16", ld=features)
    s = g.mul(g.lit(features ** -0.5 if scale is None else scale), g.recomputed(q, k, features))
    if causal:
        s = g.select(g.add(g.sub(g.row_index(), g.index()), g.lit(0.5)), s, g.lit(float("-inf")))
    stat = g.fold("logsumexp", s)
    o = g.fold("weighted", g.exp(g.sub(s, g.stat(stat))), payload=v)
    g.output_stat(o, "BFloat16")
    if lse:
        g.output_stat(stat, "Float32")
    return g


def row_extrema(n, rows, eltype="Float32"):
    """maximum, minimum, sum and product along the folded axis: four statistics in one sweep."""
    g = Group(n, rows)
    x = g.load(g.input("full", eltype))
    for kind in ("max", "min", "sum", "prod"):
        g.output_stat(g.fold(kind, x))
    return g


# ---- groups whose folds run over the rows (the other axis): `lib.colreduce_compiled` ------------------------
#
# The same builder with `across = True`.


def bias_gradient(n, rows, eltype="Float32"):
    """db[i] = sum over rows of g[i, row]: `sum(g; dims = 2)`, the pullback of a broadcast bias
    (test/fixtures/programs.jl:19-26 under withgradient)."""
    g = Group(n, rows, across=True)
    g.output_stat(g.fold("sum", g.load(g.input("full", eltype))), eltype)
    return g


def layernorm_weight_gradients(n, rows, eltype="Float32"):
    """dgamma[i] = sum over rows of g * (x - mean) * rstd and dbeta[i] = sum over rows of g, with the forward's
    saved mean and rstd: the two folds over the other axis of the LayerNorm pullback
    (ext/cuTileExt/emit.jl:729-753)."""
    g = Group(n, rows, across=True)
    x, dy = g.load(g.input("full", eltype)), g.load(g.input("full", eltype))
    mean, rstd = g.load(g.input("per_row", "Float32")), g.load(g.input("per_row", "Float32"))
    xh = g.mul(g.sub(x, mean), rstd)
    g.output_stat(g.fold("sum", g.mul(dy, xh)), eltype)
    g.output_stat(g.fold("sum", dy), eltype)
    return g


def column_extrema(n, rows, eltype="Float32"):
    """maximum, minimum and sum of |x| over the rows, per column."""
    g = Group(n, rows, across=True)
    x = g.load(g.input("full", eltype))
    g.output_stat(g.fold("max", x))
    g.output_stat(g.fold("min", x))
    g.output_stat(g.fold("sum", g.abs(x)))
    return g


def column_statistics(n, rows, eltype="Float32"):
    """Per column over the rows: the log-sum-exp, the mean and the variance -- the relative folds (online
    log-sum-exp, Welford / Chan) running over the other axis, `logsumexp(x; dims = 2)` and the moments of a batch."""
    g = Group(n, rows, across=True)
    x = g.load(g.input("full", eltype))
    g.output_stat(g.fold("logsumexp", x))
    mv = g.fold("meanvar", x)
    g.output_stat(mv)
    g.output_stat(mv, second=True)
    return g
