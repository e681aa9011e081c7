"""The MLP training step of examples/mlp.jl on the B200 kernels.

The reference spells it as plain Julia (examples/mlp.jl:13-35): layers
`h = act.(w * h .+ b)` with no activation after the last, loss
`sum(abs2, forward(x) .- y) / size(y, 2)`, `withgradient`, and the update
`w .- rate .* dw`, `b .- rate .* db`; `Tempest.compile` turns the step into
kernels.  Here the same step is the kernel list a Tempest plan of it reaches:

  forward   one product per layer with the bias and activation fused in its
            epilogue (the value before the activation kept for the backward),
  loss      one squared-error fold that also writes the loss's pullback,
  backward  per layer, last first: db = column sums of dz; dw = h_in' * dz;
            dz_below = (dz * w') .* act'(z_below) fused in the product's
            epilogue; and the update either fused into dw's epilogue
            (w = w - rate * dw, single GPU) or applied after the gradients of
            all replicas are summed (data parallel).

Layout: a Julia `w::(out,in)` is memory [in][out]; activations `(features,
batch)` are memory [batch][features].  All arrays BFloat16, Float32 accumulate.
Parameters live in one flat BFloat16 buffer and their gradients in a second one
laid out the same way (each array starting on a 16-byte boundary), so that a
group of layers is one contiguous range: one all-reduce sums it and one
`y += alpha x` launch applies it.  Every product is a prepared launch
(`lib.GemmPlan`): its TMA descriptors are built once, a step makes one C call per
product.

Data parallel (one process per GPU): each replica runs the step on its batch
shard; a bucket of gradients is summed across replicas by an NCCL all-reduce
issued on a side stream as soon as its layers' gradients exist, overlapping the
remaining backward products; the update runs when the bucket has landed.  The
MSE is a mean over the global batch, so each replica scales its pullback by
1 / global batch.  Given a `dp.ReplicaLink` (buffers every replica can address)
the exchange and the update of a bucket are instead one kernel of the library's
own, `tb200_dp_update`: each rank sums one slice of the bucket through the
NVSwitch, applies the step and writes the new weights to every replica.
"""
from . import lib

ACTIVATIONS = {"gelu_tanh": (lib.EPI_BIAS_GELU, lib.EPI_MUL_GELU_GRAD, "z"),
               "tanh": (lib.EPI_BIAS_TANH, lib.EPI_MUL_TANH_GRAD, "a")}


def shard_rows(total, rank, world):
    """[first, last) rows of a batch of `total` that replica `rank` of `world` trains on: equal
    contiguous shards (the batch must divide evenly, so every replica runs the same kernels)."""
    if total % world != 0:
        raise ValueError(f"a batch of {total} does not split over {world} replicas")
    per = total // world
    return rank * per, (rank + 1) * per


def sum_over_replicas(torch, buckets, group=None, stream=None):
    """Sums each gradient bucket over the replicas, last first (the order the backward produces
    them), on `stream` when given.  Returns the events that mark each bucket's sum as landed
    (None without a stream).  The collective is torch.distributed's all-reduce: NCCL over NVLink on
    GPUs, and any other backend (gloo on CPU) for the host-side tests."""
    dist = torch.distributed
    marks = []
    for b in reversed(buckets):
        if stream is None:
            dist.all_reduce(b, group=group)
            marks.append(None)
        else:
            with torch.cuda.stream(stream):
                dist.all_reduce(b, group=group)
                done = torch.cuda.Event()
                done.record(stream)
            marks.append(done)
    return list(reversed(marks))


def glorot_uniform(torch, fan_in, fan_out, generator, device="cuda"):
    """W (out, in) ~ U(+-sqrt(6 / (in + out))), stored [in][out] BFloat16."""
    limit = (6.0 / (fan_in + fan_out)) ** 0.5
    w = (torch.rand(fan_in, fan_out, device=device, generator=generator) * 2.0 - 1.0) * limit
    return w.to(torch.bfloat16)


def flat_layout(sizes, fused):
    """Where each layer's weight and bias sit in the flat parameter (and gradient) buffer, and which
    ranges are exchanged together.  Returns (order, offsets, total, buckets): `order` the layers as they
    are laid out; offsets[i] = (weight offset, bias offset) in elements, every array on a 16-byte
    boundary; buckets = [(first element, last element, layers)] in the order their exchanges start.

    The middle layers (the large arrays of an MLP whose ends are narrow) come first, one bucket each, in
    the order the backward forms their gradients; the first and the last layer lie side by side behind
    them and travel as one bucket at the end of the step -- one exchange fewer with nothing to hide
    behind.  Networks of fewer than three layers, and fused single-GPU steps (no exchange), keep the
    layers in order with one bucket per layer."""
    L = len(sizes) - 1
    if fused or L < 3:
        order, groups = list(range(L)), [[i] for i in range(L - 1, -1, -1)]
    else:
        middle = list(range(L - 2, 0, -1))
        order, groups = middle + [0, L - 1], [[i] for i in middle] + [[0, L - 1]]
    offsets, spans, at = {}, {}, 0
    for i in order:
        nw, nb = sizes[i] * sizes[i + 1], sizes[i + 1]
        first, w_at = at, at
        at = (at + nw + 7) // 8 * 8
        b_at = at
        at = (at + nb + 7) // 8 * 8
        offsets[i] = (w_at, b_at)
        spans[i] = (first, at)
    buckets = [(min(spans[i][0] for i in g), max(spans[i][1] for i in g), tuple(g)) for g in groups]
    return order, offsets, at, buckets


def _count(shape):
    n = 1
    for s in shape:
        n *= s
    return n


class MLPStep:
    """One compiled training step; `step(x, y)` runs it once."""

    def __init__(self, torch, sizes, batch, rate, activation="gelu_tanh", world=1, global_batch=None,
                 process_group=None, seed=0, weights=None, biases=None, fuse_update=None, link=None, exchange_blocks=0):
        self.torch = torch
        self.sizes, self.batch, self.rate = list(sizes), batch, rate
        self.world = world
        self.global_batch = global_batch if global_batch is not None else batch * world
        self.group = process_group
        # the update rides in dw's epilogue unless gradients must first be summed across replicas
        self.fuse_update = (world == 1) if fuse_update is None else (fuse_update and world == 1)
        self.link = None
        self.fwd_epi, self.bwd_epi, self.saved = ACTIVATIONS[activation]
        bf = torch.bfloat16
        gen = torch.Generator(device="cuda").manual_seed(seed)
        L = len(sizes) - 1
        self.L = L
        self.order, self.offsets, total, self.buckets = flat_layout(self.sizes, self.fuse_update)
        # the gaps that align each array are zero in both buffers and stay zero (0 + alpha * 0).  With a `link`
        # (dp.ReplicaLink: buffers every replica can address) the exchange and the update are one kernel of the
        # library's own (tb200_dp_update) instead of an NCCL all-reduce followed by y += alpha x
        self.link = link if world > 1 else None
        if self.link is not None:
            if self.link.elements < total:
                raise ValueError("the replica link is smaller than the step's parameters")
            self.params, self.grads = self.link.params[:total], self.link.grads[:total]
        else:
            self.params, self.grads = (torch.zeros(total, device="cuda", dtype=bf) for _ in range(2))
        self.exchange_blocks = exchange_blocks

        def view(flat, at, *shape):
            return flat[at: at + _count(shape)].view(*shape)

        self.w = [view(self.params, self.offsets[i][0], sizes[i], sizes[i + 1]) for i in range(L)]
        self.b = [view(self.params, self.offsets[i][1], sizes[i + 1]) for i in range(L)]
        self.dw = [view(self.grads, self.offsets[i][0], sizes[i], sizes[i + 1]) for i in range(L)]
        self.db = [view(self.grads, self.offsets[i][1], sizes[i + 1]) for i in range(L)]
        for i in range(L):
            self.w[i].copy_(glorot_uniform(torch, sizes[i], sizes[i + 1], gen) if weights is None else weights[i])
            if biases is not None:
                self.b[i].copy_(biases[i])
        # what is exchanged: contiguous ranges of the gradient buffer, in the order their exchanges start
        self.bucket = [self.grads[first:last] for first, last, _ in self.buckets]
        # activations a[i] (input of layer i), z[i] (what layer i's activation saw)
        self.a = [None] + [torch.empty(batch, sizes[i + 1], device="cuda", dtype=bf) for i in range(L)]
        self.z = [torch.empty(batch, sizes[i + 1], device="cuda", dtype=bf) if self.saved == "z" and i < L - 1
                  else None for i in range(L)]
        self.dz = [torch.empty(batch, sizes[i + 1], device="cuda", dtype=bf) for i in range(L)]
        self.loss = torch.zeros(1, device="cuda", dtype=torch.float32)
        self.sq_ws_bytes = lib.squared_error_workspace_bytes()
        self.sq_ws = torch.zeros(self.sq_ws_bytes, device="cuda", dtype=torch.uint8)
        cs = max(lib.colsum_workspace_bytes(batch, sizes[i + 1]) for i in range(L))
        self.cs_ws_bytes = cs
        self.cs_ws = torch.empty(max(cs, 16), device="cuda", dtype=torch.uint8)
        self.comm_stream = torch.cuda.Stream() if world > 1 else None
        self.launches = 0
        self._plans = None
        self._x_ptr = None
        self._dp = None
        if self.link is not None:
            self._dp = [self.link.desc(first, last, -rate, exchange_blocks) for first, last, _ in self.buckets]

    def parameters(self):
        return self.w, self.b

    def check(self):
        """Synchronises and raises if one of the step's tensor-core products gave up a bounded wait (the
        launches only enqueue): call it after `step()` or a replay, before the loss or the weights are read."""
        lib.check_device()

    # ---- prepared products ------------------------------------------------
    def _prepare(self, x):
        """Builds the step's products once (or moves the two that read the input batch to a new address)."""
        ptr = x.data_ptr()
        if self._plans is not None:
            if ptr != self._x_ptr:
                self._plans["fwd"][0].repoint(lib.GEMM_A, ptr)
                self._plans["grads"][0].repoint(lib.GEMM_A, ptr)
                self._x_ptr = ptr
            return
        bf16, L = lib.BF16, self.L
        fwd, below, grads = [], [None] * L, []
        self._scratch = []

        def plan(desc, *operands, **more):
            # a product with too few tiles to fill the device (a replica's slice of the batch against a narrow
            # layer) splits its sum over k when it is given scratch for the partial tiles
            need = lib.gemm_workspace_bytes(desc)
            if need:
                ws = self.torch.empty(need, dtype=self.torch.uint8, device="cuda")
                self._scratch.append(ws)
                desc.workspace, desc.workspace_bytes = ws.data_ptr(), need
            return lib.GemmPlan(desc, *operands, **more)

        for i in range(L):
            fin, fout = self.sizes[i], self.sizes[i + 1]
            last = i == L - 1
            h = ptr if i == 0 else self.a[i].data_ptr()
            fwd.append(plan(
                lib.gemm_desc(self.batch, fout, fin, a_layout=lib.K_MAJOR, b_layout=lib.MN_MAJOR, in_dtype=bf16,
                              epilogue=lib.EPI_BIAS if last else self.fwd_epi),
                h, self.w[i].data_ptr(), self.a[i + 1].data_ptr(), bias=self.b[i].data_ptr(),
                aux_out=0 if (last or self.z[i] is None) else self.z[i].data_ptr()))
            if i > 0:
                # dz[i - 1] = (dz[i] * w[i]') .* act'(saved): A = dz [batch][fout], B = w as [n = fin][k = fout]
                saved = self.z[i - 1] if self.saved == "z" else self.a[i]
                below[i] = plan(
                    lib.gemm_desc(self.batch, fin, fout, a_layout=lib.K_MAJOR, b_layout=lib.K_MAJOR, in_dtype=bf16,
                                  epilogue=self.bwd_epi),
                    self.dz[i].data_ptr(), self.w[i].data_ptr(), self.dz[i - 1].data_ptr(), aux=saved.data_ptr())
            if self.fuse_update:
                # w = w - rate * (a_in' * dz): the update rides in the product's epilogue
                grads.append(plan(
                    lib.gemm_desc(fin, fout, self.batch, a_layout=lib.MN_MAJOR, b_layout=lib.MN_MAJOR, in_dtype=bf16,
                                  epilogue=lib.EPI_AXPY, alpha=-self.rate),
                    h, self.dz[i].data_ptr(), self.w[i].data_ptr(), aux=self.w[i].data_ptr()))
            else:
                grads.append(plan(
                    lib.gemm_desc(fin, fout, self.batch, a_layout=lib.MN_MAJOR, b_layout=lib.MN_MAJOR, in_dtype=bf16),
                    h, self.dz[i].data_ptr(), self.dw[i].data_ptr()))
        self._plans = {"fwd": fwd, "below": below, "grads": grads}
        self._x_ptr = ptr

    # ---- forward + loss -------------------------------------------------
    def forward(self, x, stream):
        self._prepare(x)
        for plan in self._plans["fwd"]:
            plan.launch(stream)
        self.launches += self.L
        return self.a[self.L]

    def step(self, x, y):
        """x [batch][in], y [batch][out] BFloat16 on the device.  Returns the
        loss tensor (1 Float32 on the device; its value is this replica's share
        of the global mean when data parallel)."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        stream = cur.cuda_stream
        self._head(x, y, stream)
        events = []
        for kind, i in self._schedule():
            if kind == "below":
                self._dz_below(i, stream)
            elif kind == "grads":
                self._grads(i, stream)
            elif not self.fuse_update:
                events.append((i, self._exchange(i, cur)))
        for j, done in events:
            if done is not None:
                cur.wait_event(done)
            self._update(j, stream)
        return self.loss

    def _schedule(self):
        """The backward pass as a list of ("below", i) -- the gradient for the layer below layer i --,
        ("grads", i) -- layer i's bias and weight gradients -- and ("exchange", j) -- bucket j is complete and
        its exchange can start.
        Fused updates need layer i's weights intact until the layer below has its gradient, so they go top down:
        below(i), grads(i).  Replicas leave the weights alone until the end, which frees the order: the middle
        layers' gradients (the large buckets) are formed as soon as their dz exists, so that their exchanges start
        early, and the top and bottom layers' (small arrays here, one bucket) come last, with a whole product still
        to run behind the last large exchange."""
        L = self.L
        order = []
        if self.fuse_update or L < 3:
            for i in range(L - 1, -1, -1):
                if i > 0:
                    order.append(("below", i))
                order.append(("grads", i))
        elif self.link is not None:
            # the fused exchange writes the new weights of a bucket as soon as it runs, so a middle layer's
            # gradients (and with them its exchange) wait until the layer below has its gradient
            for i in range(L - 1, 0, -1):
                order.append(("below", i))
                if i <= L - 2:
                    order.append(("grads", i))
            order += [("grads", L - 1), ("grads", 0)]
        else:
            for i in range(L - 1, 0, -1):
                order.append(("below", i))
                if i - 1 >= 1:
                    order.append(("grads", i - 1))
            order += [("grads", L - 1), ("grads", 0)]
        pending = [len(layers) for _, _, layers in self.buckets]
        out = []
        for kind, i in order:
            out.append((kind, i))
            if kind == "grads":
                j = next(j for j, (_, _, layers) in enumerate(self.buckets) if i in layers)
                pending[j] -= 1
                if pending[j] == 0:
                    out.append(("exchange", j))
        return out

    def _head(self, x, y, stream):
        """Forward pass and loss: loss = sum(abs2, out - y) / batch ; dz_last = 2 (out - y) / batch."""
        self.a[0] = x
        out = self.forward(x, stream)
        inv = 1.0 / self.global_batch
        lib.squared_error(out.data_ptr(), y.data_ptr(), self.dz[self.L - 1].data_ptr(), self.loss.data_ptr(),
                          out.numel(), inv, inv, False, lib.BF16, self.sq_ws.data_ptr(), self.sq_ws_bytes, stream)
        self.launches += 1

    def _dz_below(self, i, stream):
        self._plans["below"][i].launch(stream)
        self.launches += 1

    def _grads(self, i, stream):
        """Layer i's bias gradient and weight gradient (applied in the product's epilogue when the update is
        fused, else left in dw[i])."""
        bf16 = lib.BF16
        fout = self.sizes[i + 1]
        lib.colsum(self.dz[i].data_ptr(), self.db[i].data_ptr(), self.batch, fout, fout, 1.0, bf16,
                   self.cs_ws.data_ptr(), self.cs_ws_bytes, stream)
        self._plans["grads"][i].launch(stream)
        self.launches += 3
        if self.fuse_update:
            lib.axpy(self.b[i].data_ptr(), self.db[i].data_ptr(), -self.rate, fout, bf16, bf16, stream)
            self.launches += 1

    def _exchange(self, j, cur):
        """Bucket j summed over the replicas on the side stream, once `cur` has produced it.
        Returns the event that marks the sum as landed (None on one GPU)."""
        if self.world == 1:
            return None
        torch = self.torch
        ready = torch.cuda.Event()
        ready.record(cur)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            if self._dp is not None:
                lib.dp_update(self._dp[j], self.comm_stream.cuda_stream)   # the sum and the update, every replica
                self.launches += 1
            else:
                torch.distributed.all_reduce(self.bucket[j], group=self.group)
            done = torch.cuda.Event()
            done.record(self.comm_stream)
        return done

    def _update(self, j, stream):
        """params[first:last] -= rate * grads[first:last]: every weight and bias of bucket j in one launch
        (nothing to do where the exchange kernel has already written the new parameters)."""
        if self._dp is not None:
            return
        first, last, _ = self.buckets[j]
        bf16 = lib.BF16
        lib.axpy(self.params.data_ptr() + 2 * first, self.grads.data_ptr() + 2 * first, -self.rate, last - first,
                 bf16, bf16, stream)
        self.launches += 1

    def capture_segments(self, x, y):
        """The data-parallel step with its own kernels recorded into CUDA graphs and the all-reduces left outside
        them: one graph per stretch between two exchanges, one per bucket's update, replayed on the current stream
        with NCCL's all-reduce launched eagerly on the side stream in between.  A replica then makes about ten host
        calls per step instead of forty, which is what eight Python processes on one host need to keep their GPUs
        fed.  No collective is ever inside a capture.  x and y are read in place at every replay.  Returns `replay()`."""
        if self.fuse_update:
            raise ValueError("capture_segments() is for data-parallel steps (unfused updates)")
        torch = self.torch
        side = torch.cuda.Stream()

        def record(body):
            graph = torch.cuda.CUDAGraph()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.graph(graph, stream=side):
                body(torch.cuda.current_stream().cuda_stream)
            torch.cuda.current_stream().wait_stream(side)
            return graph

        self.step(x, y)   # every launch and every NCCL connection once, outside any capture
        torch.cuda.synchronize()
        # cut the schedule where a bucket becomes complete: that is where its exchange is launched
        pieces, run = [], [("head", -1)]
        for kind, i in self._schedule():
            if kind == "exchange":
                pieces.append((i, run))
                run = []
            else:
                run.append((kind, i))

        def play(ops, st):
            for kind, i in ops:
                if kind == "head":
                    self._head(x, y, st)
                elif kind == "below":
                    self._dz_below(i, st)
                else:
                    self._grads(i, st)

        stretches = [(j, record(lambda st, ops=ops: play(ops, st))) for j, ops in pieces]
        # (with the fused exchange there is no separate update to record)
        updates = [record(lambda st, j=j: self._update(j, st)) if self._dp is None else None for j, _ in pieces]
        torch.cuda.synchronize()
        self._graphs = (stretches, updates)

        def replay():
            cur = torch.cuda.current_stream()
            events = []
            for j, graph in stretches:
                graph.replay()
                events.append(self._exchange(j, cur))
            # a bucket is applied as soon as its sum has landed, while later sums are still in flight
            for done, update in zip(events, updates):
                if done is not None:
                    cur.wait_event(done)
                if update is not None:
                    update.replay()
            return self.loss

        return replay

    def capture(self, x, y):
        """Records one single-GPU step into a CUDA graph, as Tempest captures a compiled call
        (ext/CUDAExt.jl:565-572), and returns `replay()`: one graph launch per step instead of some
        thirty kernel launches.  x and y are read in place at every replay; the loss lands in
        `self.loss`.  A data-parallel step is captured whole only with the fused exchange (its kernel is
        the library's own and is recorded like any other, on the side stream forked from and joined back
        into the recording; every replica must then replay the graph the same number of times, since the
        replicas meet inside it).  With NCCL the all-reduces stay outside any graph (`capture_segments`)."""
        if self.world != 1 and self._dp is None:
            raise ValueError("capture() records single-GPU steps, or data-parallel steps with the fused exchange")
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step(x, y)              # every launch once on the capturing stream before it is recorded
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            self.step(x, y)
        self._graph = graph
        return graph.replay
