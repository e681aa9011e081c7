#!/usr/bin/env python
"""Benchmark of the fused row-reduction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE.json configs[1]): softmax and LayerNorm (eps 1e-5, gamma 1,
beta 0) over X of Julia shape 4096 x 65536 (65536 rows of 4096 contiguous
elements), forward and autodiff backward, Float32 and BFloat16, X and the
upstream gradient ~ N(0,1), synthetic and seeded.  One step = the eight fused
kernels (4 operators x 2 element types) over the whole of X.

value  = algorithmic bytes of a step / device time of a step, inputs resident
         in HBM, summed over ranks (rows shard across GPUs with no exchange:
         weak scaling, every rank folds its own 65536 rows).
e2e    = the same through the plugin mirror with HOST buffers: every step
         copies X and dY from pinned host memory and reads every result back.
--impl reference times the CPU restatement of the reference's CPU path
         (oracle/) on the host cores over a bounded sample of the rows.

Prints one JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_REDUCE, ROWS = 4096, 65536
SEED = 20261125 + 2
METRIC, UNIT = "fused-kernel HBM GB/s", "GB/s"
WORKLOAD = "softmax+layernorm fwd+bwd, X 4096x65536, f32 and bf16"
# row-sized arrays each kernel reads + writes: the algorithmic traffic
STREAMS = {"softmax_fwd": 2, "softmax_bwd": 3, "layernorm_fwd": 2, "layernorm_bwd": 3}
CPU_SAMPLE_ROWS = 2048
# thread blocks (SMs) the fused gradient exchange occupies on each GPU (0 = the library's default)
DP_BLOCKS = int(os.environ.get("TB200_DP_BLOCKS", "0"))


def algorithmic_bytes(op, rows, size):
    extra = 0
    if op == "softmax_fwd":
        extra = rows * 4                      # the log-sum-exp saved for the backward
    elif op == "layernorm_fwd":
        extra = 2 * N_REDUCE * size + 2 * rows * 4   # gamma, beta; mean and rstd saved for the backward
    elif op == "layernorm_bwd":
        extra = 3 * N_REDUCE * size + 2 * rows * 4   # gamma, dgamma, dbeta; the saved mean and rstd
    return STREAMS[op] * N_REDUCE * rows * size + extra


def step_bytes(rows):
    return sum(algorithmic_bytes(op, rows, size) for op in STREAMS for size in (4, 2))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs", 6650.0), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.out = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.flush()
        self.out.seek(0)
        clocks, peak, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.out.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                peak = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        self.out.close()
        os.unlink(self.out.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak,
                "samples": len(clocks), "reasons": sorted(reasons)}


def physical_gpu_index(local):
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        ids = [v.strip() for v in visible.split(",") if v.strip()]
        if local < len(ids) and ids[local].isdigit():
            return int(ids[local])
    return local


# ------------------------------------------------------------------ GPU arm --

class Workload:
    """The eight launches of a step, built once through the plugin mirror
    (Binding -> build -> launch), as Tempest builds a plan's kernels once and
    replays them."""

    def __init__(self, torch, pkg, rows):
        I = pkg.implement
        self.torch, self.I, self.rows = torch, I, rows
        self.lib, self.target = I.B200Kernels(), I.Target()
        self.resources = self.lib.resources(self.target)
        gen = torch.Generator(device="cuda").manual_seed(SEED)
        n = N_REDUCE
        x32 = torch.randn(rows, n, device="cuda", generator=gen)
        g32 = torch.randn(rows, n, device="cuda", generator=gen)
        self.inputs = {"Float32": (x32, g32), "BFloat16": (x32.bfloat16(), g32.bfloat16())}
        self.launches = []   # (name, eltype, launch, algorithmic bytes)
        self.outputs = {}
        for eltype, (x, g) in self.inputs.items():
            size = x.element_size()
            w = torch.ones(n, device="cuda", dtype=x.dtype)
            b = torch.zeros(n, device="cuda", dtype=x.dtype)
            y, dx, yl, dxl = (torch.empty_like(x) for _ in range(4))
            lse = torch.empty(rows, device="cuda")
            mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
            dw, db = torch.empty_like(w), torch.empty_like(w)
            stat = lambda t, v: I.Strided("Float32", 0, (1, rows), (1, 1), t, v)  # noqa: E731
            self.outputs[eltype] = (y, dx, yl, dxl, lse, dw, db)
            col = lambda t, v: I.dense_columns(t, eltype, n, rows, v)  # noqa: E731
            vec = lambda t, v: I.dense_vector(t, eltype, n, v)         # noqa: E731
            plans = [
                ("softmax_fwd", "softmax_columns_lse",
                 {"x": col(x, 1), "y": col(y, 2), "lse": I.Strided("Float32", 0, (1, rows), (1, 1), lse, 3)}),
                ("softmax_bwd", "softmax_columns_pullback", {"y": col(y, 2), "g": col(g, 4), "dx": col(dx, 5)}),
                # the forward keeps each row's mean and rstd (8 bytes a row) and the backward reads them
                # instead of folding the row twice more: the planner's save-over-recompute choice
                ("layernorm_fwd", "layernorm_bias", {"x": col(x, 1), "w": vec(w, 6), "b": vec(b, 7), "y": col(yl, 8),
                                                     "mean": stat(mean, 12), "rstd": stat(rstd, 13)}),
                ("layernorm_bwd", "layernorm_pullback",
                 {"x": col(x, 1), "w": vec(w, 6), "g": col(g, 4), "dx": col(dxl, 9), "dw": vec(dw, 10),
                  "db": vec(db, 11), "mean": stat(mean, 12), "rstd": stat(rstd, 13)}),
            ]
            for name, template, arrays in plans:
                launch, _ = self.lib.build(self.target, I.Binding(template, {"n": n, "rows": rows}, arrays),
                                           self.resources)
                self.launches.append((name, eltype, launch, algorithmic_bytes(name, rows, size)))
        self.kernels_per_step = len(self.launches) + 2   # + the two dgamma/dbeta merge launches

    def step(self, events=None):
        for i, (_, _, launch, _) in enumerate(self.launches):
            if events is not None:
                events[i][0].record()
            launch()
            if events is not None:
                events[i][1].record()


def run_gpu(args):
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # NCCL's own account of what it runs (is the reduction done in the switch, which algorithm and protocol
        # its tuner picks) goes to a file per rank, set before the library is loaded; rank 0's is summarised
        # in the line's `dp.nccl`
        os.environ["NCCL_DEBUG"] = "INFO"
        os.environ["NCCL_DEBUG_SUBSYS"] = "INIT,TUNING,ENV"
        os.environ["NCCL_DEBUG_FILE"] = (os.path.join(tempfile.gettempdir(), f"tb200_nccl_{os.getpid()}.log")
                                         if os.environ.get("RANK", "0") == "0" else os.devnull)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the backend has no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    pkg.lib.load()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    rows = args.rows
    wl = Workload(torch, pkg, rows)
    nk = len(wl.launches)
    for _ in range(max(args.warmup, 3)):
        wl.step()
    barrier()

    sampler = ClockSampler(physical_gpu_index(local)) if rank == 0 else None
    if sampler:
        time.sleep(0.3)   # nvidia-smi takes a moment to start sampling
        for _ in range(3):
            wl.step()     # keep the clocks up while it does
    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nk)]
              for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for s in range(args.steps):
        wl.step(events[s])
    stop.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * step_bytes(rows) / (ms_per_step * 1e-3) / 1e9

    # per-kernel device time inside the timed region
    kernels = {}
    peak, peak_kind = measured_peaks()
    for i, (name, eltype, _, nbytes) in enumerate(wl.launches):
        ms = statistics.mean(events[s][i][0].elapsed_time(events[s][i][1]) for s in range(args.steps))
        gbs = nbytes / (ms * 1e-3) / 1e9
        kernels[f"{name}_{'f32' if eltype == 'Float32' else 'bf16'}"] = {
            "ms": round(ms, 4), "GB/s": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 4),
            "frac_of_8TBps": round(gbs / 8000.0, 4), "algorithmic_bytes": nbytes}
    dominant = max(kernels, key=lambda k: kernels[k]["ms"])
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": kernels[dominant]["GB/s"], "peak": peak,
                "peak_kind": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback",
                "unit": "GB/s", "frac": round(kernels[dominant]["GB/s"] / peak, 4),
                "traffic": load_traffic(dominant)}

    # end to end: host buffers in, host buffers out, through the same launches
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(torch, dist, wl, world, args)

    also = None
    if not args.no_also:
        try:
            also = run_also(torch, dist, pkg, world, rank, only=None if args.also == "all" else args.also)
        except Exception as err:  # the headline line must survive a failure of the side measurements
            also = {"error": repr(err)[:300]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(sample_rows=CPU_SAMPLE_ROWS, repeats=1)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD if rows == ROWS else f"reduced case: {rows} rows of {N_REDUCE}",
                   "rows_per_gpu": rows, "row_length": N_REDUCE,
                   "element_types": ["f32", "bf16"], "sharding": f"rows x{world}, no collective",
                   "l2": "inputs larger than L2 (each operand 0.5-1 GiB vs 126 MB)"},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
        "gpu_launches": wl.kernels_per_step * args.steps, "kernels": kernels,
        "dp": (also or {}).get("dp") if isinstance(also, dict) else None, "also": also,
    }
    print(json.dumps(line))


def nccl_notes(path):
    """What NCCL said it would run (its INFO lines, written to `path` by rank 0): whether NVLS (reduction
    in the switch) is available, and for each large all-reduce the algorithm, protocol and channels its tuner picked."""
    notes = {"nvls_available": None, "allreduce": {}}
    try:
        with open(path, errors="replace") as f:
            text = f.read()
    except OSError:
        return notes
    notes["nvls_available"] = "NVLS multicast support is available" in text
    for line in text.splitlines():
        if "AllReduce:" in line and " Algo " in line:
            tail = line.split("AllReduce:", 1)[1].strip()
            size = tail.split(" Bytes", 1)[0].strip()
            if size.isdigit() and int(size) >= (1 << 20):
                notes["allreduce"][size] = tail.split("->", 1)[-1].strip()
    return notes


def run_mlp(torch, dist, pkg, world, rank, timed, tensor_peak):
    """BASELINE.json configs[2]: the MLP training step (1024-4096-4096-4096-1024, GELU(tanh), bias, BFloat16, MSE,
    SGD 1e-3, batch 8192).  One GPU: the whole step replayed as one CUDA graph.  N GPUs: the global batch of
    8192 split N ways (strong scaling) and 8192 samples per replica (weak scaling), gradients summed by NCCL
    all-reduces of three flat buckets; before anything is timed one data-parallel step is checked against the
    whole-batch step on one GPU (`dp_parity`)."""
    sizes, gb = (1024, 4096, 4096, 4096, 1024), 8192
    L = pkg.lib
    flops = 2 * gb * (1024 * 4096 + 2 * 4096 * 4096 + 4096 * 1024) * 3 - 2 * gb * 1024 * 4096
    gen = torch.Generator(device="cuda").manual_seed(SEED + 40)
    gx = torch.randn(gb, sizes[0], device="cuda", generator=gen).bfloat16()     # the same global batch on every rank
    gy = torch.randn(gb, sizes[-1], device="cuda", generator=gen).bfloat16()

    # ---- one GPU, whole batch: the figure every efficiency below is taken against (every rank runs it)
    one = pkg.mlp.MLPStep(torch, sizes, gb, 1e-3, seed=1)
    start_w = one.params.clone()
    one.step(gx, gy)
    torch.cuda.synchronize()
    one_loss, one_w = float(one.loss.item()), one.params.clone()
    ms1 = timed(one.capture(gx, gy), 20, 5)
    out = {"mlp_train": {"steps_per_s": round(1000.0 / ms1, 1), "ms_per_step": round(ms1, 4), "n_gpus": 1,
                         "global_batch": gb, "TFLOP/s": round(flops / ms1 / 1e9, 1),
                         "frac_of_measured_bf16_peak": round(flops / ms1 / 1e9 / tensor_peak, 4),
                         "launch": "the whole step as one CUDA graph", "device_error": L.device_error()}}
    del one
    if world == 1:
        return out

    # ---- data parallel, strong: parity first
    per = gb // world
    lo, hi = pkg.mlp.shard_rows(gb, rank, world)
    x, y = gx[lo:hi].contiguous(), gy[lo:hi].contiguous()
    step = pkg.mlp.MLPStep(torch, sizes, per, 1e-3, world=world, global_batch=gb, seed=1)
    assert torch.equal(step.params.view(torch.int16), _relayout(torch, pkg, start_w, sizes, step).view(torch.int16))
    step.step(x, y)
    torch.cuda.synchronize()
    loss = step.loss.clone()
    nccl_w = step.params.clone()                            # after exactly one step, for the fused path's check below
    dist.all_reduce(loss)                                   # the replicas' shares of the global mean
    ref = step.params.clone()
    dist.broadcast(ref, src=0)
    apart = (step.params.view(torch.int16).int() - ref.view(torch.int16).int()).abs().max().float()
    dist.all_reduce(apart, op=dist.ReduceOp.MAX)
    want = _relayout(torch, pkg, one_w, sizes, step)
    # against the whole-batch step: sums in another order and gradients rounded to BFloat16 before the exchange,
    # so a weight may land one BFloat16 ulp away where the update crosses a rounding boundary (weights so close
    # to zero that the update decides their value are held to 2 % of the largest update instead)
    got_w, want_w = step.params.float(), want.float()
    largest_update = 1e-3 * float((want_w - _relayout(torch, pkg, start_w, sizes, step).float()).abs().max().item() / 1e-3)
    beyond = ((got_w - want_w).abs() - (2.0 ** -7 * want_w.abs() + 2e-2 * max(largest_update, 1e-12))).max()
    differing = (step.params.view(torch.int16) != want.view(torch.int16)).float().mean()
    parity = {"replicas_bit_equal": bool(apart.item() == 0.0),
              "loss_all_reduced": float(loss.item()), "loss_one_gpu_whole_batch": one_loss,
              "loss_rel_diff": abs(float(loss.item()) - one_loss) / abs(one_loss),
              "weights_within_one_bf16_ulp_of_one_gpu": bool(beyond.item() <= 0.0),
              "weights_frac_differing_from_one_gpu": round(float(differing.item()), 6),
              "device_error": L.device_error()}
    parity["ok"] = bool(parity["replicas_bit_equal"] and parity["loss_rel_diff"] <= 2e-3 and
                        parity["weights_within_one_bf16_ulp_of_one_gpu"] and parity["device_error"] == 0)
    del ref, got_w, one_w, start_w

    # ---- the exchange alone: the floor under any overlap
    def exchange_alone(buckets):
        def run():
            for b in buckets:
                dist.all_reduce(b)
        return run
    alone = {"all_buckets_ms": round(timed(exchange_alone(step.bucket), 20, 5), 4),
             "bucket_bytes": [b.numel() * 2 for b in step.bucket]}
    alone["per_bucket_ms"] = [round(timed(exchange_alone([b]), 20, 5), 4) for b in step.bucket]
    step.grads.zero_()

    # both launch forms are timed and the faster one is reported (both figures stay in the line)
    forms = {"ms_per_step_eager": round(timed(lambda: step.step(x, y), 20, 5), 4),
             "ms_per_step_stretch_graphs": round(timed(step.capture_segments(x, y), 20, 5), 4)}
    ms = min(forms.values())
    out["mlp_train_strong"] = {"steps_per_s": round(1000.0 / ms, 1), "ms_per_step": round(ms, 4), "n_gpus": world,
                               "global_batch": gb, "scaling": "strong", "TFLOP/s": round(flops / ms / 1e9, 1),
                               "gradient_allreduce_bytes": sum(alone["bucket_bytes"]), **forms,
                               "device_error": L.device_error()}
    del step
    # ---- the same with the library's own exchange: gradient sum + update as one kernel over NVLink
    fused, link = {}, None
    try:
        total = pkg.mlp.flat_layout(list(sizes), False)[2]
        link = pkg.dp.ReplicaLink(torch, total)
        fstep = pkg.mlp.MLPStep(torch, sizes, per, 1e-3, world=world, global_batch=gb, seed=1, link=link,
                                 exchange_blocks=DP_BLOCKS)
        fstep.step(x, y)
        torch.cuda.synchronize()
        dist.barrier()
        ref = fstep.params.clone()
        dist.broadcast(ref, src=0)
        same = (fstep.params.view(torch.int16) == ref.view(torch.int16)).all().float()
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        # one step from the same start: the NCCL path's weights (sum rounded to BFloat16, then the update) bit for bit
        equal_nccl = (fstep.params.view(torch.int16) == nccl_w.view(torch.int16)).float().mean()
        fbeyond = ((fstep.params.float() - want_w).abs() - (2.0 ** -7 * want_w.abs() + 2e-2 * max(largest_update, 1e-12))).max()
        fused["dp_parity"] = {"replicas_bit_equal": bool(same.item() == 1.0),
                              "weights_within_one_bf16_ulp_of_one_gpu": bool(fbeyond.item() <= 0.0),
                              "weights_frac_equal_to_nccl_path": round(float(equal_nccl.item()), 6),
                              "dp_error": L.dp_error(), "device_error": L.device_error()}
        fused["dp_parity"]["ok"] = bool(fused["dp_parity"]["replicas_bit_equal"] and fbeyond.item() <= 0.0
                                        and fused["dp_parity"]["dp_error"] == 0 and fused["dp_parity"]["device_error"] == 0)
        fused["multimem"] = link.multimem

        def fused_alone():
            for d in fstep._dp:
                L.dp_update(d, torch.cuda.current_stream().cuda_stream)
        fused["exchange_alone_ms"] = round(timed(fused_alone, 20, 5), 4)
        fforms = {"ms_per_step_eager": round(timed(lambda: fstep.step(x, y), 20, 5), 4),
                  "ms_per_step_stretch_graphs": round(timed(fstep.capture_segments(x, y), 20, 5), 4),
                  "ms_per_step_one_graph": round(timed(fstep.capture(x, y), 20, 5), 4)}
        fused["strong"] = {"ms_per_step": min(fforms.values()), **fforms}
        del fstep
        wf = pkg.mlp.MLPStep(torch, sizes, gb, 1e-3, world=world, global_batch=gb * world, seed=1, link=link,
                              exchange_blocks=DP_BLOCKS)
        wf.step(gx, gy)
        wfforms = {"ms_per_step_eager": round(timed(lambda: wf.step(gx, gy), 20, 5), 4),
                   "ms_per_step_stretch_graphs": round(timed(wf.capture_segments(gx, gy), 20, 5), 4),
                   "ms_per_step_one_graph": round(timed(wf.capture(gx, gy), 20, 5), 4)}
        fused["weak"] = {"ms_per_step": min(wfforms.values()), **wfforms}
        fused["dp_error"] = L.dp_error()
        del wf
    except Exception as err:   # no symmetric memory on this node, or a refusal: the NCCL figures stand alone
        fused["unavailable"] = repr(err)[:300]
    finally:
        if link is not None:
            link.close()
    del x, y, nccl_w, want, want_w
    # ---- weak: 8192 samples per replica, the same 84 MB exchange behind a whole single-GPU step
    wstep = pkg.mlp.MLPStep(torch, sizes, gb, 1e-3, world=world, global_batch=gb * world, seed=1)
    wstep.step(gx, gy)
    wforms = {"ms_per_step_eager": round(timed(lambda: wstep.step(gx, gy), 20, 5), 4),
              "ms_per_step_stretch_graphs": round(timed(wstep.capture_segments(gx, gy), 20, 5), 4)}
    wms = min(wforms.values())
    out["mlp_train_weak"] = {"steps_per_s": round(1000.0 / wms, 1), "ms_per_step": round(wms, 4), "n_gpus": world,
                             "global_batch": gb * world, "scaling": "weak",
                             "samples_per_s": round(gb * world * 1000.0 / wms, 1),
                             "TFLOP/s": round(flops * world / wms / 1e9, 1), **wforms,
                             "device_error": L.device_error()}
    del wstep
    out["dp"] = {
        "n_gpus": world, "one_gpu_ms_per_step": round(ms1, 4),
        "strong_ms_per_step": round(ms, 4), "strong_steps_per_s": round(1000.0 / ms, 1),
        "strong_efficiency": round(ms1 / (world * ms), 4),
        "weak_ms_per_step": round(wms, 4), "weak_efficiency": round(ms1 / wms, 4),
        "efficiency_against": "the one-GPU whole-batch step (one CUDA graph) timed in this same run on every rank, max over ranks",
        "launch": "the faster of: every kernel launched eagerly | one CUDA graph per stretch between two gradient "
                  "exchanges; NCCL all-reduces always eager on a side stream",
        "exchange": "NCCL all-reduce of three flat buckets, then y += alpha x (the default); `fused` = the library's "
                    "own kernel, which sums a bucket through the NVSwitch, applies the step and writes every replica",
        "fused": fused,
        "strong_efficiency_fused": round(ms1 / (world * fused["strong"]["ms_per_step"]), 4) if "strong" in fused else None,
        "weak_efficiency_fused": round(ms1 / fused["weak"]["ms_per_step"], 4) if "weak" in fused else None,
        "exchange_alone": alone, "dp_parity": parity,
        "nccl": nccl_notes(os.environ.get("NCCL_DEBUG_FILE", "")) if rank == 0 else None,
    }
    return out


def _relayout(torch, pkg, flat, sizes, step):
    """The parameters of a single-GPU step's flat buffer (layers in order) copied into the layout of `step`."""
    order, offsets, total, _ = pkg.mlp.flat_layout(list(sizes), True)
    out = torch.zeros_like(step.params)
    for i in range(len(sizes) - 1):
        nw, nb = sizes[i] * sizes[i + 1], sizes[i + 1]
        out[step.offsets[i][0]: step.offsets[i][0] + nw] = flat[offsets[i][0]: offsets[i][0] + nw]
        out[step.offsets[i][1]: step.offsets[i][1] + nb] = flat[offsets[i][1]: offsets[i][1] + nb]
    return out


def run_also(torch, dist, pkg, world, rank, only=None):
    """Side measurements of the other kernel families on the same box (not the headline value):
    the MLP training step of BASELINE.json configs[2] (1024-4096-4096-4096-1024, GELU(tanh), bias,
    BFloat16, MSE, SGD 1e-3), global batch 8192 sharded over the ranks with an NCCL all-reduce of the
    gradients (strong scaling), and its largest product alone."""
    sizes, gb = (1024, 4096, 4096, 4096, 1024), 8192
    per = gb // world
    tensor_peak = 1676.5
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            tensor_peak = json.load(f).get("bf16_tflops", tensor_peak)
    L = pkg.lib

    def timed(fn, iters, warm):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    out = run_mlp(torch, dist, pkg, world, rank, timed, tensor_peak)
    if only == "mlp":
        return out
    if rank == 0 or world == 1:
        M, N, K = 8192, 4096, 4096
        A = torch.randn(M, K, device="cuda").bfloat16()
        B = torch.randn(K, N, device="cuda").bfloat16()
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        bias = torch.zeros(N, device="cuda", dtype=torch.bfloat16)
        Z = torch.empty_like(C)
        stream = torch.cuda.current_stream().cuda_stream

        def gemm():
            L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, a_layout=L.K_MAJOR, b_layout=L.MN_MAJOR,
                   epilogue=L.EPI_BIAS_GELU, bias=bias.data_ptr(), aux_out=Z.data_ptr(), stream=stream)
        for _ in range(3):
            gemm()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            gemm()
        b.record()
        torch.cuda.synchronize()
        gms = a.elapsed_time(b) / 20
        tf = 2.0 * M * N * K / gms / 1e9
        # the incumbent on the same box, same shape, same minute: the plain product by cuBLAS (torch.matmul),
        # with no bias, no activation and no second array to store
        for _ in range(3):
            torch.matmul(A, B, out=C)
        torch.cuda.synchronize()
        a.record()
        for _ in range(20):
            torch.matmul(A, B, out=C)
        b.record()
        torch.cuda.synchronize()
        cms = a.elapsed_time(b) / 20
        ctf = 2.0 * M * N * K / cms / 1e9

        def plain():
            L.gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, a_layout=L.K_MAJOR, b_layout=L.MN_MAJOR,
                   stream=stream)
        for _ in range(3):
            plain()
        torch.cuda.synchronize()
        a.record()
        for _ in range(20):
            plain()
        b.record()
        torch.cuda.synchronize()
        pms = a.elapsed_time(b) / 20
        out["gemm_bias_gelu_8192x4096x4096"] = {"TFLOP/s": round(tf, 1), "ms": round(gms, 4),
                                                "frac_of_measured_bf16_peak": round(tf / tensor_peak, 4),
                                                "plain_product_TFLOP/s": round(2.0 * M * N * K / pms / 1e9, 1),
                                                "cublas_plain_product_TFLOP/s": round(ctf, 1),
                                                "cublas_plain_product_ms": round(cms, 4)}

        def clock(fn, iters):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / iters

        # BASELINE.json configs[3]: causal attention, B=8, H=32, S=4096, D=128, BFloat16, forward + backward
        Bq, Hq, Sq, Dq = 8, 32, 4096, 128
        q, k, v, g = (torch.randn(Bq, Sq, Hq, Dq, device="cuda").bfloat16() for _ in range(4))
        o, lse = torch.empty_like(q), torch.empty(Bq, Sq, Hq, device="cuda")
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        desc = L.attn_desc(Bq, Hq, Sq, Sq, Dq, True)
        need = L.attention_bwd_workspace_bytes(desc)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        def launches(fn, warm, iters):
            """Per-launch device times (CUDA events around every launch), after `warm` untimed launches."""
            for _ in range(warm):
                fn()
            torch.cuda.synchronize()
            marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
            for a0, b0 in marks:
                a0.record()
                fn()
                b0.record()
            torch.cuda.synchronize()
            return sorted(a0.elapsed_time(b0) for a0, b0 in marks)

        watch = ClockSampler(physical_gpu_index(int(os.environ.get("LOCAL_RANK", "0"))))
        fwd_ms = launches(lambda: L.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                                  lse.data_ptr(), stream), 6, 30)
        bwd_forms = {}
        for name, det in (("atomic", 0), ("deterministic", 1)):
            desc.deterministic = det
            bwd_forms[name] = launches(
                lambda: L.attention_bwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                        g.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need,
                                        stream), 5, 30)
        attn_clocks = watch.stop()
        fwd = fwd_ms[len(fwd_ms) // 2]
        # the pullback's form is the tuner's pick between the library's two schedules (both figures stay in the line)
        picked = L.attention_bwd_tune(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                      g.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need, stream)
        best_form = "deterministic" if picked == 1 else "atomic"
        bwd = bwd_forms[best_form][15]
        fl = 4.0 * Bq * Hq * Sq * Sq * Dq * 0.5
        mhz = attn_clocks.get("sm_mhz") or 0.0
        out["attention_causal_B8_H32_S4096_D128"] = {
            "fwd_ms": round(fwd, 4), "fwd_TFLOP/s": round(fl / fwd / 1e9, 1),
            "fwd_frac_of_measured_bf16_peak": round(fl / fwd / 1e9 / tensor_peak, 4),
            "fwd_ms_min": round(fwd_ms[0], 4),
            "bwd_ms": round(bwd, 4), "bwd_TFLOP/s": round(2.5 * fl / bwd / 1e9, 1),
            "bwd_frac_of_measured_bf16_peak": round(2.5 * fl / bwd / 1e9 / tensor_peak, 4),
            "bwd_ms_min": round(bwd_forms[best_form][0], 4),
            "bwd_form": best_form + " (picked by tb200_attention_bwd_tune)",
            "bwd_deterministic_ms": round(bwd_forms["deterministic"][15], 4),
            "bwd_deterministic_TFLOP/s": round(2.5 * fl / bwd_forms["deterministic"][15] / 1e9, 1),
            "bwd_atomic_ms": round(bwd_forms["atomic"][15], 4),
            "bwd_atomic_TFLOP/s": round(2.5 * fl / bwd_forms["atomic"][15] / 1e9, 1),
            "timing": "median of 30 launches, each between its own CUDA events, after 5-6 untimed launches",
            "sm_mhz_median": mhz, "fwd_ms_x_mhz": round(fwd * mhz, 1), "bwd_ms_x_mhz": round(bwd * mhz, 1),
            "clock_reasons": attn_clocks.get("reasons"),
            "bwd_note": "algorithmic 5 products (2.5 x forward) in both forms; the one-kernel (atomic) form executes 5 and "
                        "adds dq into a Float32 workspace (memset + rounding kernel included in its time), the "
                        "deterministic two-kernel form executes 7",
            "device_error": L.attention_device_error() + L.attention_bwd_device_error()}
        # the same arrays as four packed documents of 1024 positions a sequence, the starts held on the device
        # (the reference's packed-documents program, test/cuda/attention.jl:217-246): forward and pullback on the
        # tensor cores; work counted over the visible (query, key) pairs
        docs = torch.arange(Sq, device="cuda", dtype=torch.int32) // 1024 * 1024
        starts = docs.repeat(Bq, 1).contiguous()
        mask = L.attn_mask(doc_start=starts.data_ptr())
        desc.deterministic = 0
        mneed = L.attention_bwd_masked_workspace_bytes(desc)
        mws = torch.empty(mneed, dtype=torch.uint8, device="cuda")
        mf = clock(lambda: L.attention_fwd_masked(desc, mask, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                                  lse.data_ptr(), stream), 5)
        mb = clock(lambda: L.attention_bwd_masked_ws(desc, mask, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                                     lse.data_ptr(), g.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                                     dv.data_ptr(), mws.data_ptr(), mneed, stream), 5)
        visible = 4.0 * Bq * Hq * Dq * 4 * (1024 * 1025 / 2)
        out["attention_packed_documents_B8_H32_S4096_D128"] = {
            "documents": "4 x 1024 positions a sequence, starts on the device",
            "fwd_ms": round(mf, 4), "fwd_TFLOP/s_of_visible_pairs": round(visible / mf / 1e9, 1),
            "bwd_ms": round(mb, 4), "bwd_TFLOP/s_of_visible_pairs": round(2.5 * visible / mb / 1e9, 1),
            "note": "forward: the one-tile tensor-core kernel, key tiles before a document's start skipped; pullback: the "
                    "one-kernel form, each tile's steps cut to the chunks that can see it",
            "device_error": L.attention_device_error() + L.attention_bwd_device_error()}
        del q, k, v, g, o, dq, dk, dv, ws, mws, starts
        # BASELINE.json configs[4]: chunked gated DeltaNet forward, B*H = 64 sequences of 8192, dk = dv = 128
        Hn, T = 64, 8192
        qd = torch.nn.functional.normalize(torch.randn(Hn, T, 128, device="cuda"), dim=-1).bfloat16()
        kd = torch.nn.functional.normalize(torch.randn(Hn, T, 128, device="cuda"), dim=-1).bfloat16()
        vd = torch.randn(Hn, T, 128, device="cuda").bfloat16()
        ad = -torch.nn.functional.softplus(torch.randn(Hn, T, device="cuda"))
        bd = torch.sigmoid(torch.randn(Hn, T, device="cuda"))
        od = torch.empty(Hn, 128, T, device="cuda", dtype=torch.bfloat16)
        dd = L.deltanet_desc(Hn, T)
        dneed = L.deltanet_workspace_bytes(dd)
        dws = torch.empty(dneed, dtype=torch.uint8, device="cuda")
        dms = clock(lambda: L.deltanet_fwd(dd, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ad.data_ptr(), bd.data_ptr(),
                                           od.data_ptr(), dws.data_ptr(), dneed, stream), 5)
        dbytes = 4 * Hn * T * 128 * 2 + 2 * Hn * T * 4
        hbm, _ = measured_peaks()
        out["deltanet_fwd_B4_H16_S8192"] = {"ms": round(dms, 4), "algorithmic_GB/s": round(dbytes / dms / 1e6, 1),
                                            "frac_of_measured_hbm_peak": round(dbytes / dms / 1e6 / hbm, 4)}
        del od
        # the generic term-interpreter kernel on the headline shape: softmax and RMSNorm spelled as groups
        G = pkg.groups
        n, rows = 4096, 65536
        xg = torch.randn(rows, n, device="cuda")
        yg, lg = torch.empty_like(xg), torch.empty(rows, device="cuda")
        sm = G.softmax(n, rows)
        smd = sm.desc()
        gms = clock(lambda: L.rowreduce_generic(smd, [xg.data_ptr()], [yg.data_ptr(), lg.data_ptr()], stream), 5)
        out["generic_softmax_f32_4096x65536"] = {"ms": round(gms, 4), "algorithmic_GB/s": round(sm.bytes() / gms / 1e6, 1),
                                                 "frac_of_measured_hbm_peak": round(sm.bytes() / gms / 1e6 / hbm, 4)}
        for name, group, ins, outs in (
                ("compiled_softmax_f32", sm, [xg.data_ptr()], [yg.data_ptr(), lg.data_ptr()]),
                ("compiled_log_softmax_f32", G.log_softmax(n, rows), [xg.data_ptr()], [yg.data_ptr()])):
            gd = group.desc()
            gms = clock(lambda: L.rowreduce_compiled(gd, ins, outs, stream), 10)
            out[name + "_4096x65536"] = {"ms": round(gms, 4), "algorithmic_GB/s": round(group.bytes() / gms / 1e6, 1),
                                         "frac_of_measured_hbm_peak": round(group.bytes() / gms / 1e6 / hbm, 4)}
        xb, wb = xg.bfloat16(), torch.randn(n, device="cuda").bfloat16()
        yb = torch.empty_like(xb)
        rn = G.rmsnorm(n, rows, "BFloat16")
        rnd = rn.desc()
        gms = clock(lambda: L.rowreduce_generic(rnd, [xb.data_ptr(), wb.data_ptr()], [yb.data_ptr()], stream), 5)
        out["generic_rmsnorm_bf16_4096x65536"] = {"ms": round(gms, 4), "algorithmic_GB/s": round(rn.bytes() / gms / 1e6, 1),
                                                  "frac_of_measured_hbm_peak": round(rn.bytes() / gms / 1e6 / hbm, 4)}
        gms = clock(lambda: L.rowreduce_compiled(rnd, [xb.data_ptr(), wb.data_ptr()], [yb.data_ptr()], stream), 10)
        out["compiled_rmsnorm_bf16_4096x65536"] = {"ms": round(gms, 4), "algorithmic_GB/s": round(rn.bytes() / gms / 1e6, 1),
                                                   "frac_of_measured_hbm_peak": round(rn.bytes() / gms / 1e6 / hbm, 4)}
        bb = torch.randn(n, device="cuda").bfloat16()
        ln = G.layernorm(n, rows, "BFloat16")
        lnd = ln.desc()
        gms = clock(lambda: L.rowreduce_compiled(lnd, [xb.data_ptr(), wb.data_ptr(), bb.data_ptr()], [yb.data_ptr()], stream), 10)
        out["compiled_layernorm_bf16_4096x65536"] = {"ms": round(gms, 4), "algorithmic_GB/s": round(ln.bytes() / gms / 1e6, 1),
                                                     "frac_of_measured_hbm_peak": round(ln.bytes() / gms / 1e6 / hbm, 4)}
        # a group that folds the other axis: the bias gradient of a (4096, 65536) BFloat16 activation gradient
        bg = G.bias_gradient(n, rows, "BFloat16")
        bgd = bg.desc()
        cneed = L.colreduce_workspace_bytes(bgd)
        cws2 = torch.empty(max(cneed, 16), dtype=torch.uint8, device="cuda")
        gms = clock(lambda: L.colreduce_compiled(bgd, [xb.data_ptr()], [wb.data_ptr()], cws2.data_ptr(), cneed, stream), 10)
        cb = bg.bytes()
        out["compiled_bias_gradient_bf16_4096x65536"] = {"ms": round(gms, 4), "algorithmic_GB/s": round(cb / gms / 1e6, 1),
                                                         "frac_of_measured_hbm_peak": round(cb / gms / 1e6 / hbm, 4)}
        del xg, yg, xb, yb, cws2
        # scans and a recurrence whose step is a map, 16384 rows of 4096 Float32 (268 MB an array)
        sn, srows = 4096, 16384
        sx = torch.randn(srows, sn, device="cuda")
        sy = torch.empty_like(sx)
        sneed = L.scan_workspace_bytes(L.scan_desc(sn, srows, L.SCAN_SUM, across=True))
        sws = torch.empty(max(sneed, 16), dtype=torch.uint8, device="cuda")
        along = clock(lambda: L.scan(sx.data_ptr(), sy.data_ptr(), sn, srows, L.SCAN_SUM, stream=stream), 5)
        across = clock(lambda: L.scan(sx.data_ptr(), sy.data_ptr(), sn, srows, L.SCAN_SUM, across=True,
                                      workspace=sws.data_ptr(), workspace_bytes=sneed, stream=stream), 5)
        cell = pkg.groups.gated_tanh_cell(1 << 20, 64)
        ca, ch = torch.full((1 << 20,), 0.7, device="cuda"), torch.zeros(1 << 20, device="cuda")
        cl = torch.empty_like(ch)
        cdesc = cell.desc()
        rec = clock(lambda: L.recurrence_compiled(cdesc, [sx.data_ptr(), ca.data_ptr(), ch.data_ptr()],
                                                  [sy.data_ptr(), cl.data_ptr()], stream), 5)
        sb = 2.0 * sx.numel() * 4
        out["scans_f32_16384x4096"] = {
            "cumsum_along_rows_GB/s": round(sb / along / 1e6, 1), "cumsum_across_rows_in_slabs_GB/s": round(sb / across / 1e6, 1),
            "map_recurrence_tanh_cell_2^20x64_GB/s": round(cell.bytes() / rec / 1e6, 1),
            "frac_of_measured_hbm_peak": [round(sb / along / 1e6 / hbm, 4), round(sb / across / 1e6 / hbm, 4),
                                          round(cell.bytes() / rec / 1e6 / hbm, 4)]}
        del sx, sy, sws, ca, ch, cl
        # its pullback at the same size (forward recomputed inside)
        gq, gk, gv = (torch.empty(Hn, T, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        ga, gb = torch.empty(Hn, T, device="cuda"), torch.empty(Hn, T, device="cuda")
        god = torch.randn(Hn, 128, T, device="cuda").bfloat16()
        bneed = L.deltanet_bwd_workspace_bytes(dd)
        del dws
        bws = torch.empty(bneed, dtype=torch.uint8, device="cuda")
        bms = clock(lambda: L.deltanet_bwd(dd, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ad.data_ptr(), bd.data_ptr(),
                                           god.data_ptr(), gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), ga.data_ptr(),
                                           gb.data_ptr(), bws.data_ptr(), bneed, stream), 5)
        bbytes = 7 * Hn * T * 128 * 2 + 4 * Hn * T * 4
        out["deltanet_bwd_B4_H16_S8192"] = {"ms": round(bms, 4), "algorithmic_GB/s": round(bbytes / bms / 1e6, 1),
                                            "workspace_GB": round(bneed / 1e9, 2)}
    return out


def run_profile_case(args):
    """One small case of a kernel family and nothing else, for ncu captures (not a benchmark):
    few launches before the captured ones, a few GB on the device at most."""
    import torch
    import __graft_entry__ as entry
    torch.cuda.set_device(0)
    pkg = entry.load_package()
    L = pkg.lib
    L.load()
    stream = torch.cuda.current_stream().cuda_stream
    case = args.profile_case
    if case == "gemm":
        M, N, K = 8192, 4096, 4096
        A = torch.randn(M, K, device="cuda").bfloat16()
        B = torch.randn(K, N, device="cuda").bfloat16()
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        bias = torch.zeros(N, device="cuda", dtype=torch.bfloat16)
        Z = torch.empty_like(C)
        # the forward product as a prepared launch (tiles drawn from a counter), three times
        plan = L.GemmPlan(L.gemm_desc(M, N, K, a_layout=L.K_MAJOR, b_layout=L.MN_MAJOR, epilogue=L.EPI_BIAS_GELU),
                          A.data_ptr(), B.data_ptr(), C.data_ptr(), bias=bias.data_ptr(), aux_out=Z.data_ptr())
        for _ in range(3):
            plan.launch(stream)
        # the backward's shapes: dX (both K-major) and dW (both MN-major)
        L.gemm(C.data_ptr(), B.data_ptr(), A.data_ptr(), M, K, N, a_layout=L.K_MAJOR, b_layout=L.K_MAJOR,
               epilogue=L.EPI_MUL_GELU_GRAD, aux=Z.data_ptr(), stream=stream)
        L.gemm(A.data_ptr(), C.data_ptr(), B.data_ptr(), K, N, M, a_layout=L.MN_MAJOR, b_layout=L.MN_MAJOR,
               stream=stream)
        # a long sum over a small output, split among blocks and merged (the reference's split-K shape, scaled up),
        # and a batch of the delta rule's per-chunk products
        sd = L.gemm_desc(64, 48, 30000, a_layout=L.K_MAJOR, b_layout=L.MN_MAJOR, out_dtype=L.F32)
        need = L.gemm_workspace_bytes(sd)
        sws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        As, Bs = torch.randn(64, 30000, device="cuda").bfloat16(), torch.randn(30000, 48, device="cuda").bfloat16()
        Cs = torch.empty(64, 48, device="cuda")
        L.gemm(As.data_ptr(), Bs.data_ptr(), Cs.data_ptr(), 64, 48, 30000, out_dtype=L.F32, workspace=sws.data_ptr(),
               workspace_bytes=need, stream=stream)
        Ab, Bb = torch.randn(2048, 64, 128, device="cuda").bfloat16(), torch.randn(2048, 64, 128, device="cuda").bfloat16()
        Cb = torch.empty(2048, 64, 64, device="cuda", dtype=torch.bfloat16)
        L.gemm(Ab.data_ptr(), Bb.data_ptr(), Cb.data_ptr(), 64, 64, 128, a_layout=L.K_MAJOR, b_layout=L.K_MAJOR, batch=2048,
               stream=stream)
        plan.close()
    elif case == "scan":
        n, rows = 4096, 16384
        x = torch.randn(rows, n, device="cuda")
        y = torch.empty_like(x)
        a = 0.9 + 0.1 * torch.rand(rows, n, device="cuda")
        need = L.scan_workspace_bytes(L.scan_desc(n, rows, L.SCAN_SUM, across=True))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        # a recurrence whose step is a map, h = tanh(a h + x) with h stored: 2^20 positions, 64 steps
        cell = pkg.groups.gated_tanh_cell(1 << 20, 64)
        cx = torch.randn(64, 1 << 20, device="cuda")
        ca, ch = torch.full((1 << 20,), 0.7, device="cuda"), torch.zeros(1 << 20, device="cuda")
        cy, cl = torch.empty_like(cx), torch.empty_like(ch)
        for _ in range(2):
            L.scan(x.data_ptr(), y.data_ptr(), n, rows, L.SCAN_SUM, stream=stream)
            L.scan(x.data_ptr(), y.data_ptr(), n, rows, L.SCAN_SUM, across=True, workspace=ws.data_ptr(),
                   workspace_bytes=need, stream=stream)
            L.scan(a.data_ptr(), y.data_ptr(), n, rows, L.SCAN_AFFINE, x2=x.data_ptr(), stream=stream)
            L.recurrence_compiled(cell.desc(), [cx.data_ptr(), ca.data_ptr(), ch.data_ptr()], [cy.data_ptr(), cl.data_ptr()],
                                  stream)
    elif case == "attention":
        Bq, Hq, Sq, Dq = 1, 32, 4096, 128
        q, k, v, g = (torch.randn(Bq, Sq, Hq, Dq, device="cuda").bfloat16() for _ in range(4))
        o, lse = torch.empty_like(q), torch.empty(Bq, Sq, Hq, device="cuda")
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        desc = L.attn_desc(Bq, Hq, Sq, Sq, Dq, True)
        need = L.attention_bwd_workspace_bytes(desc)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        for _ in range(2):
            L.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), stream)
            for form in (0, 1):   # the one-kernel form (dq by atomic adds), then the deterministic two-kernel form
                desc.deterministic = form
                L.attention_bwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), g.data_ptr(),
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), need, stream)
            desc.deterministic = 0
    elif case == "deltanet":
        Hn, T = 16, 8192
        qd = torch.nn.functional.normalize(torch.randn(Hn, T, 128, device="cuda"), dim=-1).bfloat16()
        kd = torch.nn.functional.normalize(torch.randn(Hn, T, 128, device="cuda"), dim=-1).bfloat16()
        vd = torch.randn(Hn, T, 128, device="cuda").bfloat16()
        ad = -torch.nn.functional.softplus(torch.randn(Hn, T, device="cuda"))
        bd = torch.sigmoid(torch.randn(Hn, T, device="cuda"))
        od = torch.empty(Hn, 128, T, device="cuda", dtype=torch.bfloat16)
        dd = L.deltanet_desc(Hn, T)
        need = L.deltanet_workspace_bytes(dd)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        for _ in range(2):
            L.deltanet_fwd(dd, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ad.data_ptr(), bd.data_ptr(), od.data_ptr(),
                           ws.data_ptr(), need, stream)
        # the pullback: the forward's two kernels again (keeping states) and three of its own
        gq, gk, gv = (torch.empty(Hn, T, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        ga, gb = torch.empty(Hn, T, device="cuda"), torch.empty(Hn, T, device="cuda")
        god = torch.randn(Hn, 128, T, device="cuda").bfloat16()
        bneed = L.deltanet_bwd_workspace_bytes(dd)
        bws = torch.empty(bneed, dtype=torch.uint8, device="cuda")
        L.deltanet_bwd(dd, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ad.data_ptr(), bd.data_ptr(), god.data_ptr(),
                       gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), ga.data_ptr(), gb.data_ptr(), bws.data_ptr(), bneed, stream)
    elif case == "groups":
        # map -> fold row groups, 16384 rows of 4096: the term interpreter and the groups' own compiled kernels
        G = pkg.groups
        n, rows = 4096, 16384
        x = torch.randn(rows, n, device="cuda")
        y, lse = torch.empty_like(x), torch.empty(rows, device="cuda")
        xb = x.bfloat16()
        yb = torch.empty_like(xb)
        w = torch.randn(n, device="cuda")
        wb = w.bfloat16()
        cases = [(G.softmax(n, rows), [x], [y, lse]),
                 (G.layernorm(n, rows), [x, w, w], [y]),
                 (G.softmax(n, rows, "BFloat16"), [xb], [yb, lse]),
                 (G.layernorm(n, rows, "BFloat16"), [xb, wb, wb], [yb]),
                 (G.rmsnorm(n, rows, "BFloat16"), [xb, wb], [yb])]
        for _ in range(2):
            for group, ins, outs in cases:
                L.rowreduce_compiled(group.desc(), [t.data_ptr() for t in ins], [t.data_ptr() for t in outs], stream)
        group, ins, outs = cases[0]
        L.rowreduce_generic(group.desc(), [t.data_ptr() for t in ins], [t.data_ptr() for t in outs], stream)
    elif case == "columns":
        # groups that fold the other axis, 16384 rows of 4096: LayerNorm's weight gradients (Float32) and the
        # bias gradient (BFloat16), each as partial folds per slab + ordered merge
        G = pkg.groups
        n, rows = 4096, 16384
        x, dy = torch.randn(rows, n, device="cuda"), torch.randn(rows, n, device="cuda")
        mean, rstd = torch.randn(rows, device="cuda"), torch.rand(rows, device="cuda") + 0.5
        o1, o2 = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
        xb, ob = x.bfloat16(), torch.empty(n, device="cuda", dtype=torch.bfloat16)
        cases = [(G.layernorm_weight_gradients(n, rows), [x, dy, mean, rstd], [o1, o2]),
                 (G.bias_gradient(n, rows, "BFloat16"), [xb], [ob])]
        need = max(L.colreduce_workspace_bytes(g.desc()) for g, _, _ in cases)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        for _ in range(2):
            for group, ins, outs in cases:
                L.colreduce_compiled(group.desc(), [t.data_ptr() for t in ins], [t.data_ptr() for t in outs], ws.data_ptr(),
                                     need, stream)
    else:
        raise SystemExit(f"unknown profile case {case}")
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": case, "device_error": L.device_error() + L.attention_device_error() +
                      L.attention_bwd_device_error()}))


def load_traffic(kernel):
    """DRAM bytes per launch of `kernel` from the committed ncu summary, if there is one."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get(kernel)
    return None


def run_e2e(torch, dist, wl, world, args):
    """Every step: X and dY from pinned host memory to the device, the eight
    kernels, every result back to pinned host memory."""
    rows, n = wl.rows, N_REDUCE
    host_in, dev_in = {}, {}
    for eltype, (x, g) in wl.inputs.items():
        host_in[eltype] = (torch.empty(x.shape, dtype=x.dtype, pin_memory=True).copy_(x),
                           torch.empty(g.shape, dtype=g.dtype, pin_memory=True).copy_(g))
        dev_in[eltype] = (x, g)
    # results land in one pinned buffer per element type, one after another
    host_out = {e: torch.empty(wl.inputs[e][0].shape, dtype=wl.inputs[e][0].dtype, pin_memory=True)
                for e in wl.inputs}
    host_small = torch.empty(rows, dtype=torch.float32, pin_memory=True)
    host_vec = {e: torch.empty(n, dtype=wl.inputs[e][0].dtype, pin_memory=True) for e in wl.inputs}
    h2d = sum(t.numel() * t.element_size() for pair in host_in.values() for t in pair)
    d2h = 0
    for eltype, outs in wl.outputs.items():
        d2h += sum(t.numel() * t.element_size() for t in outs)

    # Three streams, as a host that feeds the kernels would run them: inputs arrive on a copy-in stream, each
    # kernel waits only for the operands it reads, and each result leaves on a copy-out stream as soon as its
    # kernel has finished -- PCIe carries both directions at once.  A step still contains every byte in and out.
    compute = torch.cuda.current_stream()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    # what each launch of wl.launches reads first, and which results it completes (names of wl.outputs' slots)
    reads = {"softmax_fwd": 0, "softmax_bwd": 1, "layernorm_fwd": 0, "layernorm_bwd": 1}
    writes = {"softmax_fwd": (0, 4), "softmax_bwd": (1,), "layernorm_fwd": (2,), "layernorm_bwd": (3, 5, 6)}

    # The results are twice the inputs' bytes, so the copies out set the step's time and the step is shortest
    # when the first of them starts early: the narrower element type, whose operands arrive first, goes first.
    order = sorted(wl.inputs, key=lambda e: wl.inputs[e][0].element_size())
    launches = sorted(wl.launches, key=lambda entry: order.index(entry[1]))   # stable: each type's own order kept

    def one_step():
        copy_in.wait_stream(compute)          # the previous step's kernels are done with the input buffers
        arrived = {}
        with torch.cuda.stream(copy_in):
            for eltype in order:
                for slot in (0, 1):
                    dev_in[eltype][slot].copy_(host_in[eltype][slot], non_blocking=True)
                    arrived[(eltype, slot)] = copy_in.record_event()
        for name, eltype, launch, _ in launches:
            compute.wait_event(arrived[(eltype, reads[name])])
            launch()
            done = compute.record_event()
            outs = wl.outputs[eltype]
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                for slot in writes[name]:
                    t = outs[slot]
                    target = host_out[eltype] if slot < 4 else host_small if slot == 4 else host_vec[eltype]
                    target.copy_(t, non_blocking=True)
        compute.wait_stream(copy_out)         # the step ends when its last result is on the host

    steps = max(1, min(args.steps, args.e2e_steps))
    one_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one_step()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return {"value": round(world * step_bytes(rows) / (ms * 1e-3) / 1e9, 2), "unit": UNIT,
            "ms_per_step": round(ms, 3), "steps": steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}


# ------------------------------------------------------------------ CPU arm --

def cpu_step(O, arrays, threads):
    """The same eight operators on the host, as the reference's CPU path runs
    them (BFloat16 rounding every operation), over the sampled rows."""
    for eltype in ("f32", "bf16"):
        x, g, w, b = arrays[eltype]
        y, _ = O.softmax_fwd(x, faithful=True, threads=threads)
        O.softmax_bwd(y, g, faithful=True, threads=threads)
        O.layernorm_fwd(x, w, b, faithful=True, threads=threads)
        O.layernorm_bwd(x, w, g, threads=threads)


def cpu_arrays(O, rows):
    import numpy as np
    x = O.normal((rows, N_REDUCE), SEED)
    g = O.normal((rows, N_REDUCE), SEED + 1)
    w, b = np.ones(N_REDUCE, np.float32), np.zeros(N_REDUCE, np.float32)
    return {"f32": (x, g, w, b), "bf16": tuple(O.to_bf16(a) for a in (x, g, w, b))}


def cpu_baseline(sample_rows, repeats):
    import __graft_entry__ as entry
    O = entry.load_oracle()
    O.build()
    threads = O.threads_available()
    arrays = cpu_arrays(O, sample_rows)
    cpu_step(O, cpu_arrays(O, 64), threads)   # touch the code once
    t0 = time.perf_counter()
    for _ in range(repeats):
        cpu_step(O, arrays, threads)
    dt = (time.perf_counter() - t0) / repeats
    return {"value": round(step_bytes(sample_rows) / dt / 1e9, 4), "unit": UNIT, "cores": threads, "kind": "port",
            "seconds_per_sample": round(dt, 3),
            "sample": f"{sample_rows} of {ROWS} rows of the same workload (all 8 operators), rows over "
                      f"{threads} host threads; the reference's CPU path itself runs on one thread "
                      "(timed here as the C restatement in oracle/: no Julia runtime on this host)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import __graft_entry__ as entry
    O = entry.load_oracle()
    O.build()
    threads = O.threads_available()
    rows = CPU_SAMPLE_ROWS
    arrays = cpu_arrays(O, rows)
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_step(O, arrays, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(O, arrays, threads)
    dt = (time.perf_counter() - t0) / args.steps
    value = round(step_bytes(rows) / dt / 1e9, 4)
    sample = (f"each step = {rows} of {ROWS} rows of the same workload (all 8 operators); rows spread over "
              f"{threads} host threads; the reference's CPU path itself is single-threaded")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_step": rows, "row_length": N_REDUCE,
                   "element_types": ["f32", "bf16"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS, help="rows per GPU (smaller only for profiling captures)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the side measurements (MLP step, GEMM)")
    ap.add_argument("--also", default="all", choices=["all", "mlp"],
                    help="which side measurements to take: all of them, or the MLP training step alone")
    ap.add_argument("--profile-case", default=None, choices=["gemm", "attention", "deltanet", "groups", "columns", "scan"],
                    help="run one small case of a kernel family only (for ncu captures)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
