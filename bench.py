#!/usr/bin/env python
"""Benchmark of the hyper-connection hot path: one HyperConnection layer, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4|c3|c1]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = HyperConnection(H) -> identity branch -> add_residual -> backward with an upstream
gradient on H_new, through the public module API.  The default workload is the bf16
H(8, 4096, 4, 4096) configuration (phi [16384, 24] ~ N(0, 0.02^2), 20 Sinkhorn iterations).
With N ranks every rank processes its own batch of that size (whole sequences are the sharding
unit; weak scaling) and the replicated-parameter gradients are SUM all-reduced over NCCL.

Rank 0 prints one JSON line: tokens/s over all ranks (device-timed, max over ranks), the roofline
of the dominant kernel (CUDA events around its launches inside the timed region), the same
metric end to end from pinned host buffers, and the CPU oracle timed on the host cores.

`--impl reference` times the CPU implementation of the same layer (the oracle under oracle/,
a restatement of the reference's pure-PyTorch path) on the host cores, on a bounded sample.

`--workload per_token [--rows R --k K]` is a side measurement, not the headline: the dynamic-weights
op on one row per token (x [R, K] fp32), forward + backward, with the per-kernel times.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "mhc-triton_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

WORKLOADS = {
    # name: (B per rank, S, D, dtype)
    "c4": (8, 4096, 4096, torch.bfloat16),
    "c3": (8, 4096, 2048, torch.bfloat16),
    "c1": (2, 128, 512, torch.float32),
    "c5": (2, 4096, 7168, torch.bfloat16),   # the 16-layer stack, hyper-connection kernels only (identity branches)
    # the reference README's own protocol: fp16 module and tensors, batch 16 x seq 2048, branch = 0.5 * branch_input,
    # loss = H_new.sum() (so the upstream gradient arrives as an expanded scalar)
    "readme": (16, 2048, 4096, torch.float16),
}
LAYERS = {"c5": 16}
METRIC = "hc_fwd_bwd_tokens_per_s"
# Published by the reference for the "readme" workload only: 13.66 ms per fwd+bwd of 32 768 tokens on one H100.
README_PUBLISHED_TOKENS_PER_S = 32768 / 13.66e-3
# Algorithmic HBM bytes per token, in units of D * element size: each logical tensor is read once
# per consuming op and written once (mean-pool 4, stream mix 9, add residual 9, add-residual
# backward 6, stream-mix backward: reduction pass 9 + apply pass 9).
OP_UNITS = {
    "k_meanpool_partial": 4, "k_stream_mix_fwd": 9, "k_stream_premix_fwd": 5, "k_add_residual_mix_fwd": 9,
    "k_add_residual_mix_pool_fwd": 9, "k_add_residual_fwd": 9, "k_add_residual_pool_fwd": 9,
    "k_add_residual_bwd": 6,
    "k_stream_mix_bwd_reduce": 9, "k_stream_mix_bwd_apply": 9,
}
TOTAL_UNITS = 46
# What the fused module path actually moves per token: the residual mix is recomputed inside the
# add-residual kernel instead of being written (4) and read back (4), and the pre-mix kernel then
# moves 5 instead of 9:  4 + 5 + 9 + 6 + 9 + 9.
MOVED_UNITS = 42
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/, keyed by (workload, kernel); None = not captured.
NCU_TRAFFIC = {
    # batch-2 capture x4 (traffic is proportional to the batch); writes still dirty in L2 at kernel end are not counted
    ("c4", "k_stream_mix_bwd_apply"): 4 * (335.689216e6 + 212.662016e6),
    ("c4", "k_add_residual_mix_fwd"): 4 * (335.556096e6 + 212.420864e6),
    ("c4", "k_stream_mix_bwd_reduce"): 4 * (604.002304e6 + 3.213056e6),
    ("c4", "k_add_residual_bwd"): 4 * (335.597568e6 + 13.030144e6),
    ("c4", "k_stream_premix_fwd"): 4 * (268.445952e6 + 13.323520e6),
    ("c4", "k_meanpool_partial"): 4 * (268.504064e6 + 4.123392e6),
}


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.12)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_layer(D, device):
    import mhc
    hc = mhc.HyperConnection(dim=D, num_streams=4, dynamic=True, sinkhorn_iters=20, init_scale=0.1, layer_idx=0)
    gen = torch.Generator().manual_seed(0)
    phi_t = torch.randn(24, 4 * D, generator=gen) * 0.02
    with torch.no_grad():
        hc.phi.copy_(phi_t.T.contiguous())
    return hc.to(device)


def cpu_oracle_sample(D, S, dtype, steps, warmup, threads=None):
    """Oracle forward+backward on the host cores for ONE batch element of S tokens (batch elements
    are independent, so tokens/s of the sample is tokens/s of the workload).  Returns (tokens/s, cores)."""
    from oracle import mhc_oracle as O
    cores = threads or os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(0)
    H = torch.randn(1, S, 4, D, generator=gen)
    g = torch.randn(1, S, 4, D, generator=gen)
    if dtype != torch.float32:   # the CPU path computes in fp32 on the up-cast half-precision values
        H, g = H.to(dtype).float(), g.to(dtype).float()
    p = O.default_params(D, 0, 0.1)
    p.phi.copy_((torch.randn(24, 4 * D, generator=gen) * 0.02).T)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.layer_fwd_bwd(p, H, g, None, "fused")
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return S / statistics.mean(times), cores, statistics.mean(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B, S, D, dtype = WORKLOADS[args.workload]
    tps, cores, sec = cpu_oracle_sample(D, S, dtype, args.steps, args.warmup)
    sample = f"1 of {B} batch elements per step: {S} tokens, D={D}, fp32 math, fwd+bwd"
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": describe(args.workload), "timed": sample},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def describe(name):
    B, S, D, dtype = WORKLOADS[name]
    nl = LAYERS.get(name, 1)
    stack = f"stack of {nl} layers, " if nl > 1 else ""
    return (f"{name}: {stack}dynamic HyperConnection fwd+bwd, {str(dtype).split('.')[-1]} H({B},{S},4,{D}) per GPU, "
            f"fp32 phi[{4 * D},24], 20 Sinkhorn iters, identity branch")


def run_per_token(args):
    """Side workload, not the headline: the dynamic-weights op applied to every token's own state
    (x [rows, K] fp32 with K = 4 D), forward + backward, one GPU.  Prints one JSON line with the time per
    forward+backward and the per-kernel breakdown from the library's own CUDA events."""
    from mhc import _lib
    from mhc._backward import fused_dynamic_weights_backward
    from mhc._kernels import fused_dynamic_weights_forward
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rows, K = args.rows, args.k
    gen = torch.Generator(device=dev).manual_seed(1234)
    x = torch.randn(rows, K, device=dev, generator=gen)
    phi = torch.randn(K, 24, device=dev, generator=gen) * 0.02
    bias = torch.randn(24, device=dev, generator=gen)
    al = [torch.full((1,), v, device=dev) for v in (0.3, -0.2, 0.5)]
    gr = [torch.randn(rows, 4, device=dev, generator=gen), torch.randn(rows, 4, device=dev, generator=gen),
          torch.randn(rows, 4, 4, device=dev, generator=gen)]

    def step():
        saved = fused_dynamic_weights_forward(x, phi, bias, *al, 20, 1e-6, return_saved=True)[3]
        return fused_dynamic_weights_backward(x, phi, bias, *al, saved, *gr, 20, 1e-6)

    for _ in range(max(args.warmup, 2)):
        step()
    torch.cuda.synchronize()
    _lib.profile_start()
    for _ in range(args.steps):
        step()
    prof = _lib.profile_stop()
    per_kernel = {k: round(t / n * 1e3, 1) for k, (n, t) in prof.items()}          # microseconds per launch
    ms = sum(t / n for n, t in prof.values())
    x_bytes = rows * K * 4
    print(json.dumps({
        "metric": "dynamic_weights_fwd_bwd_rows_per_s", "value": round(rows / (ms * 1e-3), 1), "unit": "rows/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 2), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"per-token dynamic weights, x [{rows}, {K}] fp32, forward + backward",
                   "l2": "x is larger than L2" if x_bytes > 126e6 else "x fits in L2"},
        "kernels_us": per_kernel,
        "hbm_floor_ms": round(3 * x_bytes / (hbm_peak()[0] * 1e9) * 1e3, 4),   # read x twice, write grad_x once
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + ["per_token"])
    ap.add_argument("--rows", type=int, default=32768, help="per_token workload: rows of x")
    ap.add_argument("--k", type=int, default=16384, help="per_token workload: columns of x (4 * dim)")
    ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch (profiling small cases)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--cpu-steps", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="all-reduce on the compute stream")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank runs the workload's batch; strong: the workload's batch is split over the ranks")
    ap.add_argument("--layers", type=int, default=None, help="override the number of stacked layers")
    ap.add_argument("--no-cross-layer", action="store_true",
                    help="stacks: let every layer pool its own input instead of taking the sums from the layer before")
    ap.add_argument("--graph", action="store_true",
                    help="replay the step from a CUDA graph (for small per-GPU batches, where the host would be the limit)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "per_token":
        if args.impl != "ours" or args.gpus != 1:
            raise SystemExit("the per_token workload is a single-GPU measurement of this library only")
        args.steps = min(args.steps, 20)
        return run_per_token(args)
    if args.impl == "reference":
        return run_reference(args)

    import torch.distributed as dist
    from mhc import _lib
    from mhc.parallel import GradSync

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, S, D, dtype = WORKLOADS[args.workload]
    if args.batch:
        B = args.batch
    if args.scaling == "strong":
        if B % world:
            raise SystemExit(f"batch {B} does not split over {world} ranks")
        B //= world
    esz = torch.empty(0, dtype=dtype).element_size()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    H = torch.randn(B, S, 4, D, device=dev, dtype=torch.float32, generator=gen).to(dtype) if B * S * D <= 2 ** 24 else \
        torch.cat([torch.randn(1, S, 4, D, device=dev, dtype=torch.float32, generator=gen).to(dtype) for _ in range(B)])
    g = torch.cat([torch.randn(1, S, 4, D, device=dev, dtype=torch.float32, generator=gen).to(dtype) for _ in range(B)])
    H.requires_grad_(True)
    n_layers = args.layers or LAYERS.get(args.workload, 1)
    layers = [make_layer(D, dev) for _ in range(n_layers)]
    hc = layers[0]
    lib = _lib.load()

    readme = args.workload == "readme"
    if readme:
        for layer in layers:
            layer.half()
        args.no_e2e = True

    class _NoSync:      # half-precision parameters: gradients flow through autograd, nothing to all-reduce at N=1
        flat = torch.zeros(1)

        def finish(self):
            pass

        def all_reduce_now(self):
            pass

    if readme and world > 1:
        raise SystemExit("the readme workload is a single-GPU protocol")
    sync = _NoSync() if readme else GradSync(layers, overlap=not args.no_overlap)

    params = [q for layer in layers for q in layer.parameters()]

    def step():
        H.grad = None
        if readme:
            for q in params:
                q.grad = None
        h = H
        for i, layer in enumerate(layers):
            bi, add = layer(h)
            bo = bi * 0.5 if readme else bi                                    # identity branch unless "readme"
            h = add(bo, pool_for_next=(i + 1 < n_layers and not args.no_cross_layer))
        if readme:
            h.sum().backward()
        else:
            h.backward(g)
        sync.finish()
        return h

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    eager_step = step
    if args.graph:
        # Warm up on a side stream, then capture one step and replay it.  Collectives stay OUT of the
        # graph: the captured step leaves this rank's gradients in the flat record and the all-reduce
        # is issued eagerly after every replay.
        hooks = [l.grads_ready_hook for l in layers]
        for l in layers:
            l.grads_ready_hook = None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                eager_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: NCCL's watchdog thread may query events while this thread captures
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            eager_step()
        torch.cuda.synchronize()

        def step():  # noqa: F811
            graph.replay()
            sync.all_reduce_now()

        def eager_step_with_hooks():
            for l, h in zip(layers, hooks):
                l.grads_ready_hook = h
            try:
                return eager_step()
            finally:
                for l in layers:
                    l.grads_ready_hook = None

    for _ in range(args.warmup):
        step()
    barrier()
    # ---- breakdown pass (untimed): every kernel bracketed by events, to find the dominant one ----
    _lib.profile_start()
    for _ in range(3):
        (eager_step_with_hooks if args.graph else eager_step)()
    breakdown = _lib.profile_stop()
    dom = max((n for n in breakdown if n in OP_UNITS), key=lambda n: breakdown[n][1])
    barrier()
    # ---- timed region: K steps, device-timed; only the dominant kernel's launches carry events ----
    _lib.profile_start(only=dom)
    n0 = lib.mhc_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    launches = lib.mhc_launch_count() - n0
    timed_prof = _lib.profile_stop()
    dom_calls, dom_ms = timed_prof.get(dom) or breakdown[dom]   # a replayed graph carries no events: use the breakdown pass
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    tokens = B * S * world
    value = tokens / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel (largest share of device time), timed inside the timed region ----
    peak, peak_kind = hbm_peak()
    per_op = {}
    for name, (calls, total_ms) in breakdown.items():
        units = OP_UNITS.get(name)
        avg_ms = total_ms / calls
        ent = {"launches_per_step": calls / 3, "avg_ms": avg_ms, "share_of_kernel_time": total_ms / sum(v[1] for v in breakdown.values())}
        if units:
            ent["algorithmic_bytes"] = units * D * esz * B * S
            ent["gbs"] = ent["algorithmic_bytes"] / (avg_ms * 1e-3) / 1e9
            ent["frac"] = ent["gbs"] / peak
        per_op[name] = ent
    dom_bytes = OP_UNITS[dom] * D * esz * B * S
    dom_avg_ms = dom_ms / dom_calls
    step_bytes = TOTAL_UNITS * D * esz * B * S * n_layers
    roofline = {
        "bound": "hbm", "kernel": dom, "achieved": dom_bytes / (dom_avg_ms * 1e-3) / 1e9, "peak": peak,
        "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": dom_bytes / (dom_avg_ms * 1e-3) / 1e9 / peak,
        "traffic": NCU_TRAFFIC.get((args.workload, dom)), "algorithmic_bytes_per_launch": dom_bytes,
        "avg_launch_ms": dom_avg_ms, "launches_timed": dom_calls,
        "whole_step": {"algorithmic_bytes": step_bytes, "achieved": step_bytes / (ms_per_step * 1e-3) / 1e9,
                       "frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
                       "note": "algorithmic = 46 D*e bytes per token and layer (every op's tensors read once, written once); "
                               "the kernels move 42 (H_residual is never materialised), which is why frac can exceed 1",
                       "moved_bytes": step_bytes * MOVED_UNITS // TOTAL_UNITS,
                       "frac_of_moved": step_bytes * MOVED_UNITS / TOTAL_UNITS / (ms_per_step * 1e-3) / 1e9 / peak},
    }

    # ---- end to end: same step from pinned host buffers, results read back to the host ----
    e2e = None
    if not args.no_e2e and n_layers == 1:   # the host-streamed step drives one layer
        H_host = H.detach().cpu().pin_memory()
        g_host = g.cpu().pin_memory()
        out_new = torch.empty_like(H_host).pin_memory()
        out_dH = torch.empty_like(H_host).pin_memory()
        out_grads = torch.empty(sync.flat.numel(), dtype=torch.float32).pin_memory()
        h2d = H_host.numel() * esz * 2
        d2h = H_host.numel() * esz * 2 + out_grads.numel() * 4

        from mhc.host import HostStreamedStep
        streamed = HostStreamedStep(hc, sync, group=1)

        def e2e_step():
            streamed(H_host, g_host, out_new, out_dH, out_grads)

        e2e_step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / args.e2e_steps
        e2e = {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
               "what": "mhc.HostStreamedStep: pinned host H and upstream grad -> device, module fwd+bwd per batch element, "
                       "H_new + dH + parameter grads -> pinned host, copies overlapped with kernels on three streams"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and n_layers == 1:
        tps, cores, sec = cpu_oracle_sample(D, S, dtype, args.cpu_steps, 1)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"1 of {B} batch elements ({S} tokens, D={D}), fp32 math, fwd+bwd, {args.cpu_steps} timed runs "
                         f"of {sec:.2f} s"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": (value / README_PUBLISHED_TOKENS_PER_S) if readme else None,
            "dtype": {torch.bfloat16: "bf16", torch.float16: "f16"}.get(dtype, "f32"), "data": "synthetic",
            "config": {"workload": describe(args.workload) + (f" [batch overridden to {B}]" if args.batch else ""),
                       "global_tokens": tokens, "sharding": f"batch x{world}", "per_gpu_batch": B, "layers": n_layers,
                       "cross_layer_pooling": n_layers > 1 and not args.no_cross_layer, "cuda_graph": bool(args.graph),
                       "l2": "inputs larger than L2 (H alone is %.0f MiB per GPU)" % (B * S * 4 * D * esz / 2 ** 20),
                       "collective": "NCCL SUM all-reduce of phi/bias/alpha grads" if world > 1 else "none"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches) * world,
            "clocks": clocks.summary(), "kernels_breakdown_pass": per_op,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
