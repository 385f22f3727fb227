#!/usr/bin/env python
"""Benchmark of the hyper-connection hot path: HyperConnection layer(s), forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_triton]
                    [--workload c4|c3|c1|c5|readme|per_token] [--scaling strong|weak] [--graph|--no-graph]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = HyperConnection(H) -> branch -> add_residual -> backward with an upstream gradient on
H_new, through the public module API.  The default workload ("c4") is ONE batch of 8 sequences,
bf16 H(8, 4096, 4, 4096), phi [16384, 24] ~ N(0, 0.02^2), 20 Sinkhorn iterations, identity branch.
With N ranks that batch is split into whole sequences, 8/N per GPU (strong scaling; the sharding
needs no communication in the forward pass nor for any activation gradient) and the
replicated-parameter gradients are SUM all-reduced over NCCL.  With fewer than 8 sequences per
GPU the step is replayed from two CUDA graphs (forward, backward) so that the host is not the
limit; collectives stay outside the graphs: the all-reduce of step i runs on a side stream beside
the forward of step i+1 and is waited for before the backward of step i+1 writes the gradient
record again.  The same line carries, under "weak", the measurement with the whole 8-sequence
batch on every GPU (`--scaling weak` makes that the headline instead).

Rank 0 prints one JSON line: tokens/s over all ranks (device-timed, max over ranks; median of five
timed regions of K steps each), the roofline of the dominant kernel (CUDA events around its
launches in every 5th step of the timed regions when the step runs eagerly, else from the breakdown
pass), the
same metric end to end from pinned host buffers with the measured PCIe ceiling beside it, the CPU
implementation timed on the host cores, and a parity check of the batch-sharded and the
sequence-sharded multi-GPU paths against the CPU oracle (untimed, after the timed regions; a failed
check makes the process exit non-zero).

`--impl reference` times the reference's own pure-PyTorch CPU implementation of the same layer on
the host cores when a copy of the reference package has been installed under baseline/_ref
(`kind: "reference"`), else the CPU oracle under oracle/ (`kind: "port"`), on a bounded sample of
whole sequences.  `--impl reference_triton` (a side arm, one GPU) times the reference's Triton
kernels from baseline/_ref on the same workload.

`--workload per_token [--rows R --k K]` is a side measurement: the dynamic-weights op on one row
per token (x [R, K] fp32), forward + backward, with the per-kernel times.
`--workload c5` is the 16-layer D=7168 stack, 2 sequences per GPU, every layer wrapping a bf16 MLP
branch (7168 -> 28672 -> 7168, SiLU); the hyper-connection kernels are timed apart from the MLP.
`--workload c3` is bf16 H(8,4096,4,2048) around a bf16 Linear(2048 -> 2048) branch, reported the same way.
"""

import argparse
import importlib.util
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
    # name: (sequences in the batch, S, D, dtype)
    "c4": (8, 4096, 4096, torch.bfloat16),
    "c3": (8, 4096, 2048, torch.bfloat16),
    "c1": (2, 128, 512, torch.float32),
    "c5": (2, 4096, 7168, torch.bfloat16),   # per GPU: the 16-layer stack is defined as 2 sequences on each of 8 GPUs
    # the reference README's own protocol: fp16 module and tensors, batch 16 x seq 2048, branch = 0.5 * branch_input,
    # loss = H_new.sum() (so the upstream gradient arrives as an expanded scalar)
    "readme": (16, 2048, 4096, torch.float16),
}
LAYERS = {"c5": 16}
PER_GPU_BATCH = {"c5"}          # workloads whose batch is per GPU at every N (weak scaling only)
METRIC = "hc_fwd_bwd_tokens_per_s"
REPEATS = 5                     # timed regions of `steps` steps each; the median is the value
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
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
# summarised under profiles/, per batch element of the c4 shape (traffic is proportional to the
# batch; writes still dirty in L2 at kernel end are not counted); None = not captured.
NCU_TRAFFIC_PER_SEQUENCE = {
    ("c4", "k_stream_mix_bwd_apply"): (335.690752e6 + 212.552704e6) / 2,
    ("c4", "k_add_residual_mix_fwd"): (335.570688e6 + 213.849856e6) / 2,
    ("c4", "k_stream_mix_bwd_reduce"): (604.014592e6 + 3.558144e6) / 2,
    ("c4", "k_add_residual_bwd"): (335.564800e6 + 13.082880e6) / 2,
    ("c4", "k_stream_premix_fwd"): (268.446464e6 + 12.829440e6) / 2,
    ("c4", "k_meanpool_partial"): (268.447488e6 + 4.223744e6) / 2,
}


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi (read-only queries) from
    start() to stop(); started before the warm-up so that even a short timed region has samples."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.t_mark = index, None, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark(self):
        """Samples taken from here on are the ones under load (the timed regions)."""
        self.t_mark = time.perf_counter()

    def stop(self):
        if self.proc is not None:
            time.sleep(0.05)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for t, ln in self.lines:
            if self.t_mark is not None and t < self.t_mark:
                continue
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


def make_layer(D, device, seed=0, layer_idx=0):
    import mhc
    hc = mhc.HyperConnection(dim=D, num_streams=4, dynamic=True, sinkhorn_iters=20, init_scale=0.1, layer_idx=layer_idx)
    gen = torch.Generator().manual_seed(seed)
    phi_t = torch.randn(24, 4 * D, generator=gen) * 0.02
    with torch.no_grad():
        hc.phi.copy_(phi_t.T.contiguous())
    return hc.to(device)


def describe(name, world=1, scaling="strong", identity=False, layers=None):
    B, S, D, dtype = WORKLOADS[name]
    nl = layers or LAYERS.get(name, 1)
    stack = f"stack of {nl} layers, " if nl > 1 else ""
    branch = {"c5": "bf16 MLP branch (D -> 4D -> D, SiLU)", "c3": "bf16 Linear(D -> D) branch"}.get(name, "identity branch")
    if identity:
        branch = "identity branch"
    if name in PER_GPU_BATCH or scaling == "weak":
        batch = f"H({B},{S},4,{D}) on every GPU"
    else:
        batch = f"one batch H({B},{S},4,{D}) split into whole sequences over {world} GPU(s)"
    return (f"{name}: {stack}dynamic HyperConnection fwd+bwd, {str(dtype).split('.')[-1]} {batch}, "
            f"fp32 phi[{4 * D},24], 20 Sinkhorn iters, {branch}")


def config_of(name, world, scaling, per_gpu_batch, tokens, n_layers, identity=False, **more):
    """The `config` object of the JSON line; the reference arms use the same keys."""
    B, S, D, dtype = WORKLOADS[name]
    esz = torch.empty(0, dtype=dtype).element_size()
    cfg = {"workload": describe(name, world, scaling, identity, n_layers), "global_tokens": tokens, "sharding": f"batch x{world}",
           "per_gpu_batch": per_gpu_batch, "layers": n_layers,
           "l2": "inputs larger than L2 (H alone is %.0f MiB per GPU)" % (per_gpu_batch * S * 4 * D * esz / 2 ** 20)}
    cfg.update(more)
    return cfg


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own pure-PyTorch layer when baseline/_ref holds a copy, else the oracle.
# ------------------------------------------------------------------------------------------------
def load_reference_torch_baseline():
    """The reference's src/mhc/_torch_baseline.py from the git-ignored install under baseline/_ref
    (made by `python baseline/install_reference.py` where the reference sources exist), loaded as a
    lone file so that neither Triton nor this repository's own `mhc` package is involved."""
    path = os.path.join(REF_DIR, "mhc", "_torch_baseline.py")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location("mhc_reference_torch_baseline", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cpu_step_factory(D, S, dtype, nseq, threads=None):
    """(step function, kind, cores): forward + backward of the CPU implementation on `nseq` sequences."""
    cores = threads or os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(0)
    H = torch.randn(nseq, S, 4, D, generator=gen)
    g = torch.randn(nseq, S, 4, D, generator=gen)
    if dtype != torch.float32:   # the CPU path computes in fp32 on the up-cast half-precision values
        H, g = H.to(dtype).float(), g.to(dtype).float()
    phi = (torch.randn(24, 4 * D, generator=gen) * 0.02).T.contiguous()
    ref = load_reference_torch_baseline()
    if ref is not None:
        layer = ref.HyperConnectionTorch(dim=D, num_streams=4, layer_idx=0, dynamic=True, sinkhorn_iters=20, init_scale=0.1)
        with torch.no_grad():
            layer.phi.copy_(phi)

        def step():
            Hl = H.clone().requires_grad_(True)
            for q in layer.parameters():
                q.grad = None
            branch_input, add_residual = layer(Hl)
            add_residual(branch_input).backward(g)

        return step, "reference", cores
    from oracle import mhc_oracle as O
    p = O.default_params(D, 0, 0.1)
    p.phi.copy_(phi)

    def step():
        O.layer_fwd_bwd(p, H, g, None, "fused")

    return step, "port", cores


def cpu_sample(D, S, dtype, nseq, steps, warmup):
    step, kind, cores = cpu_step_factory(D, S, dtype, nseq)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        step()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.mean(times)
    return nseq * S / sec, cores, sec, kind


def mem_available_gb():
    try:
        with open("/proc/meminfo") as f:
            for ln in f:
                if ln.startswith("MemAvailable"):
                    return int(ln.split()[1]) / 2 ** 20
    except Exception:
        pass
    return 0.0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B, S, D, dtype = WORKLOADS[args.workload]
    # Whole batch when the host has the memory (the CPU path keeps ~24 fp32 copies of H alive for
    # its backward) and the run stays within a few minutes; else a sample of whole sequences.
    per_seq_gb = 24 * S * 4 * D * 4 / 2 ** 30
    nseq = max(1, min(B, int(0.5 * mem_available_gb() / per_seq_gb)))
    t0 = time.perf_counter()
    cpu_sample(D, S, dtype, 1, 1, 0)
    one = time.perf_counter() - t0
    budget = 150.0 / max(1, args.steps + args.warmup)
    nseq = max(1, min(nseq, int(budget / max(one, 1e-3))))
    tps, cores, sec, kind = cpu_sample(D, S, dtype, nseq, args.steps, args.warmup)
    whole = nseq == B
    sample = (f"{'whole batch' if whole else 'sample'}: {nseq} of {B} sequences per step ({nseq * S} tokens, D={D}), "
              f"fp32 math on {cores} threads, fwd+bwd; sequences are independent, so tokens/s of a sample is tokens/s "
              f"of the batch")
    cfg = config_of(args.workload, 1, "strong", nseq, nseq * S, 1, identity=True, collective="none", cuda_graph=False,
                    timed="whole batch" if whole else f"sample of {nseq} of {B} sequences")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_reference_triton(args):
    """Side arm: the reference's own Triton kernels (unmodified package from baseline/_ref) on one GPU,
    same workload, same step, timed like the main arm."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if not os.path.exists(os.path.join(REF_DIR, "mhc", "__init__.py")):
        print(json.dumps({"impl": "reference_triton", "unavailable": "baseline/_ref holds no copy of the reference package"}))
        return
    sys.path[:] = [p for p in sys.path if os.path.basename(p.rstrip("/")) != "mhc-triton_b200"]
    sys.path.insert(0, REF_DIR)
    import mhc as ref_mhc
    assert os.path.abspath(ref_mhc.__file__).startswith(REF_DIR), ref_mhc.__file__
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, S, D, dtype = WORKLOADS[args.workload]
    if args.batch:
        B = args.batch
    readme = args.workload == "readme"
    gen = torch.Generator(device=dev).manual_seed(1234)
    H = torch.cat([torch.randn(1, S, 4, D, device=dev, generator=gen).to(dtype) for _ in range(B)]).requires_grad_(True)
    g = torch.cat([torch.randn(1, S, 4, D, device=dev, generator=gen).to(dtype) for _ in range(B)])
    # this arm times the hyper-connection layers alone: identity branches (0.5 x in the README protocol), --layers deep
    n_layers = args.layers or 1
    layers = []
    for i in range(n_layers):
        layer = ref_mhc.HyperConnection(dim=D, num_streams=4, dynamic=True, sinkhorn_iters=20, init_scale=0.1, layer_idx=i)
        cpu_gen = torch.Generator().manual_seed(i)
        with torch.no_grad():
            layer.phi.copy_((torch.randn(24, 4 * D, generator=cpu_gen) * 0.02).T.contiguous())
        layer = layer.to(dev)
        layers.append(layer.half() if readme else layer)

    def step():
        H.grad = None
        h = H
        for layer in layers:
            for q in layer.parameters():
                q.grad = None
            bi, add = layer(h)
            h = add(bi * 0.5 if readme else bi)
        if readme:
            h.sum().backward()
        else:
            h.backward(g)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    vals = []
    for _ in range(REPEATS):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        torch.cuda.synchronize()
        vals.append(a.elapsed_time(b) / args.steps)
    ms = statistics.median(vals)
    tokens = B * S
    esz = torch.empty(0, dtype=dtype).element_size()
    print(json.dumps({
        "impl": "reference_triton", "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": (tokens / (ms * 1e-3) / README_PUBLISHED_TOKENS_PER_S) if readme else None,
        "dtype": {torch.bfloat16: "bf16", torch.float16: "f16"}.get(dtype, "f32"), "data": "synthetic",
        "config": config_of(args.workload, 1, "strong", B, tokens, n_layers, identity=True, collective="none", cuda_graph=False),
        "value_spread": {"min_ms": min(vals), "max_ms": max(vals), "regions": REPEATS},
        "hbm_gbs_on_algorithmic_bytes": TOTAL_UNITS * D * esz * tokens * n_layers / (ms * 1e-3) / 1e9,
    }))


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
    floor_ms = 3 * x_bytes / (hbm_peak()[0] * 1e9) * 1e3                            # read x twice, write grad_x once
    print(json.dumps({
        "metric": "dynamic_weights_fwd_bwd_rows_per_s", "value": round(rows / (ms * 1e-3), 1), "unit": "rows/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 2), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"per-token dynamic weights, x [{rows}, {K}] fp32, forward + backward",
                   "l2": "x is larger than L2" if x_bytes > 126e6 else "x fits in L2"},
        "kernels_us": per_kernel,
        "hbm_floor_ms": round(floor_ms, 4), "frac_of_hbm_floor": round(floor_ms / ms, 4),
    }))


# ------------------------------------------------------------------------------------------------
# Multi-GPU parity (untimed): small seeded fp32 cases through the batch-sharded and the
# sequence-sharded paths, each rank against the CPU oracle evaluated on the UNSHARDED batch.
# ------------------------------------------------------------------------------------------------
def parity_leg(dev, rank, world):
    import torch.distributed as dist
    import mhc
    from mhc.parallel import GradSync, SequenceShardedHyperConnection, shard_batch
    from oracle import mhc_oracle as O   # the checker, never the thing measured

    def params(D, seed):
        p = O.default_params(D, 0, 0.1)
        gen = torch.Generator().manual_seed(seed)
        p.phi.copy_(torch.randn(p.phi.shape, generator=gen) * 0.02)
        for t in (p.H_pre_base, p.H_post_base, p.H_res_base):
            t.add_(torch.randn(t.shape, generator=gen) * 0.1)
        return p

    def module(D, p):
        hc = mhc.HyperConnection(dim=D)
        hc.load_state_dict({k: v.clone() for k, v in p.tensors().items()})
        return hc.to(dev)

    def worst(pairs):
        w = 0.0
        for got, ref, atol in pairs:
            ref = ref.double()
            err = float((got.detach().double().cpu() - ref).abs().max())
            w = max(w, err / (atol + 1e-5 * float(ref.abs().max())))
        return w

    out = {}
    # (1) batch sharding + GradSync: whole sequences per rank, gradients all-reduced in the backward
    torch.manual_seed(0)
    B, S, D = 2 * world + 1, 160, 128
    H, g = torch.randn(B, S, 4, D), torch.randn(B, S, 4, D)
    p = params(D, 3)
    full = O.layer_fwd_bwd(p, H, g, None, "fused", dtype=torch.float64)
    hc = module(D, p)
    sync = GradSync([hc])
    Hs = shard_batch(H, rank, world).to(dev).requires_grad_(True)
    lo = sum(shard_batch(H, r, world).shape[0] for r in range(rank))
    n = Hs.shape[0]
    bi, add = hc(Hs)
    H_new = add(bi)
    H_new.backward(shard_batch(g, rank, world).to(dev))
    sync.finish()
    torch.cuda.synchronize()
    pairs = [(bi, full["branch_input"][lo:lo + n], 2e-6), (H_new, full["H_new"][lo:lo + n], 2e-6),
             (Hs.grad, full["dH"][lo:lo + n], 2e-6)]
    pairs += [(q.grad, full["d" + name], 1e-6) for name, q in hc.named_parameters()]
    out["batch_sharded"] = worst(pairs)
    # (2) sequence sharding: every rank holds a slice of every sequence
    torch.manual_seed(1)
    B, S, D = 3, 64 * world, 64
    H, g = torch.randn(B, S, 4, D), torch.randn(B, S, 4, D)
    p = params(D, 4)
    full = O.layer_fwd_bwd(p, H, g, None, "fused", dtype=torch.float64)
    hc = module(D, p)
    sp = SequenceShardedHyperConnection(hc)
    Sl = S // world
    sl = slice(rank * Sl, (rank + 1) * Sl)
    Hs = H[:, sl].contiguous().to(dev).requires_grad_(True)
    bi, add = sp(Hs)
    H_new = add(bi)
    H_new.backward(g[:, sl].contiguous().to(dev))
    torch.cuda.synchronize()
    pairs = [(bi, full["branch_input"][:, sl], 2e-6), (H_new, full["H_new"][:, sl], 2e-6), (Hs.grad, full["dH"][:, sl], 2e-6)]
    pairs += [(q.grad, full["d" + name], 1e-6) for name, q in hc.named_parameters()]
    out["sequence_sharded"] = worst(pairs)
    t = torch.tensor([out["batch_sharded"], out["sequence_sharded"]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {"batch_sharded": float(t[0]), "sequence_sharded": float(t[1])}
    out["ok"] = bool(max(out.values()) <= 1.0)
    out["what"] = ("worst |got - oracle| / (atol + 1e-5 max|oracle|) over outputs, dH and all parameter gradients, max "
                   "over ranks; fp32 inputs, fp64 CPU oracle on the unsharded batch; atol 2e-6 activations, 1e-6 "
                   f"parameter gradients; world size {world}")
    return out


def pcie_ceiling(dev, h2d_bytes, d2h_bytes):
    """Pinned-memory copy ceiling for the bytes one end-to-end step moves: both directions at once on
    two streams (plain tensor.copy_, i.e. one cudaMemcpyAsync each).  Returns (seconds, GB/s in, GB/s out)."""
    n_in, n_out = max(h2d_bytes // 2, 1), max(d2h_bytes // 2, 1)
    src = torch.empty(n_in, dtype=torch.int16).pin_memory()
    dst_d = torch.empty(n_in, dtype=torch.int16, device=dev)
    src_d = torch.empty(n_out, dtype=torch.int16, device=dev)
    dst = torch.empty(n_out, dtype=torch.int16).pin_memory()
    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    best = None
    for _ in range(3):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        s1.wait_event(a); s2.wait_event(a)
        with torch.cuda.stream(s1):
            dst_d.copy_(src, non_blocking=True)
        with torch.cuda.stream(s2):
            dst.copy_(src_d, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s1)
        torch.cuda.current_stream().wait_stream(s2)
        b.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b) * 1e-3
        best = t if best is None else min(best, t)
    return best, h2d_bytes / best / 1e9, d2h_bytes / best / 1e9


class Bench:
    """One workload on this rank: inputs, layers, GradSync, the eager step and the graph-replayed step."""

    def __init__(self, args, name, B, dev, rank, world, use_graph):
        from mhc.parallel import GradSync
        _, S, D, dtype = WORKLOADS[name]
        self.args, self.name, self.B, self.S, self.D, self.dtype = args, name, B, S, D, dtype
        self.dev, self.rank, self.world, self.use_graph = dev, rank, world, use_graph
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        draw = lambda: torch.randn(1, S, 4, D, device=dev, dtype=torch.float32, generator=gen).to(dtype)
        self.H = torch.cat([draw() for _ in range(B)]).requires_grad_(True)
        self.g = torch.cat([draw() for _ in range(B)])
        self.n_layers = args.layers or LAYERS.get(name, 1)
        self.layers = [make_layer(D, dev, seed=i, layer_idx=i) for i in range(self.n_layers)]
        self.readme = name == "readme"
        self.branches = None
        if name == "c5" and not args.identity_branch:
            torch.manual_seed(100 + rank)
            self.branches = [torch.nn.Sequential(torch.nn.Linear(D, 4 * D), torch.nn.SiLU(), torch.nn.Linear(4 * D, D))
                             .to(dev).to(dtype) for _ in range(self.n_layers)]
        elif name == "c3" and not args.identity_branch:
            torch.manual_seed(100 + rank)
            self.branches = [torch.nn.Linear(D, D).to(dev).to(dtype) for _ in range(self.n_layers)]
        if self.readme:
            for layer in self.layers:
                layer.half()
            self.sync = None
        else:
            self.sync = GradSync(self.layers, overlap=not args.no_overlap)
        self.other_params = [q for l in self.layers for q in l.parameters()] if self.readme else []
        if self.branches:
            self.other_params += [q for m in self.branches for q in m.parameters()]
        self.cross = not args.no_cross_layer
        self.graphs = None

    def forward(self):
        h = self.H
        for i, layer in enumerate(self.layers):
            bi, add = layer(h)
            if self.branches:
                bo = self.branches[i](bi)
            else:
                bo = bi * 0.5 if self.readme else bi            # identity branch unless "readme"
            h = add(bo, pool_for_next=(i + 1 < self.n_layers and self.cross))
        return h

    def backward(self, h):
        if self.readme:
            h.sum().backward()
        else:
            h.backward(self.g)

    def eager_step(self):
        self.H.grad = None
        for q in self.other_params:
            q.grad = None
        self.backward(self.forward())
        if self.sync is not None:
            self.sync.finish()

    def capture(self):
        """Forward and backward as two CUDA graphs sharing one memory pool.  Collectives stay outside:
        the in-backward hooks are off during capture and replay."""
        self.sync.set_hooks(False)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self.eager_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.H.grad = None
        gF, gB = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        # thread-local capture mode: NCCL's watchdog thread may query events while this thread captures
        with torch.cuda.graph(gF, capture_error_mode="thread_local"):
            h = self.forward()
        with torch.cuda.graph(gB, pool=gF.pool(), capture_error_mode="thread_local"):
            self.backward(h)
        torch.cuda.synchronize()
        self.graphs = (gF, gB)

    def graph_step(self):
        gF, gB = self.graphs
        gF.replay()
        self.sync.wait_reduced()          # the previous step's all-reduce still owns the gradient record
        gB.replay()
        self.sync.all_reduce_async()      # overlaps the next forward

    def step(self):
        if self.graphs is not None:
            self.graph_step()
        else:
            self.eager_step()

    def drain(self):
        if self.sync is not None:
            self.sync.finish()

    def eager_step_with_hooks(self):
        """Eager step with the collectives started inside the backward (breakdown pass of a graph run)."""
        if self.graphs is None:
            return self.eager_step()
        self.sync.set_hooks(True)
        try:
            self.eager_step()
        finally:
            self.sync.set_hooks(False)


PROFILE_EVERY = 5   # the dominant kernel's launches carry CUDA events in every 5th step of a timed region


def _profile_resume(kernel):
    from mhc import _lib
    _lib.load().mhc_profile_enable(2)   # resume, keeping the records of the earlier sampled steps


def _profile_pause():
    from mhc import _lib
    _lib.load().mhc_profile_enable(0)


def timed_regions(bench, steps, repeats, barrier, world, dev, profiled_kernel=None):
    """`repeats` regions of exactly `steps` steps, each bracketed by a barrier + synchronize and timed
    with CUDA events on the launching stream; returns per-region milliseconds (max over ranks).
    profiled_kernel: its launches are bracketed by the library's own events in every PROFILE_EVERY-th step
    (an event on either side of a kernel keeps it from overlapping its neighbours' tails under programmatic
    dependent launch, about 30 us per step at config 4, so not in every step)."""
    import torch.distributed as dist
    out = []
    for _ in range(repeats):
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            if profiled_kernel is not None:
                if i % PROFILE_EVERY == 0:
                    _profile_resume(profiled_kernel)
                elif i % PROFILE_EVERY == 1:
                    _profile_pause()
            bench.step()
        if profiled_kernel is not None:
            _profile_pause()
        bench.drain()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out.append(float(t.item()))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_triton"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + ["per_token"])
    ap.add_argument("--rows", type=int, default=32768, help="per_token workload: rows of x")
    ap.add_argument("--k", type=int, default=16384, help="per_token workload: columns of x (4 * dim)")
    ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch (profiling small cases)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--cpu-steps", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-weak", action="store_true", help="skip the secondary weak-scaling measurement at N > 1")
    ap.add_argument("--no-overlap", action="store_true", help="all-reduce on the compute stream")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong: the workload's batch is split over the ranks; weak: every rank runs the whole batch")
    ap.add_argument("--layers", type=int, default=None, help="override the number of stacked layers")
    ap.add_argument("--identity-branch", action="store_true", help="c5 / c3: identity branches instead of the MLP / Linear")
    ap.add_argument("--no-cross-layer", action="store_true",
                    help="stacks: let every layer pool its own input instead of taking the sums from the layer before")
    ap.add_argument("--graph", dest="graph", action="store_true", default=None,
                    help="replay the step from CUDA graphs (default: when a GPU holds fewer sequences than the workload's batch)")
    ap.add_argument("--no-graph", dest="graph", action="store_false")
    ap.add_argument("--repeats", type=int, default=REPEATS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "per_token":
        if args.impl != "ours" or args.gpus != 1:
            raise SystemExit("the per_token workload is a single-GPU measurement of this library only")
        args.steps = min(args.steps, 20)
        return run_per_token(args)
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference_triton":
        if args.gpus != 1:
            raise SystemExit("the reference_triton arm is a single-GPU measurement")
        return run_reference_triton(args)

    import torch.distributed as dist
    from mhc import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    clocks = ClockSampler(local).start()

    name = args.workload
    B0, S, D, dtype = WORKLOADS[name]
    readme = name == "readme"
    if readme and world > 1:
        raise SystemExit("the readme workload is a single-GPU protocol")
    scaling = "weak" if name in PER_GPU_BATCH else args.scaling
    B = args.batch or B0
    if scaling == "strong" and not args.batch:
        if B0 % world:
            raise SystemExit(f"batch {B0} does not split over {world} ranks")
        B = B0 // world
    branchy = name == "c5" or (name == "c3" and not args.identity_branch)   # steps with torch branch modules run eagerly
    use_graph = args.graph if args.graph is not None else (B < B0 and not readme and not branchy)
    if readme:
        args.no_e2e = True
        use_graph = False
    esz = torch.empty(0, dtype=dtype).element_size()
    lib = _lib.load()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    bench = Bench(args, name, B, dev, rank, world, use_graph)
    n_layers = bench.n_layers
    for _ in range(args.warmup):
        bench.eager_step()
    if use_graph:
        bench.capture()
        for _ in range(args.warmup):
            bench.step()
        bench.drain()
    barrier()
    # ---- breakdown pass (untimed): every kernel bracketed by events, to find the dominant one ----
    _lib.profile_start()
    for _ in range(3):
        bench.eager_step_with_hooks()
    breakdown = _lib.profile_stop()
    dom = max((n for n in breakdown if n in OP_UNITS), key=lambda n: breakdown[n][1])
    hc_ms_per_step = sum(t for _, t in breakdown.values()) / 3          # all hyper-connection kernels of one step
    barrier()
    # ---- timed regions: K steps each, device-timed; the dominant kernel carries events in every 5th step ----
    _lib.profile_start(only=dom)
    lib.mhc_profile_enable(0)          # switched on for every PROFILE_EVERY-th step inside the regions
    n0 = lib.mhc_launch_count()
    clocks.mark()
    regions = timed_regions(bench, args.steps, max(1, args.repeats), barrier, world, dev,
                            profiled_kernel=None if use_graph else dom)
    launches = (lib.mhc_launch_count() - n0) // max(1, args.repeats)
    if use_graph:   # replayed launches are not seen by the library's counter: count the captured step's kernels
        launches = int(sum(c for c, _ in breakdown.values()) / 3) * args.steps
    timed_prof = _lib.profile_stop()
    clock_summary = clocks.summary()
    ms = statistics.median(regions)
    dom_calls, dom_ms = timed_prof.get(dom) or breakdown[dom]   # a replayed graph carries no events: use the breakdown pass
    ms_per_step = ms / args.steps
    tokens = B * S * world
    value = tokens / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel (largest share of device time) ----
    peak, peak_kind = hbm_peak()
    per_op = {}
    for kname, (calls, total_ms) in breakdown.items():
        units = OP_UNITS.get(kname)
        avg_ms = total_ms / calls
        ent = {"launches_per_step": calls / 3, "avg_ms": avg_ms, "share_of_kernel_time": total_ms / sum(v[1] for v in breakdown.values())}
        if units:
            ent["algorithmic_bytes"] = units * D * esz * B * S
            ent["gbs"] = ent["algorithmic_bytes"] / (avg_ms * 1e-3) / 1e9
            ent["frac"] = ent["gbs"] / peak
        per_op[kname] = ent
    dom_bytes = OP_UNITS[dom] * D * esz * B * S
    dom_avg_ms = dom_ms / dom_calls
    step_bytes = TOTAL_UNITS * D * esz * B * S * n_layers
    traffic = NCU_TRAFFIC_PER_SEQUENCE.get((name, dom))
    step_ms_for_bytes = hc_ms_per_step if bench.branches else ms_per_step
    roofline = {
        "bound": "hbm", "kernel": dom, "achieved": dom_bytes / (dom_avg_ms * 1e-3) / 1e9, "peak": peak,
        "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": dom_bytes / (dom_avg_ms * 1e-3) / 1e9 / peak,
        "traffic": traffic * B if traffic else None, "algorithmic_bytes_per_launch": dom_bytes,
        "avg_launch_ms": dom_avg_ms, "launches_timed": dom_calls,
        "timed_where": "breakdown pass (the timed regions replay CUDA graphs)" if use_graph
                       else f"inside the timed regions, every {PROFILE_EVERY}th step",
        "whole_step": {"algorithmic_bytes": step_bytes, "achieved": step_bytes / (step_ms_for_bytes * 1e-3) / 1e9,
                       "frac": step_bytes / (step_ms_for_bytes * 1e-3) / 1e9 / peak,
                       "note": "per GPU; algorithmic = 46 D*e bytes per token and layer (every op's tensors read once, "
                               "written once); the kernels move 42 (H_residual is never materialised), which is why "
                               "frac can exceed 1",
                       "moved_bytes": step_bytes * MOVED_UNITS // TOTAL_UNITS,
                       "frac_of_moved": step_bytes * MOVED_UNITS / TOTAL_UNITS / (step_ms_for_bytes * 1e-3) / 1e9 / peak},
    }

    # ---- end to end: same step from pinned host buffers, results read back to the host ----
    e2e = None
    weak, streamed, e2e_step = None, None, None
    has_branches = bool(bench.branches)
    if not args.no_e2e and n_layers == 1 and not has_branches:   # the host-streamed step drives one layer, no branch
        Bh = bench.B
        H_host = bench.H.detach().cpu().pin_memory()
        g_host = bench.g.cpu().pin_memory()
        out_new = torch.empty_like(H_host).pin_memory()
        out_dH = torch.empty_like(H_host).pin_memory()
        out_grads = torch.empty(bench.sync.flat.numel(), dtype=torch.float32).pin_memory()
        h2d = H_host.numel() * esz * 2
        d2h = H_host.numel() * esz * 2 + out_grads.numel() * 4

        from mhc.host import HostStreamedStep
        bench.sync.set_hooks(True)
        streamed = HostStreamedStep(bench.layers[0], bench.sync, group=1)

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
        barrier()
        ceil_s, gbs_in, gbs_out = pcie_ceiling(dev, h2d, d2h)   # all ranks at once, like the step itself
        t = torch.tensor([ceil_s], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ceil_s = float(t.item())
        e2e_tokens = Bh * S * world
        e2e = {"value": e2e_tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "global_tokens": e2e_tokens,
               "pcie_gbs": {"h2d_per_gpu": h2d / ceil_s / 1e9, "d2h_per_gpu": d2h / ceil_s / 1e9,
                            "what": "the same bytes as plain pinned copies, both directions at once, all ranks at "
                                    "once, slowest rank"},
               "pcie_floor_ms": ceil_s * 1e3, "frac": ceil_s * 1e3 / e2e_ms,
               "what": "mhc.HostStreamedStep: pinned host H and upstream grad -> device, module fwd+bwd per batch element, "
                       "H_new + dH + parameter grads -> pinned host, copies overlapped with kernels on three streams; "
                       "frac = time of the bare copies / time of the step"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and n_layers == 1:
        tps, cores, sec, kind = cpu_sample(D, S, dtype, 1, args.cpu_steps, 1)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind,
               "sample": f"sample: 1 of {B0} sequences ({S} tokens, D={D}), fp32 math, fwd+bwd, {args.cpu_steps} timed runs "
                         f"of {sec:.2f} s"}

    # ---- secondary measurement at N > 1: the whole batch on every GPU (weak scaling), eager ----
    if scaling == "strong" and world > 1 and not args.no_weak and not args.batch:
        del bench, streamed, e2e_step      # frees the captured graphs' memory pool and the staging buffers
        torch.cuda.empty_cache()
        wb = Bench(args, name, B0, dev, rank, world, False)
        for _ in range(3):
            wb.eager_step()
        wsteps = max(3, min(args.steps, 20))
        wreg = timed_regions(wb, wsteps, 3, barrier, world, dev)
        wms = statistics.median(wreg) / wsteps
        weak = {"value": B0 * S * world / (wms * 1e-3), "unit": "tokens/s", "ms_per_step": wms, "steps": wsteps,
                "global_tokens": B0 * S * world, "per_gpu_batch": B0, "cuda_graph": False,
                "what": "every GPU runs the whole 8-sequence batch, eager, all-reduce started inside the backward "
                        "beside the pass that writes dH"}
    elif world == 1 and scaling == "strong":
        weak = {"value": value, "unit": "tokens/s", "ms_per_step": ms_per_step, "global_tokens": tokens,
                "per_gpu_batch": B, "what": "one GPU: the same measurement"}

    parity = None
    if not args.no_parity and not readme:
        parity = parity_leg(dev, rank, world)
    clocks.stop()

    if rank == 0:
        vals = [tokens / (r / args.steps * 1e-3) for r in regions]
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": (value / README_PUBLISHED_TOKENS_PER_S) if readme else None,
            "dtype": {torch.bfloat16: "bf16", torch.float16: "f16"}.get(dtype, "f32"), "data": "synthetic",
            "config": config_of(name, world, scaling, B, tokens, n_layers,
                                cross_layer_pooling=n_layers > 1 and not args.no_cross_layer, cuda_graph=bool(use_graph),
                                collective=("NCCL SUM all-reduce of phi/bias/alpha grads, " +
                                            ("outside the graphs, beside the next forward" if use_graph else
                                             "started inside the backward beside the pass that writes dH"))
                                if world > 1 else "none",
                                identity=args.identity_branch,
                                **({"batch_overridden": B} if args.batch else {})),
            "value_spread": {"regions": len(regions), "steps_per_region": args.steps, "median": value,
                             "min": min(vals), "max": max(vals)},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches) * world,
            "weak": weak, "parity": parity, "clocks": clock_summary, "kernels_breakdown_pass": per_op,
        }
        if has_branches:
            total_hc = hc_ms_per_step
            line["hc_only"] = {"ms_per_step": total_hc, "value": tokens / (total_hc * 1e-3), "unit": "tokens/s",
                               "mlp_and_rest_ms_per_step": ms_per_step - total_hc,
                               "what": "sum of the hyper-connection kernels' durations per step (CUDA events around "
                                       "every one of them, breakdown pass); `value` of the line is the whole step "
                                       "including the branch modules"}
        print(json.dumps(line))
    ok = parity is None or parity["ok"]
    if world > 1:
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("multi-GPU parity check failed: " + json.dumps(parity))


if __name__ == "__main__":
    main()
