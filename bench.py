"""Benchmark of the fused-network hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|c5]

Default workload (the driver's contract): BASELINE configuration 2, fused inference of the identity-encoded
3 -> 64 relu -> 64 celu -> 64 sine -> 64 relu -> 1 MLP over 2^22 points per GPU. A step is one pass of the fused
inference kernel over one batch. N > 1 (under torchrun, one rank per GPU): every rank runs the same batch size on its
own replica, no data-path communication (inference shards by points), weak scaling.

One JSON line is printed by rank 0. `value` is device-timed throughput with inputs resident in HBM; `e2e` is the same
call with pinned host buffers (host->device copy of the points, device->host copy of the outputs inside the timed
region); `roofline` scores the dominant kernel against the measured tensor peak; `cpu_baseline` times the CPU
restatement of the reference algorithm (oracle/) on the host cores. `--impl reference` times only that CPU restatement,
with all host threads (the reference's own CPU code is Eigen test math that cannot be built here).
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "quick-mlp_b200"), os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

METRIC = "points/sec inference & training step, hashgrid+64-wide MLP, 1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# per-point algorithmic work (unpadded layer sizes, 2*in*out per layer; bytes = fp32 inputs + fp32 outputs
# [+ fp16 grid features actually consumed]) and the measured DRAM traffic per launch of the profiled kernel
WORKLOADS = {
    "c1": dict(points=1 << 16, mode="inference", flops=128, bytes=16, lo=0.0, hi=1.0,
               name="config1: identity 3->16 relu->1 relu, no bias, 65536 points, fused inference"),
    "c2": dict(points=1 << 22, mode="inference", flops=25088, bytes=16, lo=-1.0, hi=1.0,
               name="config2: identity 3->64 relu->64 celu->64 sine->64 relu->1, bias, 2^22 points, fused inference"),
    "c3": dict(points=1 << 20, mode="train", flops=3 * 12416, bytes=3100, lo=0.0, hi=1.0,
               name="config3: 3-D hash grid 16x2 (2^19) + 32->64->64->1, 2^20 points, fused training step"),
    "c4": dict(points=1 << 21, mode="train", flops=3 * 27776, bytes=3600, lo=0.0, hi=1.0,
               name="config4: dense 64^3x4 + hash 8x4 (2^18) + 36->128->64->16->4, 2^21 points per GPU, training step"),
    "c5": dict(points=1 << 22, mode="inference", flops=82944, bytes=2080, lo=0.0, hi=1.0,
               name="config5: 4-D hash grid 16x4 (2^22) + 64->128x3->4, 2^22 points per GPU, fused inference"),
}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised under profiles/
# (c2: 250.0 MB captured on a 2^24-point launch of the tcgen05 kernel, scaled by points to the 2^22-point launch)
MEASURED_TRAFFIC = {"c2": 62.5e6}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def config_of(key):
    import specs
    return {"c1": specs.config1, "c2": specs.config2, "c3": specs.config3, "c4": specs.config4, "c5": specs.config5}[key]()


def xavier_parameters(net, cfg, seed=7):
    """fp16 parameter vector for the benchmark: Xavier-uniform on the unpadded block of every layer, padding and biases
    zero (layout from the library's own layer table)."""
    rng = np.random.default_rng(seed)
    p = np.zeros(net.num_network_parameters(), dtype=np.float32)
    n_in = sum(net.encoding(i).num_output_channels() for i in range(net.num_encodings()))
    for i, layer in enumerate(cfg["network"]):
        cin, cout, _, ws, _ = net.layer_info(i)
        n_out = layer["n_out"]
        bound = float(np.sqrt(6.0 / (n_in + n_out)))
        wmat = np.zeros((cout, cin), dtype=np.float32)
        wmat[:n_out, :n_in] = rng.uniform(-bound, bound, size=(n_out, n_in)).astype(np.float32)
        p[ws:ws + wmat.size] = wmat.ravel()
        n_in = n_out
    return p.astype(np.float16)


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region (read-only query)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------------------------
def host_threads():
    """All host cores this process may use (torchrun exports OMP_NUM_THREADS=1, so OpenMP's default is not it)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_baseline(key, max_seconds=12.0, threads=0):
    """CPU restatement of the reference algorithm (oracle/cpu_ref.cpp, OpenMP) on a bounded sample of the workload."""
    threads = threads or host_threads()
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_ref
    import helpers
    import qmlp_oracle as oracle
    w = WORKLOADS[key]
    cfg = config_of(key)
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg)
    tables = []
    for i, e in enumerate(spec.encodings):
        if e.num_parameters:
            rng = np.random.default_rng(1234 + i)
            tables.append(((rng.random(e.num_parameters, dtype=np.float32) * 2 - 1) * 1e-1).astype(np.float32))
        else:
            tables.append(None)
    net = cpu_ref.CpuNetwork(spec, params, tables)
    probe = 1 << 16
    x = helpers.uniform(42, 1, (probe, spec.num_inputs), w["lo"], w["hi"])
    net.forward(x, threads)                                    # warm-up (thread pool, page faults)
    t0 = time.perf_counter(); net.forward(x, threads); dt = time.perf_counter() - t0
    rate = probe / max(dt, 1e-9)
    sample = int(min(w["points"], max(probe, rate * max_seconds)))
    sample = 1 << int(np.floor(np.log2(sample)))
    x = helpers.uniform(42, 2, (sample, spec.num_inputs), w["lo"], w["hi"])
    passes = int(max(1, min(64, rate * max_seconds / sample)))      # about max_seconds of CPU work in total
    t0 = time.perf_counter()
    for _ in range(passes):
        net.forward(x, threads)
    dt = time.perf_counter() - t0
    kind = "forward pass only" if w["mode"] == "train" else "fused inference"
    return {"value": sample * passes / dt, "unit": "points/s", "cores": threads, "kind": "port",
            "sample": f"{passes} x {sample} points of the workload ({kind}), {dt:.2f} s, C++/OpenMP restatement of the reference math"}


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path (here: the oracle port) on the box's host cores."""
    if rank != 0:
        return
    key = args.workload
    w = WORKLOADS[key]
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_ref
    import helpers
    import qmlp_oracle as oracle
    cfg = config_of(key)
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg)
    tables = []
    for i, e in enumerate(spec.encodings):
        if e.num_parameters:
            rng = np.random.default_rng(1234 + i)
            tables.append(((rng.random(e.num_parameters, dtype=np.float32) * 2 - 1) * 1e-1).astype(np.float32))
        else:
            tables.append(None)
    net = cpu_ref.CpuNetwork(spec, params, tables)
    cores = host_threads()
    probe = 1 << 16
    x = helpers.uniform(42, 1, (probe, spec.num_inputs), w["lo"], w["hi"])
    net.forward(x, cores)
    t0 = time.perf_counter(); net.forward(x, cores); dt = time.perf_counter() - t0
    rate = probe / max(dt, 1e-9)
    # each step: a bounded sample sized so the whole run stays within about two minutes
    budget = 100.0 / max(1, args.steps + args.warmup)
    sample = int(min(w["points"], max(probe, rate * budget)))
    sample = 1 << int(np.floor(np.log2(sample)))
    x = helpers.uniform(42, 2, (sample, spec.num_inputs), w["lo"], w["hi"])
    for _ in range(args.warmup):
        net.forward(x, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        net.forward(x, cores)
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "points/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "points_per_step": sample,
                       "note": "CPU restatement of the reference's Eigen test math (oracle/cpu_ref.cpp, OpenMP); the "
                               "reference's own CPU code needs Eigen and its host library, neither buildable here"},
            "cpu_baseline": {"value": value, "unit": "points/s", "cores": cores, "kind": "port",
                             "sample": f"{sample} points per step x {args.steps} steps"},
            "e2e": {"value": value, "unit": "points/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    gpu_ref = reference_gpu_kernel(key, cfg, spec, params, tables, w)
    if gpu_ref is not None:
        line["reference_gpu_kernel"] = gpu_ref
    print(json.dumps(line), flush=True)


def reference_gpu_kernel(key, cfg, spec, params, tables, w):
    """Extra figure of the reference arm: the reference's own fused inference kernel (its CUDA template filled for this
    configuration and compiled for sm_100a by oracle/build_ref_kernels.py, its own launch configuration) timed on this
    GPU at the workload's full batch. None when it was not built, there is no GPU, or the workload is a training step
    (the reference has no working fused hash-grid training step to time)."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        import ref_kernels
        ref = ref_kernels.ReferenceInference(cfg)
    except Exception:
        return None
    n = w["points"]
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    tp = torch.from_numpy(params.astype(np.float16)).to(dev)
    tt = [torch.from_numpy(t).to(dev) if t is not None else None for t in tables]
    x = torch.rand((n, spec.num_inputs), device=dev) * (w["hi"] - w["lo"]) + w["lo"]
    ref(x, tp, tt, 3)
    _, ms = ref(x, tp, tt, 10)
    grid, block, smem = ref.launch_info
    out = {"value": n / (ms * 1e-3), "unit": "points/s", "ms_per_launch": ms, "points": n,
           "kind": "reference CUDA kernel template (wmma, half accumulation, fp32 tables) compiled for sm_100a; "
                   "inference only" + ("; forward pass of the training workload" if w["mode"] == "train" else ""),
           "launch": {"grid": grid, "block": block, "dynamic_smem": smem}}
    if w["mode"] == "train":
        # The rest of a training step from the reference's kernels: backward (delta chain, table-gradient atomics) and
        # the per-layer single-block weight update, timed on random stash contents of the right shapes (their timing
        # does not depend on the values). No loss, no optimiser, no bias gradients: the reference has none.
        try:
            rb, rw = ref_kernels.ReferenceBackward(cfg), ref_kernels.ReferenceWeightUpdate(cfg)
            n32 = (n + 31) // 32 * 32
            pre = torch.randn((n32 * rb.stash_halfs,), device=dev, dtype=torch.float16)
            adj = torch.randn((n, spec.num_outputs), device=dev)
            grads = [torch.zeros_like(t) if t is not None else None for t in tt]
            rb(x, adj, tp, pre, tt, grads)
            _, deltas = rb(x, adj, tp, pre, tt, grads)
            bwd_ms = rb.last_ms
            rw(x, pre, deltas, tt)
            wu_ms = rw.last_ms
            out["training_step_kernels"] = {
                "forward_ms": ms, "backward_ms": bwd_ms, "weight_update_ms": wu_ms,
                "value": n / ((ms + bwd_ms + wu_ms) * 1e-3), "unit": "points/s",
                "note": "forward (without stash) + backward + single-block weight update per layer; no loss, optimiser or "
                        "bias gradient exists in the reference"}
        except Exception as exc:   # not built for this configuration
            out["training_step_kernels"] = {"unavailable": str(exc)[:200]}
    return out


# ----------------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--points", type=int, default=0, help="override the points per GPU and step")
    ap.add_argument("--fp32-tables", action="store_true", help="gather from fp32 grid tables (reference layout)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from qmlp import bindings, load_library
    from qmlp._capi import check, current_stream, lib, wrap
    from qmlp.trainer import FusedTrainer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the fused kernels")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    load_library()
    bindings.QuickMLP.set_log_level("error")

    key = args.workload
    w = dict(WORKLOADS[key])
    if args.points > 0:
        w["points"] = args.points
    n = w["points"]
    cfg = config_of(key)
    net = bindings.Network(json.dumps(cfg))
    num_inputs, num_outputs = net.channels_in(), net.channels_out()
    params = torch.from_numpy(xavier_parameters(net, cfg)).to(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(42 + rank)
    tables = []
    for i in range(net.num_encodings()):
        e = net.encoding(i)
        if e.has_parameters():
            t = (torch.rand(e.parameter_count(), device=dev, generator=gen) * 2 - 1) * 1e-4
            tables.append(t if args.fp32_tables else t.half())
        else:
            tables.append(None)

    # rotating buffer sets: the working set of consecutive steps exceeds the 126 MB L2
    per_set = n * (num_inputs + num_outputs) * 4
    nsets = max(2, int(np.ceil(300e6 / per_set)))
    nsets = min(nsets, 64)
    xs = [torch.rand((n, num_inputs), device=dev, generator=gen) * (w["hi"] - w["lo"]) + w["lo"] for _ in range(nsets)]
    outs = [torch.empty((n, num_outputs), device=dev) for _ in range(nsets)]
    stream = torch.cuda.current_stream()

    trainer = None
    if w["mode"] == "train":
        trainer = FusedTrainer(net, lr=1e-2, grid_half_copy=not args.fp32_tables, device=dev)
        trainer.set_parameters(params.float(), [t.float() if t is not None else None for t in tables])
        targets = [torch.sin(8 * x[:, :1]) * torch.cos(6 * x[:, 1:2]) * torch.sin(4 * x[:, 2:3]) for x in xs]
        targets = [t.expand(n, num_outputs).contiguous() for t in targets]

        def step(i):
            trainer.step(xs[i % nsets], targets[i % nsets])
    else:
        net._bind(params, tables)

        # tensor views and the stream handle are built once, as a C caller would hold them: at 2^16 points the kernel
        # takes a few microseconds and per-call Python work would be what is timed
        views = [(wrap(x), wrap(o)) for x, o in zip(xs, outs)]
        stream_handle = current_stream()

        def step(i):
            vx, vo = views[i % nsets]
            check(lib().qmlp_network_inference(net._h, vx, vo, stream_handle))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler starts first (it needs a moment to come up), so that the warm-up steps run directly before
    # the timed ones and the GPU does not idle in between
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    for i in range(args.warmup):
        step(i)
    barrier()
    launches0 = net.launch_count()
    # A launch-bound workload (a few microseconds of kernel per step) is captured, K steps in a row, in one CUDA graph
    # and the timed region is one replay of it: otherwise the host's launch rate is what gets measured.
    graph = None
    if trainer is None and n <= (1 << 17):
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            handle = current_stream()
            for i in range(args.steps):
                vx, vo = views[i % nsets]
                check(lib().qmlp_network_inference(net._h, vx, vo, handle))
        graph.replay()
        torch.cuda.synchronize()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    t0 = time.perf_counter()
    if graph is not None:
        events[0][0].record(stream)
        graph.replay()
        events[-1][1].record(stream)
    else:
        for i in range(args.steps):
            events[i][0].record(stream)
            step(i)
            events[i][1].record(stream)
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    launches = net.launch_count() - launches0
    span_ms = events[0][0].elapsed_time(events[-1][1])        # whole timed region on the device
    if graph is not None:
        launches = args.steps                                   # counted at capture; the replay launches the same K kernels
        dev_ms = [span_ms / args.steps] * args.steps
    else:
        dev_ms = [a.elapsed_time(b) for a, b in events]
    t = torch.tensor([span_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    span_ms = float(t.item())
    ms_per_step = span_ms / args.steps
    value = world * n * args.steps / (span_ms * 1e-3)

    # end to end through the public call with host buffers
    hx = torch.empty((n, num_inputs), dtype=torch.float32).pin_memory()
    hx.copy_(xs[0].cpu())
    ho = torch.empty((n, num_outputs), dtype=torch.float32).pin_memory()
    if trainer is not None:
        ht = torch.empty((n, num_outputs), dtype=torch.float32).pin_memory()
        ht.copy_(targets[0].cpu())
        hloss = torch.empty((1,), dtype=torch.float32).pin_memory()

        def e2e_step(i):
            # the public host-memory step: this step's batch was uploaded while the previous step ran (prefetch of the
            # following batch on a copy stream); the loss comes back to the host every step
            trainer.step_host(hx, ht, next_batch=(hx, ht))
            hloss.copy_(trainer.loss_sum, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        h2d, d2h = hx.numel() * 4 + ht.numel() * 4, 4
    else:
        def e2e_step(i):
            # the public host-memory call: chunks of the batch move through upload -> kernel -> download concurrently
            check(lib().qmlp_network_inference_host(net._h, hx.data_ptr(), ho.data_ptr(), n, 0, current_stream()))
            torch.cuda.current_stream().synchronize()
        h2d, d2h = hx.numel() * 4, ho.numel() * 4
    e2e_steps = max(3, min(args.steps, 20))
    for i in range(2):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    barrier()
    e2e_wall = time.perf_counter() - t0
    te = torch.tensor([e2e_wall], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = world * n * e2e_steps / float(te.item())

    if rank == 0:
        peaks, src = load_peaks()
        kernel_ms = float(np.mean(dev_ms))
        if w["mode"] == "inference" and key != "c5":
            peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
            achieved = w["flops"] * n / (kernel_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": MEASURED_TRAFFIC.get(key) if args.points == 0 else None,
                    "peak_source": f"{src} bf16_tflops_sustained", "kernel_ms": kernel_ms,
                    "algorithmic_flops_per_point": w["flops"]}
        else:
            peak = float(peaks["hbm_gbs"])
            achieved = w["bytes"] * n / (kernel_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "peak_source": f"{src} hbm_gbs", "kernel_ms": kernel_ms,
                    "algorithmic_bytes_per_point": w["bytes"]}
        line = {"metric": METRIC, "value": value, "unit": "points/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                "config": {"workload": w["name"], "points_per_gpu_per_step": n, "mode": w["mode"],
                           "l2": f"{nsets} rotating input/output buffer sets ({nsets * per_set / 1e6:.0f} MB) exceed the 126 MB L2",
                           "grid_tables": "fp32" if args.fp32_tables else "fp16", "parallelism": f"replicas x{world}, no data-path collective"
                           if w["mode"] == "inference" else f"dp{world}, one all-reduce of the fused gradient buffer per step"},
                "e2e": {"value": e2e_value, "unit": "points/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "steps": e2e_steps},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
                "wall_s_timed_region": wall}
        if graph is not None:
            line["config"]["launch"] = "the K steps are one CUDA graph (launch-bound workload); the timed region is one replay"
        if w["mode"] == "train":
            line["config"]["parallelism"] = (f"dp{world}: all-reduce of the table gradients under the weight-gradient kernel, "
                                             "then of the network gradients")
        if not args.no_cpu_baseline and world == 1:
            try:
                line["cpu_baseline"] = cpu_baseline(key)
            except Exception as e:   # the baseline is a reported extra; never lose the measured line over it
                line["cpu_baseline"] = {"value": None, "unit": "points/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
