"""Benchmark of the fused-network hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3|c3i|c2|c1|c4|c5]

Default workload: the fused training step of the hash-grid network the metric is named after (3-D hash grid, 16 levels x
2 features, 2^19 rows per level, + 32 -> 64 -> 64 -> 1 with bias): forward with stash, L2-loss gradient, backward,
table-gradient scatter, weight / bias gradients and Adam over 2^20 points per GPU. With N > 1 (under torchrun, one rank
per GPU) the step is data parallel: every rank draws its own points and the fused gradient vector is all-reduced over
NCCL inside the timed step. The same line carries two secondary blocks, each with its own timing, roofline and
end-to-end figure: fused inference of the same network, and fused inference of the identity-encoded 64-wide MLP
(`--no-secondary` leaves them out).

One JSON line is printed by rank 0. `value` is device-timed throughput with inputs resident in HBM; `e2e` is the public
call with page-locked host buffers (host->device copy of the points and targets, device->host read of the loss or the
outputs, inside the timed region); `roofline` scores the step's algorithmic bytes against the measured copy bandwidth
and names the dominant kernel from a live per-kernel timing pass; `cpu_baseline` times the C++ restatement of the
reference algorithm (oracle/) on the host cores on the same kind of step. `--impl reference` times only that CPU
restatement, with all host threads (the reference's own CPU code is Eigen test math that cannot be built here).
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.join(ROOT, "quick-mlp_b200")
if _PKG not in sys.path:
    sys.path.insert(0, _PKG)

import numpy as np  # noqa: E402

METRIC = "points/sec inference & training step, hashgrid+64-wide MLP, 1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
SECONDARY = {"c3": ("c3i", "c2"), "c4": ("c2",)}



def measured_traffic_per_point():
    """{workload: {kernel: DRAM bytes per point}} from the table in profiles/dram_traffic.md (dram__bytes_read.sum +
    dram__bytes_write.sum of ncu captures, divided by the points of the captured case)."""
    table = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if not os.path.exists(path):
        return table
    with open(path) as f:
        for line in f:
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) != 5 or cells[0] in ("workload", "") or set(cells[0]) <= set("-"):
                continue
            try:
                table.setdefault(cells[0], {})[cells[1]] = float(cells[4])
            except ValueError:
                continue
    return table


KERNEL_NAMES = {0: "inference", 1: "forward_stash", 2: "forward_loss", 3: "backward", 4: "wgrad", 9: "encode_planes",
                10: "inference_planes", 11: "scatter_planes", 12: "forward_loss_planes", 13: "sort_points",
                15: "scatter_sorted", 100: "adam", 101: "refresh_half"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def xavier_blocks(layers, cfg, n_in, count, seed=7):
    """fp32 parameter vector of `count` entries: Xavier-uniform on the unpadded block of every layer, padding and biases
    zero. `layers` = [(cin_padded, cout_padded, weights_start)] from the library's (or the oracle's) own layer table."""
    rng = np.random.default_rng(seed)
    p = np.zeros(count, dtype=np.float32)
    for (cin, cout, ws), layer in zip(layers, cfg["network"]):
        n_out = layer["n_out"]
        bound = float(np.sqrt(6.0 / (n_in + n_out)))
        wmat = np.zeros((cout, cin), dtype=np.float32)
        wmat[:n_out, :n_in] = rng.uniform(-bound, bound, size=(n_out, n_in)).astype(np.float32)
        p[ws:ws + wmat.size] = wmat.ravel()
        n_in = n_out
    return p


def table_values(count, index, scale=1e-4, seed=1234):
    rng = np.random.default_rng(seed + index)
    return ((rng.random(count, dtype=np.float32) * 2 - 1) * scale).astype(np.float32)


def targets_of(x, num_outputs, xp):
    """Smooth analytic targets of the first three input coordinates (xp = numpy or torch): output 0 is
    sin(8x) cos(6y) sin(4z); further outputs use other small integer frequencies."""
    a, b, c = x[:, 0:1], x[:, 1:2], x[:, 2:3]
    cols = [xp.sin(8 * a) * xp.cos(6 * b) * xp.sin(4 * c), xp.cos(5 * a) * xp.sin(3 * b) * xp.cos(7 * c),
            xp.sin(2 * a + 3 * b) * xp.cos(4 * c), xp.cos(6 * a) * xp.cos(2 * b) * xp.sin(5 * c)]
    while len(cols) < num_outputs:
        cols.append(cols[len(cols) % 4])
    return xp.concatenate(cols[:num_outputs], 1) if xp is np else xp.cat(cols[:num_outputs], 1)


def config_block(key, w, n, world, fp32_tables):
    """The `config` object of the JSON line; both arms print the same keys and values for the same workload."""
    per_gpu = n
    cfg = {"workload": w["name"], "points_per_gpu_per_step": per_gpu, "mode": w["mode"],
           "grid_tables": "fp32" if fp32_tables else "fp16",
           "l2": "rotating input/output buffer sets and the step's scratch exceed the 126 MB L2"}
    if w["mode"] == "train":
        nvls = os.environ.get("NCCL_NVLS_ENABLE", "0" if world >= 8 else "default")
        cfg["parallelism"] = (f"dp{world}, all-reduce (NCCL, NCCL_NVLS_ENABLE={nvls}) of the fused gradient vector inside "
                              "the timed step") if world > 1 else "dp1"
    else:
        cfg["parallelism"] = f"replicas x{world}, points sharded, no data-path collective"
    return cfg


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the GPU is under load (read-only query)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
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
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}


def host_threads(affinity=None):
    """All host cores this process may use (torchrun exports OMP_NUM_THREADS=1, so OpenMP's default is not it)."""
    if affinity is not None:
        return max(1, len(affinity))
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def bind_to_gpu_numa_node(torch, device_index):
    """Runs this process (and so the first touch of its page-locked buffers) on the cores of the NUMA node the GPU hangs
    off. Returns a short description, or None when the topology cannot be read."""
    try:
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return f"numa node {node}, {len(allowed)} cores"
    except Exception:
        return None


# ----------------------------------------------------------------------------------------------------------------------
# CPU legs (oracle/): the only part of this file that touches the restatement of the reference algorithm
# ----------------------------------------------------------------------------------------------------------------------
def _cpu_network(key):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_ref
    import qmlp_oracle as oracle
    from qmlp import configs
    cfg = configs.workload_config(key)
    spec = oracle.parse_spec(cfg)
    layers = [(l.channels_in, l.channels_out, l.weights_start) for l in spec.layers]
    params = xavier_blocks(layers, cfg, spec.encoded_channels, spec.num_parameters).astype(np.float16).astype(np.float32)
    tables = [table_values(e.num_parameters, i) if e.num_parameters else None for i, e in enumerate(spec.encodings)]
    return cpu_ref.CpuNetwork(spec, params, tables), spec


def _cpu_pass(net, spec, w, x, threads):
    """One step of the workload on the host: a fused inference pass, or a whole training step (forward, loss, backward,
    weight / bias / table gradients, Adam over every parameter)."""
    if w["mode"] == "train":
        net.train_step(x, targets_of(x, spec.num_outputs, np), threads=threads)
    else:
        net.forward(x, threads)


def _cpu_sample_size(net, spec, w, threads, seconds_per_step):
    rng = np.random.default_rng(42)
    probe = 1 << 15
    x = (rng.random((probe, spec.num_inputs), dtype=np.float32) * (w["hi"] - w["lo"]) + w["lo"]).astype(np.float32)
    _cpu_pass(net, spec, w, x, threads)                               # warm-up (thread pool, page faults)
    t0 = time.perf_counter(); _cpu_pass(net, spec, w, x, threads); dt = time.perf_counter() - t0
    rate = probe / max(dt, 1e-9)
    sample = int(min(w["points"], max(probe, rate * seconds_per_step)))
    sample = 1 << int(np.floor(np.log2(sample)))
    x = (rng.random((sample, spec.num_inputs), dtype=np.float32) * (w["hi"] - w["lo"]) + w["lo"]).astype(np.float32)
    return sample, x


def cpu_baseline(key, w, threads, max_seconds=14.0):
    """CPU restatement of the reference algorithm (oracle/cpu_ref.cpp, OpenMP) on a bounded sample of the workload."""
    net, spec = _cpu_network(key)
    sample, x = _cpu_sample_size(net, spec, w, threads, max_seconds / 4)
    passes = 0
    t0 = time.perf_counter()
    while passes < 64 and (passes < 2 or time.perf_counter() - t0 < max_seconds):
        _cpu_pass(net, spec, w, x, threads)
        passes += 1
    dt = time.perf_counter() - t0
    what = ("training step: forward, L2 loss, backward, weight/bias/table gradients, Adam over all parameters"
            if w["mode"] == "train" else "fused inference")
    return {"value": sample * passes / dt, "unit": "points/s", "cores": threads, "kind": "port",
            "sample": f"{passes} steps x {sample} points of the workload ({what}), {dt:.2f} s, "
                      "C++/OpenMP restatement of the reference math, fp32"}


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path (here: the C++ restatement) on the box's host cores."""
    if rank != 0:
        return
    from qmlp import configs
    key = args.workload
    w = dict(configs.WORKLOADS[key])
    n = args.points if args.points > 0 else (w["points"] // world if w.get("sharded") else w["points"])
    cores = host_threads()
    net, spec = _cpu_network(key)
    # each step: a bounded sample sized so the whole run stays within about two minutes
    budget = 100.0 / max(1, args.steps + args.warmup)
    sample, x = _cpu_sample_size(net, spec, w, cores, budget)
    for _ in range(args.warmup):
        _cpu_pass(net, spec, w, x, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _cpu_pass(net, spec, w, x, cores)
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    what = "whole training step incl. Adam" if w["mode"] == "train" else "fused inference"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "points/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong" if w.get("sharded") else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": config_block(key, w, n, world, args.fp32_tables),
            "cpu_baseline": {"value": value, "unit": "points/s", "cores": cores, "kind": "port",
                             "sample": f"{sample} points per step x {args.steps} steps ({what}); C++/OpenMP restatement of "
                                       "the reference's Eigen test math and grid encoder (oracle/cpu_ref.cpp): the "
                                       "reference's own CPU code needs Eigen and its host library, neither buildable here"},
            "e2e": {"value": value, "unit": "points/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    gpu_ref = reference_gpu_kernel(key, w, spec, net)
    if gpu_ref is not None:
        line["reference_gpu_kernel"] = gpu_ref
    print(json.dumps(line), flush=True)


def reference_gpu_kernel(key, w, spec, cpu_net):
    """Extra figure of the reference arm: the reference's own fused kernels (its CUDA templates filled for this
    configuration and compiled for sm_100a by oracle/build_ref_kernels.py, its own launch configuration) timed on this
    GPU at the workload's full batch. None when they were not built or there is no GPU."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        import ref_kernels
        from qmlp import configs
        cfg = configs.workload_config(key)
        ref = ref_kernels.ReferenceInference(cfg)
    except Exception:
        return None
    n = w["points"]
    if n > (1 << 22):
        n = 1 << 22
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    tp = torch.from_numpy(cpu_net.params.astype(np.float16)).to(dev)
    tt = [torch.from_numpy(t).to(dev) if t is not None else None for t in cpu_net.tables]
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
class Bench:
    """Shared state of one benchmark process (one rank)."""

    def __init__(self, args, rank, local_rank, world):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.args, self.rank, self.local_rank, self.world = args, rank, local_rank, world
        self.dev = torch.device("cuda", local_rank)
        self.peaks, self.peak_source = load_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def all_ranks_agree(self, flag):
        """True only if `flag` holds on every rank (a collective at N > 1: all ranks call it the same number of times)."""
        if self.world == 1:
            return bool(flag)
        t = self.torch.tensor([1 if flag else 0], device=self.dev, dtype=self.torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def max_over_ranks(self, v):
        t = self.torch.tensor([v], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    # ------------------------------------------------------------------------------------------------------------------
    def run(self, key, steps, warmup, primary):
        torch = self.torch
        from qmlp import bindings, configs
        from qmlp._capi import check, current_stream, lib, wrap
        from qmlp.trainer import FusedTrainer
        args, dev, world, rank = self.args, self.dev, self.world, self.rank
        w = dict(configs.WORKLOADS[key])
        n = w["points"] // world if w.get("sharded") else w["points"]
        if primary and args.points > 0:
            n = args.points
        cfg = configs.workload_config(key)
        net = bindings.Network(json.dumps(cfg))
        num_inputs, num_outputs = net.channels_in(), net.channels_out()
        layers = [net.layer_info(i) for i in range(net.num_layers())]
        n_enc = sum(net.encoding(i).num_output_channels() for i in range(net.num_encodings()))
        p32 = xavier_blocks([(cin, cout, ws) for cin, cout, _, ws, _ in layers], cfg, n_enc, net.num_network_parameters())
        params = torch.from_numpy(p32.astype(np.float16)).to(dev)
        # parameters and tables are the same on every rank (a data-parallel replica set); only the points differ
        tables = []
        for i in range(net.num_encodings()):
            e = net.encoding(i)
            if e.has_parameters():
                t = torch.from_numpy(table_values(e.parameter_count(), i)).to(dev)
                tables.append(t if args.fp32_tables else t.half())
            else:
                tables.append(None)
        gen = torch.Generator(device=dev)
        gen.manual_seed(42 + rank)

        # rotating buffer sets: the working set of consecutive steps exceeds the 126 MB L2
        per_set = n * (num_inputs + num_outputs) * 4
        nsets = min(64, max(2, int(np.ceil(300e6 / per_set))))
        xs = [torch.rand((n, num_inputs), device=dev, generator=gen) * (w["hi"] - w["lo"]) + w["lo"] for _ in range(nsets)]
        outs = [torch.empty((n, num_outputs), device=dev) for _ in range(nsets)]
        stream = torch.cuda.current_stream()

        trainer = None
        if w["mode"] == "train":
            trainer = FusedTrainer(net, lr=1e-2, grid_half_copy=not args.fp32_tables, device=dev)
            if args.dp_levels_per_launch >= 0:
                trainer.level_group_size = args.dp_levels_per_launch
            trainer.set_parameters(params.float(), [t.float() if t is not None else None for t in tables])
            targets = [targets_of(x, num_outputs, torch).contiguous() for x in xs]

            def step(i):
                trainer.step(xs[i % nsets], targets[i % nsets])
        else:
            net._bind(params, tables)
            # tensor views and the stream handle are built once, as a C caller would hold them: at 2^16 points the
            # kernel takes a few microseconds and per-call Python work would be what is timed
            views = [(wrap(x), wrap(o)) for x, o in zip(xs, outs)]
            stream_handle = current_stream()

            def step(i):
                vx, vo = views[i % nsets]
                check(lib().qmlp_network_inference(net._h, vx, vo, stream_handle))

        # The clock sampler starts first and the GPU is kept under the same load until it has had time to deliver
        # samples; the W warm-up steps then run directly before the timed ones.
        sampler = ClockSampler(self.local_rank) if (primary and rank == 0) else None
        if sampler:
            sampler.start()
        step(0)
        torch.cuda.synchronize()
        if primary:
            # Blocks of eight steps until 0.4 s have passed. Every rank must take the same number of steps (a step of the
            # data-parallel workload contains collectives, and a rank that took one step more would leave its last
            # all-reduces without partners): the decision to go on is taken after each block and agreed over the ranks.
            t_settle = time.perf_counter()
            i = 0
            go_on = True
            while go_on:
                for _ in range(8):
                    step(i); i += 1
                torch.cuda.synchronize()
                go_on = self.all_ranks_agree(time.perf_counter() - t_settle < 0.4)
        for i in range(warmup):
            step(i)
        self.barrier()
        launches0 = net.launch_count()
        # A launch-bound workload (a few microseconds of kernel per step) is captured, K steps in a row, in one CUDA
        # graph and the timed region is one replay of it: otherwise the host's launch rate is what gets measured.
        graph = None
        if trainer is None and n <= (1 << 17):
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                handle = current_stream()
                for i in range(steps):
                    vx, vo = views[i % nsets]
                    check(lib().qmlp_network_inference(net._h, vx, vo, handle))
            graph.replay()
            torch.cuda.synchronize()
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        self.barrier()
        t0 = time.perf_counter()
        if graph is not None:
            events[0][0].record(stream)
            graph.replay()
            events[-1][1].record(stream)
        else:
            for i in range(steps):
                events[i][0].record(stream)
                step(i)
                events[i][1].record(stream)
        self.barrier()
        wall = time.perf_counter() - t0
        clocks = sampler.stop() if sampler else None
        launches = net.launch_count() - launches0
        span_ms = events[0][0].elapsed_time(events[-1][1])        # whole timed region on the device
        if graph is not None:
            launches = steps                                        # counted at capture; the replay launches the same K kernels
            dev_ms = [span_ms / steps] * steps
        else:
            dev_ms = [a.elapsed_time(b) for a, b in events]
        span_ms = self.max_over_ranks(span_ms)
        ms_per_step = span_ms / steps
        value = world * n * steps / (span_ms * 1e-3)

        # per-kernel device times of a few more steps (events around every launch inside the library; not part of the
        # timed region, the events cost a little)
        kernels = None
        if graph is None:
            check(lib().qmlp_set_kernel_timing(1))
            reps = 5
            for i in range(reps):
                step(i)
            torch.cuda.synchronize()
            kernels = read_kernel_timing(lib(), reps)
            check(lib().qmlp_set_kernel_timing(0))

        # end to end through the public call with host buffers
        e2e, host_link = self.end_to_end(net, trainer, xs, targets if trainer is not None else None, n, num_inputs, num_outputs,
                                         steps)

        out = {"ms_per_step": ms_per_step, "value": value, "n": n, "launches": int(launches), "clocks": clocks, "wall": wall,
               "kernel_ms": float(np.mean(dev_ms)), "e2e": e2e, "host_link": host_link, "kernels": kernels, "w": w, "key": key,
               "graph": graph is not None}
        if trainer is not None and world > 1:
            out["dp_check"] = self.dp_check(trainer)
        if trainer is not None:
            out["loss"] = trainer.mean_loss(world * n * max(1, trainer.step_count))
        return out

    # ------------------------------------------------------------------------------------------------------------------
    def end_to_end(self, net, trainer, xs, targets, n, num_inputs, num_outputs, steps):
        torch = self.torch
        from qmlp._capi import check, current_stream, lib
        hx = torch.empty((n, num_inputs), dtype=torch.float32).pin_memory()
        hx.copy_(xs[0].cpu())
        ho = torch.empty((n, num_outputs), dtype=torch.float32).pin_memory()
        if trainer is not None:
            ht = torch.empty((n, num_outputs), dtype=torch.float32).pin_memory()
            ht.copy_(targets[0].cpu())
            hloss = torch.empty((1,), dtype=torch.float32).pin_memory()

            def e2e_step(i):
                # the public host-memory step: this step's batch was uploaded while the previous step ran (prefetch of
                # the following batch on a copy stream); the loss comes back to the host every step
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
        e2e_steps = max(3, min(steps, 20))
        for i in range(2):
            e2e_step(i)
        self.barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        self.barrier()
        e2e_wall = self.max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": self.world * n * e2e_steps / e2e_wall, "unit": "points/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": e2e_wall / e2e_steps * 1e3}

        # what the host link alone allows: the step's uploads and downloads, both directions at once, on every rank at
        # the same time, no kernel
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        dx = torch.empty((h2d // 4,), dtype=torch.float32, device=self.dev)
        src = torch.empty((h2d // 4,), dtype=torch.float32).pin_memory()
        do = torch.empty((max(d2h // 4, 1),), dtype=torch.float32, device=self.dev)
        dst = torch.empty((max(d2h // 4, 1),), dtype=torch.float32).pin_memory()

        def link_step():
            with torch.cuda.stream(up):
                dx.copy_(src, non_blocking=True)
            with torch.cuda.stream(down):
                dst.copy_(do, non_blocking=True)
        for _ in range(2):
            link_step()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            link_step()
        self.barrier()
        link_wall = self.max_over_ranks(time.perf_counter() - t0)
        host_link = {"ms_per_step": link_wall / e2e_steps * 1e3, "gbs_all_ranks": self.world * (h2d + d2h) * e2e_steps / link_wall / 1e9,
                     "ceiling_points_per_s": self.world * n * e2e_steps / link_wall,
                     "note": "concurrent page-locked H2D + D2H of one step's bytes on all ranks, no kernel"}
        return e2e, host_link

    def dp_check(self, trainer):
        """After the timed steps: every replica must hold bit-identical parameters (same start, same all-reduced sums)."""
        torch, dist = self.torch, self.dist
        m0 = trainer.master.clone()
        dist.broadcast(m0, src=0)
        h0 = trainer.half.clone()
        dist.broadcast(h0, src=0)
        d = torch.stack([(trainer.master - m0).abs().max().double(), (trainer.half.float() - h0.float()).abs().max().double()])
        dist.all_reduce(d, op=dist.ReduceOp.MAX)
        # (every rank has taken the same number of steps: most and fewest over the ranks)
        c = torch.tensor([trainer.step_count, -trainer.step_count], device=self.dev, dtype=torch.int64)
        dist.all_reduce(c, op=dist.ReduceOp.MAX)
        return {"max_abs_master_diff_vs_rank0": float(d[0].item()), "max_abs_half_copy_diff_vs_rank0": float(d[1].item()),
                "steps_taken": int(trainer.step_count), "steps_taken_all_ranks": [int(-c[1].item()), int(c[0].item())],
                "nccl_bytes_per_step": int(trainer.gradient.numel() * 4),
                "collectives_per_step": trainer.collectives_per_step(self.world)}


def read_kernel_timing(lib, steps):
    import ctypes as C
    ids = (C.c_int * 64)()
    ms = (C.c_float * 64)()
    counts = (C.c_int * 64)()
    n = lib.qmlp_read_kernel_timing(64, ids, ms, counts)
    total = sum(ms[i] for i in range(n)) or 1.0
    out = {}
    for i in range(n):
        name = KERNEL_NAMES.get(ids[i], f"kernel{ids[i]}")
        out[name] = {"ms_per_step": ms[i] / steps, "launches_per_step": counts[i] / steps, "share": ms[i] / total}
    return out


def roofline_block(bench, r, fp32_tables):
    w, n, key = r["w"], r["n"], r["key"]
    peaks, src = bench.peaks, bench.peak_source
    kernel_ms = r["kernel_ms"]
    traffic = {} if fp32_tables else measured_traffic_per_point().get(key, {})
    if w["mode"] == "inference" and w["bytes"] <= 64:
        # the layer chain of an identity-encoded network: tensor bound
        peak_s = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
        peak_b = float(peaks.get("bf16_tflops", peak_s))
        achieved = w["flops"] * n / (kernel_ms * 1e-3) / 1e12
        per_point = traffic.get("inference")
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak_b, "unit": "TFLOP/s", "frac": achieved / peak_b,
                "traffic": per_point * n if per_point is not None else None,
                "peak_source": f"{src} bf16_tflops (burst: the timed region is a few milliseconds at full clock)",
                "frac_of_sustained": achieved / peak_s, "kernel_ms": kernel_ms, "algorithmic_flops_per_point": w["flops"]}
    else:
        peak = float(peaks["hbm_gbs"])
        bytes_per_point = w["bytes"] + (w.get("gather_bytes", 0) if fp32_tables else 0)   # fp32 rows are twice as wide
        achieved = bytes_per_point * n / (kernel_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic["all"] * n if "all" in traffic else None, "peak_source": f"{src} hbm_gbs", "kernel_ms": kernel_ms,
                "algorithmic_bytes_per_point": bytes_per_point,
                "scope": "all kernels of one step (the step is a chain of kernels; `kernels` lists each one's share)"}
    if r["kernels"]:
        name, k = max(r["kernels"].items(), key=lambda kv: kv[1]["ms_per_step"])
        roof["dominant_kernel"] = {"name": name, "ms_per_step": k["ms_per_step"], "share": k["share"],
                                   "traffic": traffic[name] * n if name in traffic else None}
    return roof


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=["c1", "c2", "c3", "c3i", "c4", "c5"])
    ap.add_argument("--points", type=int, default=0, help="override the points per GPU and step of the primary workload")
    ap.add_argument("--fp32-tables", action="store_true", help="gather from fp32 grid tables (reference layout)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="only the primary workload")
    ap.add_argument("--dp-levels-per-launch", type=int, default=-1,
                    help="grid levels per scatter launch of the data-parallel step (0: one launch, one all-reduce of all "
                         "table gradients under the weight-gradient kernel; default: the trainer's own choice)")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="tuning switch of the training step for an A/B measurement (qmlp_set_tuning), e.g. sort_points=0")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    # A run that has produced no line after a quarter of an hour (several times what any configuration needs) ends itself
    # instead of holding the GPUs; the timer thread fires even while the main thread waits inside a CUDA or NCCL call.
    import threading

    def give_up():
        sys.stderr.write("bench.py: no result within 900 s, giving up\n")
        sys.stderr.flush()
        os._exit(124)
    watchdog = threading.Timer(900.0, give_up)
    watchdog.daemon = True
    watchdog.start()

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from qmlp import bindings, load_library

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the fused kernels")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    try:
        all_cores = os.sched_getaffinity(0)
    except AttributeError:
        all_cores = None
    numa = bind_to_gpu_numa_node(torch, local_rank)
    if world > 1:
        # The data-parallel step runs its all-reduces underneath kernels that are bound by the L2; on eight GPUs NCCL's
        # ring kernels disturb them less than its NVSwitch-multicast (NVLS) ones: 1.47 against 1.54 ms per step. (Four
        # GPUs: 1.36 against 1.39; left at NCCL's default there.) A user's own setting wins.
        if world >= 8:
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        # a collective that does not complete within three minutes ends the run with an error instead of hanging it
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    load_library()
    bindings.QuickMLP.set_log_level("error")
    for item in args.tune:
        k, _, v = item.partition("=")
        bindings.QuickMLP.set_tuning(k, int(v))

    bench = Bench(args, rank, local_rank, world)
    key = args.workload
    r = bench.run(key, args.steps, args.warmup, primary=True)
    secondary = {}
    if not args.no_secondary and args.points == 0:
        for k2 in SECONDARY.get(key, ()):
            s = bench.run(k2, max(3, min(args.steps, 30)), args.warmup, primary=False)
            blk = {"workload": s["w"]["name"], "points_per_gpu_per_step": s["n"], "ms_per_step": s["ms_per_step"],
                   "value": s["value"], "unit": "points/s", "roofline": roofline_block(bench, s, args.fp32_tables),
                   "e2e": s["e2e"], "host_link": s["host_link"], "kernels": s["kernels"]}
            secondary[k2] = blk

    if rank == 0:
        w = r["w"]
        line = {"metric": METRIC, "value": r["value"], "unit": "points/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                "scaling": "strong" if w.get("sharded") else "weak",
                "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
                "config": config_block(key, w, r["n"], world, args.fp32_tables),
                "e2e": r["e2e"], "host_link": r["host_link"], "gpu_launches": r["launches"], "clocks": r["clocks"],
                "roofline": roofline_block(bench, r, args.fp32_tables), "kernels": r["kernels"],
                "wall_s_timed_region": r["wall"], "host_binding": numa}
        if args.tune:
            line["tuning"] = args.tune
        if r["graph"]:
            line["launch"] = "the K steps are one CUDA graph (launch-bound workload); the timed region is one replay"
        if "dp_check" in r:
            line["dp_check"] = r["dp_check"]
        if "loss" in r:
            line["mean_loss"] = r["loss"]
        if secondary:
            line["secondary"] = secondary
        if not args.no_cpu_baseline and world == 1:
            if all_cores is not None:
                try:
                    os.sched_setaffinity(0, all_cores)
                except OSError:
                    pass
            try:
                line["cpu_baseline"] = cpu_baseline(key, w, host_threads(all_cores))
            except Exception as e:   # the baseline is a reported extra; never lose the measured line over it
                line["cpu_baseline"] = {"value": None, "unit": "points/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
