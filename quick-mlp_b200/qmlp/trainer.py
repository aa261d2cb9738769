"""Fused training step and batch sharding for one process per GPU.

The reference has no trainer: its users write ``mse_loss`` + ``torch.optim.Adam`` around ``FusedNetwork.forward``
(tests_py/qmlp_tests/test_network_image.py:41-55). ``FusedTrainer`` runs that loop as a handful of kernels per step
(encode pass, forward with stash and loss gradient, backward, table-gradient scatter, weight/bias gradients, Adam) over
one fused fp32 gradient buffer ``[network | encoding 0 | encoding 1 ...]``. With ``torch.distributed`` initialised the
step is data parallel: the gradient buffer is summed over the ranks slice by slice, each slice as soon as the launch
that produces it has finished, so that the all-reduces run underneath the kernels that follow. Inference needs no
communication and is sharded by ``shard_points``.
"""
import ctypes as C
from typing import Optional

import torch

from . import _capi
from ._capi import check, current_stream, lib, wrap
from .bindings import Network


def shard_points(num_points: int, rank: int, world_size: int):
    """Contiguous, balanced shard [begin, end) of a point batch for ``rank``; the first ``num_points % world_size``
    ranks hold one point more."""
    base, rem = divmod(num_points, world_size)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class _CudaStep:
    """The compute backend of a training step: the CUDA kernels behind the C ABI."""

    def __init__(self, network: Network, lr, beta1, beta2, eps, grid_half_copy, device):
        self.network = network
        cfg = _capi.TrainerConfig(lr, beta1, beta2, eps, int(grid_half_copy), 0)
        h = C.c_void_p()
        check(lib().qmlp_trainer_create(network._h, C.byref(cfg), C.byref(h)))
        self._h = h
        self.fused_count = lib().qmlp_trainer_fused_count(h)
        self.segments = [lib().qmlp_trainer_segment_start(h, i) for i in range(1 + network.num_encodings())]
        self.device = device
        self._workspace = None

    def __del__(self):
        try:
            if getattr(self, "_h", None) and _capi._lib is not None:
                _capi._lib.qmlp_trainer_destroy(self._h)
                self._h = None
        except Exception:   # interpreter shutdown: module globals may already be gone
            pass

    def bind(self, master, grad, m, v, half):
        check(lib().qmlp_trainer_bind(self._h, master.data_ptr(), grad.data_ptr(), m.data_ptr(), v.data_ptr(), half.data_ptr()))

    def refresh_half(self):
        check(lib().qmlp_trainer_refresh_half(self._h, current_stream()))

    split_gradients = True   # gradients(..., parts=1) then gradients(..., parts=2) is supported

    def scatter_levels(self):
        """[(first element, end element)] of every grid level in the fused buffers, in scatter order; [] when the table
        gradients of this network are not scattered by a kernel of their own."""
        n = lib().qmlp_trainer_scatter_levels(self._h, 0, None, None)
        if n <= 0:
            return []
        b, e = (C.c_int64 * n)(), (C.c_int64 * n)()
        lib().qmlp_trainer_scatter_levels(self._h, n, b, e)
        return [(b[i], e[i]) for i in range(n)]

    def gradients(self, x, target, global_points, loss_sum, parts=3):
        """parts: 1 = forward, backward, table gradients; 2 = weight/bias gradients of the layers; 3 = both;
        4 = forward and backward with the scatter deferred; 8 | first << 8 | end << 16 = scatter of grid levels
        [first, end)."""
        b = C.c_size_t()
        check(lib().qmlp_trainer_workspace_bytes(self._h, x.shape[0], C.byref(b)))
        if self._workspace is None or self._workspace.numel() < b.value:
            self._workspace = torch.empty((b.value,), dtype=torch.uint8, device=x.device)
        check(lib().qmlp_trainer_gradients_part(self._h, wrap(x), wrap(target), global_points, self._workspace.data_ptr(),
                                                self._workspace.numel(), loss_sum.data_ptr() if loss_sum is not None else None,
                                                parts, current_stream()))

    def update(self, step, grad_scale):
        check(lib().qmlp_trainer_update(self._h, step, grad_scale, current_stream()))


class FusedTrainer:
    """Data-parallel fused trainer for one replica of a network.

    master / gradient / Adam moments are fp32 vectors of ``fused_count`` elements; ``half`` is the fp16 working copy
    the kernels read (network weights always, grid tables when ``grid_half_copy``). Gradients are normalised by the
    global point count inside the kernels, so the all-reduce is a plain sum.
    """

    def __init__(self, network: Network, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, grid_half_copy=True,
                 device="cuda", process_group=None, backend=None):
        self.network = network
        self.device = torch.device(device)
        self.backend = backend if backend is not None else _CudaStep(network, lr, beta1, beta2, eps, grid_half_copy, self.device)
        n = self.backend.fused_count
        self.master = torch.zeros((n,), dtype=torch.float32, device=self.device)
        self.gradient = torch.zeros((n,), dtype=torch.float32, device=self.device)
        self.adam_m = torch.zeros((n,), dtype=torch.float32, device=self.device)
        self.adam_v = torch.zeros((n,), dtype=torch.float32, device=self.device)
        self.half = torch.zeros((n,), dtype=torch.float16, device=self.device)
        self.loss_sum = torch.zeros((1,), dtype=torch.float32, device=self.device)
        self.backend.bind(self.master, self.gradient, self.adam_m, self.adam_v, self.half)
        self.step_count = 0
        self.process_group = process_group
        self.level_group_size = 3      # grid levels per scatter launch of a data-parallel step (0: one launch)

    # -- parameter access ---------------------------------------------------------------------------------------------
    def segment(self, buffer: torch.Tensor, index: int) -> Optional[torch.Tensor]:
        """View of segment ``index`` (0 = network, 1 + i = encoding i) of one of the fused buffers."""
        start = self.backend.segments[index]
        if start < 0:
            return None
        count = self.network.num_network_parameters() if index == 0 else self.network.encoding(index - 1).parameter_count()
        return buffer[start:start + count]

    def set_parameters(self, network_parameters: torch.Tensor, encoding_parameters=()):
        """Loads fp32 (or fp16) parameters into the master copy and refreshes the half copy."""
        self.segment(self.master, 0).copy_(network_parameters.to(torch.float32))
        for i, p in enumerate(encoding_parameters):
            if p is not None and self.backend.segments[1 + i] >= 0:
                self.segment(self.master, 1 + i).copy_(p.to(torch.float32))
        self._sync_replicas()
        self.backend.refresh_half()

    def _sync_replicas(self):
        """Data-parallel replicas must start from the same parameters: rank 0's master copy (and Adam state) is broadcast,
        so that a caller who seeds by rank, or loads a checkpoint on one rank only, still gets one consistent model."""
        dist, world = self._world()
        if world > 1:
            src = dist.get_global_rank(self.process_group, 0) if self.process_group is not None else 0
            for t in (self.master, self.adam_m, self.adam_v):
                dist.broadcast(t, src=src, group=self.process_group)

    def _level_groups(self, world_size: int):
        """[(first level, end level, first element, end element)]: the launches the table-gradient scatter is cut into
        for a data-parallel step, each followed by the all-reduce of its part of the gradient vector. The element ranges
        tile [first table segment, fused_count). Three levels per launch, the first launch takes what is left over (the
        coarse levels are small): the last all-reduce is then short enough to hide under the weight-gradient kernel.
        [] when the scatter is not a kernel of its own, or on one rank."""
        key = ("groups", world_size, self.level_group_size)
        cached = getattr(self, "_groups_cache", None)
        if cached is not None and cached[0] == key:
            return cached[1]
        levels = self.backend.scatter_levels() if (world_size > 1 and hasattr(self.backend, "scatter_levels")) else []
        groups = []
        if len(levels) >= 2 and self.level_group_size > 0:
            cuts = list(range(len(levels), 0, -self.level_group_size))[::-1][-4:]      # at most four: L - 9, L - 6, L - 3, L
            first_table = min(s for s in self.backend.segments[1:] if s >= 0)
            lo = 0
            for hi in cuts:
                begin = first_table if lo == 0 else levels[lo][0]
                end = self.backend.fused_count if hi == len(levels) else levels[hi][0]
                groups.append((lo, hi, begin, end))
                lo = hi
        self._groups_cache = (key, groups)
        return groups

    def collectives_per_step(self, world_size: int) -> int:
        """Number of all-reduce calls one step issues at this world size."""
        if world_size <= 1:
            return 0
        table_starts = [s for s in self.backend.segments[1:] if s >= 0]
        groups = self._level_groups(world_size) if table_starts else []
        if groups:
            return len(groups) + 1
        return 2 if (table_starts and getattr(self.backend, "split_gradients", False)) else 1

    def state_dict(self):
        return {"master": self.master, "adam_m": self.adam_m, "adam_v": self.adam_v, "step": self.step_count}

    def load_state_dict(self, state):
        self.master.copy_(state["master"])
        self.adam_m.copy_(state["adam_m"])
        self.adam_v.copy_(state["adam_v"])
        self.step_count = int(state["step"])
        self._sync_replicas()
        self.backend.refresh_half()

    # -- one step -----------------------------------------------------------------------------------------------------
    def _world(self):
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist, dist.get_world_size(self.process_group)
        return None, 1

    def step(self, x: torch.Tensor, target: torch.Tensor, global_points: Optional[int] = None):
        """forward + L2 loss + backward + (all-reduce) + Adam on this rank's points.
        ``global_points`` defaults to ``world_size * x.shape[0]`` (equal shards)."""
        dist, world = self._world()
        if global_points is None:
            global_points = world * x.shape[0]
        table_starts = [s for s in self.backend.segments[1:] if s >= 0]
        groups = self._level_groups(world) if world > 1 and table_starts else []
        if groups:
            # The scatter kernel works through the grid levels in a few launches. The gradient of a level is final when
            # its launch is: its all-reduce starts then (on the communication stream) and runs underneath the scatter of
            # the following levels, the last one underneath the layers' weight-gradient kernel.
            self.backend.gradients(x, target, global_points, self.loss_sum, parts=4)
            pending = []
            for level_begin, level_end, begin, end in groups:
                self.backend.gradients(x, target, global_points, self.loss_sum, parts=8 | (level_begin << 8) | (level_end << 16))
                pending.append(dist.all_reduce(self.gradient[begin:end], op=dist.ReduceOp.SUM, group=self.process_group, async_op=True))
            self.backend.gradients(x, target, global_points, self.loss_sum, parts=2)
            dist.all_reduce(self.gradient[:groups[0][2]], op=dist.ReduceOp.SUM, group=self.process_group)
            for p in pending:
                p.wait()
        elif world > 1 and table_starts and getattr(self.backend, "split_gradients", False):
            # The table gradients (nearly all of the vector) are final before the layers' weight gradients are computed:
            # their all-reduce runs on the communication stream underneath the weight-gradient kernel.
            first = min(table_starts)
            self.backend.gradients(x, target, global_points, self.loss_sum, parts=1)
            pending = dist.all_reduce(self.gradient[first:], op=dist.ReduceOp.SUM, group=self.process_group, async_op=True)
            self.backend.gradients(x, target, global_points, self.loss_sum, parts=2)
            dist.all_reduce(self.gradient[:first], op=dist.ReduceOp.SUM, group=self.process_group)
            pending.wait()
        else:
            self.backend.gradients(x, target, global_points, self.loss_sum)
            if world > 1:
                dist.all_reduce(self.gradient, op=dist.ReduceOp.SUM, group=self.process_group)
        self.step_count += 1
        self.backend.update(self.step_count, 1.0)

    # -- batches that live in host memory ---------------------------------------------------------------------------
    def _staging(self, x: torch.Tensor, target: torch.Tensor):
        st = getattr(self, "_host_staging", None)
        if st is None or st["x"][0].shape != x.shape or st["t"][0].shape != target.shape:
            st = {"x": [torch.empty(x.shape, dtype=torch.float32, device=self.device) for _ in range(2)],
                  "t": [torch.empty(target.shape, dtype=torch.float32, device=self.device) for _ in range(2)],
                  "ready": [torch.cuda.Event(), torch.cuda.Event()], "free": [torch.cuda.Event(), torch.cuda.Event()],
                  "stream": torch.cuda.Stream(device=self.device), "slot": 0, "pending": None}
            self._host_staging = st
        return st

    def _upload(self, st, slot, x, target):
        """Queues the upload of a host batch into staging slot `slot` on the copy stream."""
        copy = st["stream"]
        copy.wait_event(st["free"][slot])           # the step that last read this slot has been queued and will finish first
        with torch.cuda.stream(copy):
            st["x"][slot].copy_(x, non_blocking=True)
            st["t"][slot].copy_(target, non_blocking=True)
            st["ready"][slot].record(copy)
        st["pending"] = (slot, x.data_ptr(), target.data_ptr())

    def step_host(self, x: torch.Tensor, target: torch.Tensor, next_batch=None, global_points: Optional[int] = None):
        """One training step on a batch in (page-locked) host memory. ``next_batch`` = (x, target) of the following
        call: its upload is queued on a copy stream before this step's kernels, so it crosses the host link while they
        run, and the following ``step_host`` finds it on the device."""
        assert x.device.type == "cpu" and target.device.type == "cpu"
        st = self._staging(x, target)
        main = torch.cuda.current_stream()
        pending = st["pending"]
        if pending is not None and pending[1:] == (x.data_ptr(), target.data_ptr()):
            slot = pending[0]                       # prefetched by the previous call
        else:
            slot = st["slot"]
            st["free"][slot].record(main)
            self._upload(st, slot, x, target)
        st["pending"] = None
        main.wait_event(st["ready"][slot])
        if next_batch is not None:
            other = slot ^ 1
            st["free"][other].record(main)          # everything queued so far (all earlier steps) precedes the overwrite
            self._upload(st, other, next_batch[0], next_batch[1])
        self.step(st["x"][slot], st["t"][slot], global_points)
        st["slot"] = slot ^ 1

    def mean_loss(self, global_points: int, reset=True) -> float:
        """Mean squared error accumulated since the last reset (synchronises)."""
        dist, world = self._world()
        s = self.loss_sum.clone()
        if world > 1:
            dist.all_reduce(s, op=dist.ReduceOp.SUM, group=self.process_group)
        if reset:
            self.loss_sum.zero_()
        return float(s.item()) / (global_points * self.network.channels_out())

    def inference(self, x: torch.Tensor) -> torch.Tensor:
        """Fused inference with the current half copy of all parameters."""
        out = torch.empty((x.shape[0], self.network.channels_out()), dtype=torch.float32, device=x.device)
        check(lib().qmlp_network_inference(self.network._h, wrap(x), wrap(out), current_stream()))
        return out
