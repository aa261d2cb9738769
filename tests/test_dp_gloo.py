"""Data-parallel path of FusedTrainer on CPU ranks (gloo, world size 2): the sharding helper, the single all-reduce of
the fused gradient buffer and the update ordering, with the oracle standing in for the CUDA step (injected through the
trainer's `backend` argument, which only tests use). Two ranks on half batches must reproduce one rank on the whole
batch. The reference has no multi-GPU path; this covers what this build adds around its hot path."""
import json
import os
import socket

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs


class OracleStep:
    """Test double with the interface of qmlp.trainer._CudaStep, computing on the CPU with the oracle."""

    def __init__(self, cfg):
        self.spec = oracle.parse_spec(cfg)
        align = lambda v: (v + 63) // 64 * 64
        self.segments, pos = [0], align(self.spec.num_parameters)
        for e in self.spec.encodings:
            if e.num_parameters:
                self.segments.append(pos)
                pos = align(pos + e.num_parameters)
            else:
                self.segments.append(-1)
        self.fused_count = pos

    def bind(self, master, grad, m, v, half):
        self.master, self.grad, self.m, self.v, self.half = master, grad, m, v, half

    def refresh_half(self):
        self.half.copy_(self.master.half())

    def _views(self, buf):
        w = buf[:self.spec.num_parameters].numpy()
        t = [buf[s:s + e.num_parameters].numpy() if s >= 0 else None for s, e in zip(self.segments[1:], self.spec.encodings)]
        return w, t

    split_gradients = True

    def scatter_levels(self):
        """Element ranges of the grid levels in the fused buffers, as qmlp_trainer_scatter_levels reports them."""
        out = []
        for seg, e in zip(self.segments[1:], self.spec.encodings):
            for i, lv in enumerate(e.levels):
                end = e.levels[i + 1].memory_offset if i + 1 < len(e.levels) else e.num_parameters
                out.append((seg + lv.memory_offset, seg + end))
        return out

    def gradients(self, x, target, global_points, loss_sum, parts=3):
        """parts as in qmlp_trainer_gradients_part: 1 = up to the table gradients, 2 = the layers' weight gradients,
        4 = forward and backward with the scatter deferred, 8 | first << 8 | end << 16 = scatter of a level range."""
        what, first, end = parts & 0xff, (parts >> 8) & 0xff, (parts >> 16) & 0xff
        if what in (4, 8):
            if what == 4:
                w, t = self._views(self.half.float())
                out = oracle.network_forward(self.spec, w, x.numpy(), t)
                adj = oracle.mse_loss_grad(out, target.numpy(), global_points)
                self._pending = oracle.network_backward(self.spec, w, x.numpy(), adj, t, want_input=False)
                loss_sum += float(((out - target.numpy()) ** 2).sum())
                self._scattered = []
            else:
                ranges = self.scatter_levels()[first:end]
                flat = np.zeros(self.fused_count, dtype=np.float32)
                for seg, g in zip(self.segments[1:], self._pending.grad_encodings):
                    if g is not None:
                        flat[seg:seg + g.size] = g
                for b, e in ranges:
                    self.grad[b:e] += torch_from(flat[b:e])
                self._scattered += list(range(first, end))
            self.parts_seen = getattr(self, "parts_seen", []) + [parts]
            return
        if parts & 1:
            w, t = self._views(self.half.float())
            out = oracle.network_forward(self.spec, w, x.numpy(), t)
            adj = oracle.mse_loss_grad(out, target.numpy(), global_points)
            self._pending = oracle.network_backward(self.spec, w, x.numpy(), adj, t, want_input=False)
            _, gt = self._views(self.grad)
            for a, b in zip(gt, self._pending.grad_encodings):
                if a is not None:
                    a += b
            loss_sum += float(((out - target.numpy()) ** 2).sum())
            self.parts_seen = getattr(self, "parts_seen", []) + [1]
        if parts & 2:
            gw, _ = self._views(self.grad)
            gw += self._pending.grad_params
            self.parts_seen = getattr(self, "parts_seen", []) + [2]

    def update(self, step, grad_scale):
        oracle.adam_step(self.master.numpy(), self.grad.numpy() * grad_scale, self.m.numpy(), self.v.numpy(), step)
        self.grad.zero_()
        self.refresh_half()


def torch_from(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a))


def _cfg():
    cfg = specs.config3(log2_hashmap_size=8)
    cfg["encodings"][0].update(n_levels=4, max_resolution=54)
    cfg["network"] = specs.mlp([16, 1], ["celu", "identity"], True)
    return cfg


def _train(rank, world, x, t, steps):
    import torch
    from qmlp.trainer import FusedTrainer, shard_points

    class FakeNetwork:       # the trainer only asks the network for sizes
        def __init__(self, spec):
            self.spec = spec

        def num_network_parameters(self):
            return self.spec.num_parameters

        def num_encodings(self):
            return len(self.spec.encodings)

        def channels_out(self):
            return self.spec.num_outputs

        def encoding(self, i):
            e = self.spec.encodings[i]
            return type("E", (), {"parameter_count": lambda self_: e.num_parameters})()

    cfg = _cfg()
    backend = OracleStep(cfg)
    tr = FusedTrainer(FakeNetwork(backend.spec), device="cpu", backend=backend)
    params = helpers.xavier_parameters(backend.spec, cfg, bias_scale=0.05).astype(np.float32)
    if rank > 0:
        params = params + np.float32(0.25)   # a replica seeded differently: set_parameters broadcasts rank 0's copy over it
    tr.set_parameters(torch.from_numpy(params), [torch.from_numpy(tb) if tb is not None else None
                                                 for tb in helpers.grid_tables(backend.spec, scale=0.1)])
    b, e = shard_points(x.shape[0], rank, world)
    for _ in range(steps):
        tr.step(torch.from_numpy(x[b:e]), torch.from_numpy(t[b:e]), global_points=x.shape[0])
    if world > 1:
        # the data-parallel step cut the scatter into level groups, each followed by its own all-reduce
        seen = [p & 0xff for p in backend.parts_seen]
        assert seen.count(4) == steps and seen.count(8) == steps * len(tr._level_groups(world)) and seen.count(2) == steps
        assert sorted(backend._scattered) == list(range(len(backend.scatter_levels())))
    return tr.master.numpy().copy(), tr.mean_loss(x.shape[0] * steps)


def _worker(rank, world, port, x, t, steps, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    master, loss = _train(rank, world, x, t, steps)
    np.save(os.path.join(out_dir, f"master{rank}.npy"), master)
    np.save(os.path.join(out_dir, f"loss{rank}.npy"), np.array([loss]))
    dist.destroy_process_group()


def test_shard_points():
    from qmlp.trainer import shard_points
    for n, w in ((10, 3), (1 << 24, 8), (7, 8), (0, 2)):
        shards = [shard_points(n, r, w) for r in range(w)]
        assert shards[0][0] == 0 and shards[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(shards, shards[1:]))
        sizes = [e - b for b, e in shards]
        assert max(sizes) - min(sizes) <= 1


def test_level_groups_tile_the_table_gradients():
    """Whatever the number of grid levels: the scatter launches of a data-parallel step cover every level exactly once,
    and the slices that are all-reduced after them tile [first table element, fused_count) without gap or overlap."""
    from qmlp.trainer import FusedTrainer

    class Levels:
        segments = [0, 7360]

        def __init__(self, count):
            self.count = count
            self.fused_count = 7360 + 100 * count + 28   # with alignment slack after the last level

        def scatter_levels(self):
            return [(7360 + 100 * i, 7360 + 100 * (i + 1)) for i in range(self.count)]

    for count in (1, 2, 3, 4, 7, 8, 9, 16, 17, 32):
        for size in (0, 1, 3, 8):
            tr = FusedTrainer.__new__(FusedTrainer)
            tr.backend, tr.level_group_size = Levels(count), size
            groups = tr._level_groups(4)
            if count < 2 or size == 0:
                assert groups == []
                continue
            assert 1 <= len(groups) <= 4
            by_level = sorted(groups)
            assert by_level[0][0] == 0 and by_level[-1][1] == count
            assert all(a[1] == b[0] and a[3] == b[2] for a, b in zip(by_level, by_level[1:]))
            assert by_level[0][2] == 7360 and by_level[-1][3] == tr.backend.fused_count
            assert tr.collectives_per_step(4) == len(groups) + 1
        assert FusedTrainer._level_groups(tr, 1) == []          # one rank: no groups


@pytest.mark.timeout(300)
def test_two_ranks_equal_one_rank(tmp_path):
    import torch.multiprocessing as mp
    n, steps = 512, 3
    x = helpers.uniform(5, 1, (n, 3))
    t = (np.sin(8 * x[:, 0]) * np.cos(6 * x[:, 1]) * np.sin(4 * x[:, 2])).astype(np.float32)[:, None]
    single, loss1 = _train(0, 1, x, t, steps)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, x, t, steps, str(tmp_path)), nprocs=2, join=True)
    m0, m1 = np.load(tmp_path / "master0.npy"), np.load(tmp_path / "master1.npy")
    np.testing.assert_array_equal(m0, m1)                                  # replicas stay identical
    # Adam normalises each update to about lr, so compare the update with a floor well below lr = 1e-2
    np.testing.assert_allclose(m0, single, rtol=1e-3, atol=2e-4)
    l0, l1 = float(np.load(tmp_path / "loss0.npy")[0]), float(np.load(tmp_path / "loss1.npy")[0])
    assert abs(l0 - l1) < 1e-9 and abs(l0 - loss1) < 1e-5 * max(1.0, abs(loss1))
