"""The data-parallel training step on real GPUs: FusedTrainer.step over NCCL with one process per GPU (the CUDA
kernels and the all-reduce calls the CPU test of the same logic replaces by test doubles). Needs two devices; skipped
with fewer. Replicas must hold bit-identical parameters after every step (same start, same all-reduced sums), and two
ranks on half batches must reproduce one GPU on the whole batch within the tolerance of the trainer tests."""
import json
import os
import socket

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs
from test_gpu_trainer import _target, smooth_config3

pytestmark = pytest.mark.gpu

STEPS, POINTS = 3, 4096


def _batches():
    return [helpers.uniform(200 + s, 1, (POINTS, 3)) for s in range(STEPS)]


def _train(rank, world, device, seed_offset=0):
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer, shard_points
    cfg = smooth_config3()
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.05).astype(np.float32)
    table = helpers.grid_tables(spec, scale=0.1)[0]
    if seed_offset:
        params = params + np.float32(0.125) * seed_offset        # a replica initialised differently: corrected by the broadcast
    tr = FusedTrainer(bindings.Network(json.dumps(cfg)), lr=1e-2, device=device)
    tr.set_parameters(torch.from_numpy(params).to(device), [torch.from_numpy(table).to(device)])
    hashes = []
    for x in _batches():
        b, e = shard_points(POINTS, rank, world)
        xs = torch.from_numpy(x[b:e]).to(device)
        tr.step(xs, torch.from_numpy(_target(x[b:e])).to(device), global_points=POINTS)
        hashes.append(tr.master.clone())
    torch.cuda.synchronize(device)
    return tr, hashes


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from qmlp import bindings, load_library
    load_library()
    tr, per_step = _train(rank, world, device, seed_offset=rank)
    # bit-identical replicas after every step: compare with rank 0's copy on the device
    worst = 0.0
    for m in per_step:
        m0 = m.clone()
        dist.broadcast(m0, src=0)
        worst = max(worst, float((m - m0).abs().max().item()))
    loss = tr.mean_loss(POINTS * STEPS)
    np.save(os.path.join(out_dir, f"master{rank}.npy"), tr.master.cpu().numpy())
    np.save(os.path.join(out_dir, f"info{rank}.npy"), np.array([worst, loss, float(bindings.QuickMLP.device_status())]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_gpu_replicas_identical_and_equal_to_one_gpu(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    m0, m1 = np.load(tmp_path / "master0.npy"), np.load(tmp_path / "master1.npy")
    i0, i1 = np.load(tmp_path / "info0.npy"), np.load(tmp_path / "info1.npy")
    assert i0[2] == 0 and i1[2] == 0                                   # no kernel gave up on a wait
    assert i0[0] == 0.0 and i1[0] == 0.0, "replicas differed after a step"
    np.testing.assert_array_equal(m0, m1)
    assert abs(i0[1] - i1[1]) < 1e-9

    from qmlp import load_library
    load_library()
    single, _ = _train(0, 1, torch.device("cuda", 0))
    ms = single.master.cpu().numpy()
    cfg = smooth_config3()
    spec = oracle.parse_spec(cfg)
    start_w = helpers.xavier_parameters(spec, cfg, bias_scale=0.05).astype(np.float32)
    n_w = spec.num_parameters
    # Adam moves every touched entry by about lr per step whatever the gradient's size: compare the updates
    helpers.assert_close(m0[:n_w] - start_w, ms[:n_w] - start_w, "network update, 2 GPUs against 1", rtol=5e-2, atol=2e-3,
                         max_violations=0.02)
    seg = single.backend.segments[1]
    table = helpers.grid_tables(spec, scale=0.1)[0]
    helpers.assert_close(m0[seg:seg + table.size] - table, ms[seg:seg + table.size] - table, "grid update, 2 GPUs against 1",
                         rtol=5e-2, atol=2e-3, max_violations=0.02)
    loss_single = single.mean_loss(POINTS * STEPS)
    assert abs(loss_single - i0[1]) <= 1e-4 * max(1.0, abs(loss_single))
