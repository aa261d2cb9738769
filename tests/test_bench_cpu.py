"""Host-side pieces of bench.py that need no GPU: the reference arm on a tiny sample, the workload table, the DRAM
traffic figures it reads from profiles/dram_traffic.md."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_traffic_table_is_read_from_the_profile():
    table = _bench().measured_traffic_per_point()
    assert table["c2"]["inference"] > 0
    c3 = table["c3"]
    kernels = [k for k in c3 if k != "all"]
    assert set(kernels) >= {"scatter_planes", "encode_planes", "forward_loss_planes", "backward", "wgrad", "adam"}
    assert abs(sum(c3[k] for k in kernels) - c3["all"]) < 1.0   # the `all` row is the sum of the kernel rows


def test_config_block_is_the_same_on_both_arms():
    bench = _bench()
    from qmlp import configs
    w = dict(configs.WORKLOADS["c3"])
    a = bench.config_block("c3", w, w["points"], 1, False)
    b = bench.config_block("c3", w, w["points"], 1, False)
    assert a == b and a["mode"] == "train" and "workload" in a and a["parallelism"] == "dp1"
    assert bench.config_block("c3", w, w["points"], 8, False)["parallelism"].startswith("dp8")


def test_reference_arm_prints_one_json_line():
    env = dict(os.environ, OMP_NUM_THREADS="4")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.strip().splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["value"] > 0 and d["cpu_baseline"]["kind"] == "port"
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0


def _agree_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    bench = _bench()
    b = bench.Bench.__new__(bench.Bench)
    b.torch, b.dist, b.world, b.rank, b.dev = torch, dist, world, rank, torch.device("cpu")
    # the settling loop of a data-parallel run: a rank whose own clock says "stop" makes every rank stop
    answers = [b.all_ranks_agree(True), b.all_ranks_agree(rank == 0), b.all_ranks_agree(False)]
    with open(os.path.join(out_dir, f"agree{rank}.json"), "w") as f:
        json.dump(answers, f)
    dist.destroy_process_group()


def test_ranks_agree_on_going_on(tmp_path):
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_agree_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        with open(tmp_path / f"agree{rank}.json") as f:
            assert json.load(f) == [True, False, False]
