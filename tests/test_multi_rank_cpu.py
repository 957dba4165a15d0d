"""World-size-2 gloo test of the multi-rank plumbing the benchmark uses: every rank takes its own batch of
independent images (no collective on the data path), times are reduced with MAX, rank 0 aggregates units."""
import os
import socket
import subprocess
import sys
import textwrap

HERE = os.path.dirname(os.path.abspath(__file__))

WORKER = textwrap.dedent("""
    import os, sys, json
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, os.path.join(sys.argv[1], "tests")); sys.path.insert(0, sys.argv[1])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    import importlib
    from conftest import load_package
    enn = load_package()
    import mobilenet_ref
    mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")
    layers, _ = mn.build_model(seed=0, calib_images=1, resolution=32, num_classes=10)
    # each rank owns a contiguous slice of the global batch, seeded by rank as the benchmark does
    x = np.random.default_rng(1000 + rank).integers(0, 256, (2, 32, 32, 3), dtype=np.int64).astype(np.uint8)
    y = mobilenet_ref.run_oracle(layers, x)                 # CPU stand-in for the per-rank device graph
    t = torch.tensor([1.0 + rank, 2.0 + 0.5 * rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)                # timing rule: max over ranks
    gathered = [torch.zeros(2, 10, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(y.copy()))   # only the final logits are gathered
    if rank == 0:
        print(json.dumps({"max_ms": t.tolist(), "units": 2 * world, "rows": int(torch.cat(gathered).shape[0]),
                          "distinct": bool((gathered[0] != gathered[1]).any())}))
    dist.destroy_process_group()
""")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_gloo_sharding(tmp_path):
    import json
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    root = os.path.dirname(HERE)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(script), root]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env={**os.environ, "OMP_NUM_THREADS": "2"})
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    out = json.loads(line)
    assert out["max_ms"] == [2.0, 2.5]
    assert out["units"] == 4 and out["rows"] == 4 and out["distinct"]


def test_reference_arm_runs_on_rank0_only():
    """bench.py --impl reference: rank 0 prints the line, other ranks exit 0 without work."""
    root = os.path.dirname(HERE)
    env = {**os.environ, "RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                       capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""
