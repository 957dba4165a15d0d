"""World-size-2 gloo test of the multi-rank plumbing the benchmark uses: ONE global batch is partitioned into
contiguous slices, one per rank (no collective on the data path), times are reduced with MAX, and only the logits are
gathered on rank 0, where they must equal the whole batch run in one piece."""
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
    # every rank draws the same global batch and owns a contiguous slice of it, as the benchmark does
    batch = 4
    per_rank = batch // world
    x_full = np.random.default_rng(1000).integers(0, 256, (batch, 32, 32, 3), dtype=np.int64).astype(np.uint8)
    x = np.ascontiguousarray(x_full[rank * per_rank:(rank + 1) * per_rank])
    y = mobilenet_ref.run_oracle(layers, x)                 # CPU stand-in for the per-rank device graph
    t = torch.tensor([1.0 + rank, 2.0 + 0.5 * rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)                # timing rule: max over ranks
    gathered = [torch.zeros(per_rank, 10, dtype=torch.uint8) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.from_numpy(y.copy()), gathered, dst=0)   # only the final logits travel
    if rank == 0:
        whole = mobilenet_ref.run_oracle(layers, x_full)
        print(json.dumps({"max_ms": t.tolist(), "units": batch, "rows": int(torch.cat(gathered).shape[0]),
                          "equal": bool(np.array_equal(torch.cat(gathered).numpy(), whole)),
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
    assert out["units"] == 4 and out["rows"] == 4 and out["distinct"] and out["equal"]


def test_reference_arm_runs_on_rank0_only():
    """bench.py --impl reference: rank 0 prints the line, other ranks exit 0 without work."""
    root = os.path.dirname(HERE)
    env = {**os.environ, "RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                       capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""
