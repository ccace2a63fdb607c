"""Multi-process tests: a world_size-2 gloo run on CPU (host-side sharding logic) and, on a
box with >= 2 GPUs, the real expert-parallel layer with one process per GPU."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(n, mode, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "mp_worker.py"), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def test_gloo_world_of_two():
    p = _torchrun(2, "gloo")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    assert p.stdout.count("MP_OK") == 2


def test_reference_arm_runs_on_rank0_only():
    """`bench.py --impl reference` under torchrun: rank 0 prints the line, the other rank exits 0."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    import json
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port")


@pytest.mark.gpu
def test_two_gpu_expert_parallel_layer():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    # a rank may die between steps in failure tests only; here plain peer loads, no NVLS needed
    p = _torchrun(2, "gpu", {"NCCL_NVLS_ENABLE": "0"})
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-5000:]
    assert p.stdout.count("MP_OK") == 2
