"""Expert parallel on real GPUs (needs at least two; skipped, and said so, on one)."""

from __future__ import annotations

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_on_gpus_matches_oracle(world: int) -> None:
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this box has {torch.cuda.device_count()}")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(REPO / "tests" / "ep_multi_gpu_check.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env, cwd=REPO)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert done.stdout.count("EP_CHECK_OK") == world, done.stdout[-2000:]


@pytest.mark.parametrize("world,config", [(2, "wide_e16"), (4, "mixtral")])
def test_benchmark_shapes_on_gpus_match_oracle(world: int, config: str) -> None:
    """The benchmark's own parity check (both token layouts, both transports, routing tensors
    bit-exact, every rank's rows) at benchmark shapes: the wide Zipf layer with raw +/- routing
    weights (16 experts) on two GPUs, the Mixtral-shaped sweep's ends on four."""

    import json

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this box has {torch.cuda.device_count()}")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(REPO / "bench.py"), "--gpus", str(world),
           "--config", config, "--parity-only"]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=REPO)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    line = [l for l in done.stdout.splitlines() if l.startswith("{")][-1]
    parity = json.loads(line)["parity"]
    assert parity["status"] == 0 and parity["routing_bit_exact"], parity
    assert parity["replicated_err_over_rms"] <= 2e-2 and parity["sharded_err_over_rms"] <= 2e-2
