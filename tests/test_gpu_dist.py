"""Tensor parallelism on real GPUs: spawns the multi-rank self-test under torchrun (needs >= 2 GPUs)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_selftest_two_ranks():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", "-m", "hipengine_b200.parallel.selftest"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("{")][-1]
    rep = json.loads(line)
    assert rep["ok"] and rep["fused_sum_ok"] and rep["graph_decode_ranks_agree"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_expert_parallel_selftest_two_ranks():
    """MoE with the experts dealt out over two ranks (attention / delta-net tensor-parallel, experts parallel)."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29534", "-m", "hipengine_b200.parallel.selftest",
           "--model", "tiny-hybrid-moe-tp", "--prompt", "100"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    rep = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])
    assert rep["ok"] and rep["graph_decode_ranks_agree"]
