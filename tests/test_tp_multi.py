"""Tensor-parallel decoder on real GPUs against the single-GPU decoder (which is itself checked
against the oracle): spawns one process per GPU with torchrun.  Needs at least 2 GPUs; the shard
arithmetic and the exchange protocol are covered on one GPU and on CPU ranks elsewhere."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_decoder_equals_single_gpu(built_lib, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + world), os.path.join(ROOT, "tests", "tp_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{\"tp_parity\"")]
    assert r.returncode == 0 and lines, r.stdout[-3000:]
    rep = json.loads(lines[-1])
    assert rep["ok"] and rep["world"] == world, rep
