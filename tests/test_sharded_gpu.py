"""GPU tier, needs at least two devices: the column-sharded block-scale GEMM under torchrun / NCCL.
The worker (tests/sharded_gpu_worker.py) checks, on every rank and bit for bit against the single-GPU
GEMM of the whole problem: the local shard, the blocked all-gather, the assembled all-gather, the
all-gather fused into the GEMM's epilogue (peer stores), and an uneven column split."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two CUDA devices")
def test_sharded_gemm_and_gathers_match_the_single_gpu_result(tmp_path):
    world = 2
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", HKB_TEST_OUT=str(tmp_path))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port),
                        os.path.join(ROOT, "tests", "sharded_gpu_worker.py")],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    lines = [json.load(open(tmp_path / f"rank{k}.json")) for k in range(world)]
    for ln in lines:
        for key in ("shard_equals_full_slice", "blocked_gather_ok", "assembled_gather_ok", "fused_gather_ok", "uneven_split_ok"):
            assert ln[key], ln
        assert "scatter" in ln["fused_gather_kernel"]
