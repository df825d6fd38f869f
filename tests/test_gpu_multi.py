"""Two ranks on two GPUs: sharded GEMM / GEMV / AdamW through the C interface, outputs gathered by NCCL and by the
fused epilogue of e5b_gemm_bcast, compared with the single-GPU result (tests/multi_gpu_worker.py).  Skipped where
fewer than two GPUs are visible; the partitioning arithmetic itself is covered on CPU ranks in
tests/test_sharding_gloo.py."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sharded_outputs_equal_the_single_gpu_result():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_worker.py")],
                         capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0 and "MULTI_GPU_OK" in out.stdout, (out.stdout[-3000:], out.stderr[-3000:])
