"""K-split over 2 GPUs with the reduce-scatter's exchange fused into the GEMM's epilogue stores (peer memory).
Needs two GPUs on the box; with one it is skipped (the single-GPU scatter test in test_ksplit_gpu.py and the gloo
tests of the sharding arithmetic still run)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> str:
    """A rendezvous port nobody holds right now (the machine is shared; a fixed port can be taken)."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def test_fused_exchange_two_gpus():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU path to fall back to")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), os.path.join(HERE, "helpers", "ksplit_fused_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    assert res["world"] == 2
    for rank_results in res["ranks"]:
        for it in rank_results:
            assert it["status"] == 0 and it["bit_equal"] and it["err"] <= 1e-2, res


def test_nccl_through_the_c_abi_two_gpus():
    """Communicator and reduce-scatter through libtesserae_b200 only (the id travels over gloo)."""
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU path to fall back to")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), os.path.join(HERE, "helpers", "nccl_capi_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    for it in res["ranks"]:
        assert it["exact"] and it["status"] == 0 and it["err"] <= 1e-2, res
