"""Multi-GPU checks; skipped unless at least two GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
def test_tensor_parallel_two_gpus():
    # plain peer loads / stores everywhere: no multicast binding of the symmetric buffers
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    n = os.environ.get("B200_TEST_TP", "2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", n,
           "--master-addr", "127.0.0.1", "--master-port", "29611",
           os.path.join(ROOT, "tests", "_tp_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "engine ok" in res.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
def test_gemm_allreduce_norm_over_multimem_two_gpus():
    """The fused GEMM + all-reduce + norm kernel again, this time with the multicast view of
    the symmetric buffers when the allocation has one (in-switch reduction and broadcast)."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TEST_ONLY="ar_norm")
    n = os.environ.get("B200_TEST_TP", "2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", n,
           "--master-addr", "127.0.0.1", "--master-port", "29615",
           os.path.join(ROOT, "tests", "_tp_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "gemm + all-reduce + norm ok" in res.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
def test_pipeline_parallel_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TEST_ONLY="pp")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29617",
           os.path.join(ROOT, "tests", "_tp_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "pp2 engine ok" in res.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
def test_expert_parallel_fused_dispatch_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    n = min(torch.cuda.device_count(), 8)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
           "--master-addr", "127.0.0.1", "--master-port", "29613",
           os.path.join(ROOT, "tests", "_ep_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "fused dispatch/combine ok" in res.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs >= 2 GPUs")
def test_etp_gather_scatter_two_gpus():
    """Data-parallel attention without expert parallelism: experts sharded over the replicas,
    rows gathered and sums scattered back over NCCL."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_EP_MODE="etp")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29619",
           os.path.join(ROOT, "tests", "_ep_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "gather/scatter ok" in res.stdout
