"""Fused compute+collective kernels against the torch.distributed path and the parallel layouts of the trainer, on 2 or
more GPUs (skipped on a 1-GPU box)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason='needs 2 GPUs')
def test_fused_tp_kernels_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr',
           '127.0.0.1', '--master-port', '29533', os.path.join(HERE, 'multi_gpu_fused_worker.py')]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert 'ALL OK' in res.stdout


@pytest.mark.skipif(_ngpu() < 8, reason='needs 8 GPUs')
def test_fused_tp_kernels_eight_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '8', '--master-addr',
           '127.0.0.1', '--master-port', '29536', os.path.join(HERE, 'multi_gpu_fused_worker.py')]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert 'ALL OK' in res.stdout


@pytest.mark.skipif(_ngpu() < 2, reason='needs 2 GPUs')
def test_fused_moe_expert_parallel_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr',
           '127.0.0.1', '--master-port', '29534', os.path.join(HERE, 'moe_fused_worker.py')]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert 'ALL OK' in res.stdout


@pytest.mark.skipif(_ngpu() < 2, reason='needs 2 GPUs')
def test_peer_memory_dp_collectives_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr',
           '127.0.0.1', '--master-port', '29535', os.path.join(HERE, 'dp_comm_worker.py')]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert 'ALL OK' in res.stdout, res.stdout[-3000:]


@pytest.mark.skipif(_ngpu() < 2, reason='needs 2 GPUs')
def test_parallel_layouts_train_like_data_parallel_on_gpus():
    """TP2 (+SP), PP2 (1F1B over NCCL send / recv), CP2 (ring attention with the peer-memory K/V exchange) and EP2 (fused
    MoE exchange) train a tiny model on two real GPUs to the same losses as plain data parallelism.  (Launched with four
    ranks the worker adds TP2 x PP2, TP2 x CP2 and TP2 x EP2.)"""
    n = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', str(n), '--master-addr',
           '127.0.0.1', '--master-port', '29541', os.path.join(HERE, 'gpu_layouts_worker.py')]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert 'ALL OK' in res.stdout, res.stdout[-3000:]


def test_fused_moe_single_gpu():
    res = subprocess.run([sys.executable, os.path.join(HERE, 'moe_fused_worker.py')], capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert 'ALL OK' in res.stdout
