"""Real multi-GPU parity: one process per GPU over NVLink, all the GPUs of the box (2, 4 or 8); and the
same driver on two CPU ranks over the simulated library, so that the driver's own logic has run
before it meets a GPU."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs at least two GPUs')
def test_fused_modules_across_gpus(native):
    world = min(8, 1 << (torch.cuda.device_count().bit_length() - 1))
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', FGA_TIMEOUT_S='10')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={world}',
           '--master-addr', '127.0.0.1', '--master-port', '29577',
           os.path.join(ROOT, 'tests', 'drivers', 'multi_gpu_driver.py')]
    result = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(result.stdout[-4000:])
    sys.stderr.write(result.stderr[-4000:])
    assert result.returncode == 0
    assert 'PASS mxfp8' in result.stdout
    assert 'PASS cuda graph replay' in result.stdout


@pytest.mark.timeout(900)
def test_driver_logic_on_two_simulated_ranks():
    """FGA_DRIVER_SIMULATED=1: gloo ranks, tests/abi_simulator.py in place of libfga.so, every geometry
    of the driver (incl. the benchmark configurations' head counts and the MXFP8 one) at fewer lengths,
    no CUDA-graph section."""
    env = dict(os.environ, FGA_DRIVER_SIMULATED='1', OMP_NUM_THREADS='4')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=2',
           '--master-addr', '127.0.0.1', '--master-port', '29578',
           os.path.join(ROOT, 'tests', 'drivers', 'multi_gpu_driver.py')]
    result = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=880)
    sys.stdout.write(result.stdout[-3000:])
    sys.stderr.write(result.stderr[-3000:])
    assert result.returncode == 0
    assert result.stdout.count('PASS hidden=') == 5 and 'PASS mxfp8' in result.stdout
    assert 'PASS simulated; 8 eager configurations checked on 2 CPU ranks' in result.stdout
