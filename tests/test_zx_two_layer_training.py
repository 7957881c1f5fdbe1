"""Two layers x two micro-batches through the public modules with attention in between: the
lifetime of projection outputs and saved activations across reuses of the shared workspace, eager
and under CUDA-graph replay with changed inputs (tests/drivers/two_layer_training.py).

Sorted late on purpose: it is the widest end-to-end case and depends on everything before it.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, 'tests', 'drivers'))


def test_two_layers_two_microbatches_on_one_gpu(cp1):
    import two_layer_training
    failures, errors = two_layer_training.run(torch.device('cuda', 0))
    assert not failures, failures
    assert len(errors) == 8 * 4          # eager, saved-tensor hooks, two graph replays: eight tensors each


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs at least two GPUs')
def test_two_layers_two_microbatches_across_gpus(native):
    world = min(8, 1 << (torch.cuda.device_count().bit_length() - 1))
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', FGA_TIMEOUT_S='10')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={world}',
           '--master-addr', '127.0.0.1', '--master-port', '29579',
           os.path.join(ROOT, 'tests', 'drivers', 'two_layer_training.py')]
    result = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(result.stdout[-4000:])
    sys.stderr.write(result.stderr[-4000:])
    assert result.returncode == 0
    assert 'PASS two layers' in result.stdout
