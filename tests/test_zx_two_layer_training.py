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

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, 'tests', 'drivers'))


@pytest.mark.gpu
def test_two_layers_two_microbatches_on_one_gpu(cp1):
    import two_layer_training
    failures, errors = two_layer_training.run(torch.device('cuda', 0))
    assert not failures, failures
    assert len(errors) == 8 * 4          # eager, saved-tensor hooks, two graph replays: eight tensors each


@pytest.mark.gpu
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


def _simulated_worker(rank, world, port, queue):
    import torch.distributed as dist
    tests = os.path.join(ROOT, 'tests')
    for path in (tests, os.path.join(tests, 'drivers'), ROOT, os.path.join(ROOT, 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.set_num_threads(2)
    import abi_simulator
    import fused_gemm_a2a as fused
    import two_layer_training
    _, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    try:
        failures, errors = two_layer_training.run(torch.device('cpu'), hidden=512, heads=4, total_tokens=256, replays=0)
        queue.put((rank, failures, len(errors)))
    finally:
        undo()
    dist.destroy_process_group()


@pytest.mark.parametrize('world', [1, 2])
def test_two_layer_driver_logic_on_simulated_ranks(world):
    """The driver itself (two layers, two micro-batches, attention in between, reversed backwards, the
    saved-tensor-hook pass, the dense FP32 reference) on CPU ranks over the simulated library; the
    CUDA-graph replays need a GPU and are left out."""
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=_simulated_worker, args=(r, world, 29580 + world, queue)) for r in range(world)]
    for proc in procs:
        proc.start()
    try:
        results = sorted(queue.get(timeout=600) for _ in range(world))
    finally:
        for proc in procs:
            proc.join(timeout=60)
            if proc.is_alive():
                proc.terminate()
    for rank, failures, checks in results:
        assert not failures, f'rank {rank}: {failures}'
        assert checks == 8 * 2          # eager and saved-tensor hooks: eight tensors each
