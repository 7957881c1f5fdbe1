"""Shared test configuration: import paths, the `gpu` marker and a single-rank process group."""
import os
import sys

import pytest

# Several CPU tests run two to four ranks of torch work on the same cores. OpenMP workers that spin
# while they wait for the next parallel region then steal the cores from the other ranks; let them
# sleep instead. Read when the OpenMP runtime starts, so set before anything imports torch; child
# processes inherit it.
os.environ.setdefault('OMP_WAIT_POLICY', 'PASSIVE')
os.environ.setdefault('GOMP_SPINCOUNT', '0')

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE = os.path.join(ROOT, 'fused-gemm-a2a_b200')
for path in (ROOT, PACKAGE):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a B200 (sm_100a) GPU')


@pytest.fixture(scope='session')
def native():
    """The loaded C-ABI library; building it if the shared object is stale or missing."""
    import build_native
    import _fga_native
    build_native.build()
    return _fga_native.lib()


@pytest.fixture(scope='session')
def cp1(native):
    """A world_size-1 NCCL process group on cuda:0: the fused modules need a CP group."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(0)
    if not dist.is_initialized():
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29533')
        dist.init_process_group('nccl', rank=0, world_size=1, device_id=torch.device('cuda', 0))
    yield dist.group.WORLD
