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


def pytest_collection_finish(session):
    session.config._fga_staged = any(
        item.fspath.basename == 'test_reference_programs_staged.py' and 'passes_on_the_cpu_stage' in item.name
        for item in session.items)


def pytest_runtest_setup(item):
    # The staged reference programs (minutes of CPU work in processes of their own) start when the long
    # simulated-rank tests begin and run beside them; their own test file then only collects results.
    if getattr(item.config, '_fga_staged', False) and item.fspath.basename == 'test_host_simulated_ranks.py':
        item.config._fga_staged = False
        import importlib
        importlib.import_module('tests.test_reference_programs_staged').start_all()   # the name pytest imports it by


def pytest_sessionfinish(session, exitstatus):
    staged = sys.modules.get('tests.test_reference_programs_staged')
    if staged is not None:
        staged.stop_all()


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
