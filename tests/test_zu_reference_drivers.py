"""The reference project's own benchmark harness and GPU acceptance drivers, unmodified, run against
this package.

oracle/build_ref.py stages byte-identical copies of them under oracle/_ref/ (a git-ignored build
output) together with two forwarding modules, so that their `from fused_gemm_a2a import ...` resolves
to this package. Each driver is a process of its own; it passes when it exits 0 and prints its own
success line. What they check (their docstrings): exact pad / unpad / bias / ownership row copies;
FP32-accurate bias gradients incl. rows beyond 4 GiB and graph replay; bit-exact receive transport
with zero pad rows for eleven logical lengths under graph replay; variable micro-batch lengths with
delayed backward, error messages, no allocation or synchronization after setup; the benchmark's
validation of every stage against FP32 full-token linears before it times anything.

Skipped where oracle/_ref/ was never built (no reference tree at build time). Sorted late: these
are the widest cases and take minutes.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, 'oracle', '_ref')
OUTPUT = os.path.join(ROOT, 'gpurun_out')
needs_staged = pytest.mark.skipif(not os.path.exists(os.path.join(STAGED, 'benchmark', 'run.py')),
                                  reason='oracle/_ref/ has not been built')


def run(script, *arguments, ranks=None, port=29601, timeout=1500):
    """One driver as a process (under torch.distributed.run when it needs a process group)."""
    path = os.path.join(STAGED, script)
    command = [sys.executable, path, *arguments]
    if ranks is not None:
        command = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={ranks}',
                   '--master-addr', '127.0.0.1', '--master-port', str(port), path, *arguments]
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    result = subprocess.run(command, env=env, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    sys.stdout.write(result.stdout[-3000:])
    sys.stderr.write(result.stderr[-3000:])
    assert result.returncode == 0, f'{script} exited {result.returncode}'
    return result.stdout


def all_gpus():
    return min(8, 1 << (max(torch.cuda.device_count(), 1).bit_length() - 1))


@needs_staged
def test_the_harness_imports_every_name_it_needs_from_this_package():
    """No GPU needed: the benchmark driver's module-level imports (MMA_TILER_MN, padded_rows, the three
    public classes, its own baseline) resolve, and the constants it records by name exist."""
    result = subprocess.run([sys.executable, os.path.join(STAGED, 'benchmark', 'run.py'), '--help'],
                            capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert result.returncode == 0, result.stderr[-2000:]
    assert '--validation-rounds' in result.stdout
    import fused_gemm_a2a_kernels as kernels
    for name in ('USE_2CTA', 'MMA_N', 'MMA_N_RECV', 'MMA_N_OUT_PUSH', 'CLUSTER_N', 'RASTER_ALONG_M', 'SWIZZLE',
                 'PUSHER_WARPS', 'PUSH_SPLIT', 'PUSHER_CHUNK', 'PUSHER_STREAMING', 'SWIZZLE_PUSH'):
        assert hasattr(kernels, name), name
    assert all('tcgen05.mma' in k.__ptx__ and 'block_scale' in k.__ptx__ for k in kernels._native_mxfp8_kernels)
    with open(os.path.join(STAGED, 'MANIFEST.json')) as f:
        manifest = json.load(f)
    assert 'fused_gemm_a2a.py' not in manifest['files'] and 'benchmark/reference.py' in manifest['files']


@pytest.mark.gpu
@needs_staged
def test_row_copy_driver(native):
    assert 'exact pad/unpad/bias/ownership checks passed' in run('tests/row_copy_driver.py')


@pytest.mark.gpu
@needs_staged
def test_bias_grad_driver(native):
    assert 'PASS:' in run('tests/bias_grad_driver.py', '--output', os.path.join(OUTPUT, 'reference_bias_grad.json'))


@pytest.mark.gpu
@needs_staged
def test_recv_padding_driver_on_one_gpu(native):
    out = run('tests/recv_padding_driver.py', '--output', os.path.join(OUTPUT, 'reference_recv_padding_cp1.json'),
              ranks=1, port=29602)
    assert out.count('PASS receive padding') == 3


@pytest.mark.gpu
@needs_staged
def test_variable_length_driver_on_one_gpu(native):
    out = run('tests/variable_length_driver.py', '--output', os.path.join(OUTPUT, 'reference_variable_length_cp1.json'),
              ranks=1, port=29603)
    assert 'Variable-length projections' in out


@pytest.mark.gpu
@needs_staged
def test_benchmark_harness_on_one_gpu(native):
    """benchmark/run.py with its lifetime, bias, gate and changed-input graph checks, at a size that
    keeps its full-token FP32 references small; it validates before it times and raises on a mismatch."""
    out = run('benchmark/run.py', '--cp', '1', '--tokens', '8192', '--iterations', '8', '--trials', '2', '--warmup', '2',
              '--graph-batch', '4', '--layers', '2', '--bias', '--bias-in-gemm', '--gate', '--cuda-graphs',
              '--validation-rounds', '3', '--output', os.path.join(OUTPUT, 'reference_run_cp1.json'),
              ranks=1, port=29604)
    assert 'Validation passed' in out


@pytest.mark.gpu
@needs_staged
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs at least two GPUs')
def test_drivers_across_gpus(native):
    world = all_gpus()
    out = run('tests/recv_padding_driver.py', '--output', os.path.join(OUTPUT, f'reference_recv_padding_cp{world}.json'),
              ranks=world, port=29605)
    assert out.count('PASS receive padding') == 3
    out = run('tests/variable_length_driver.py', '--output',
              os.path.join(OUTPUT, f'reference_variable_length_cp{world}.json'), ranks=world, port=29606)
    assert 'Variable-length projections' in out
    out = run('benchmark/run.py', '--cp', str(world), '--tokens', str(8192 * world), '--iterations', '8', '--trials', '2',
              '--warmup', '2', '--graph-batch', '4', '--layers', '2', '--bias', '--bias-in-gemm', '--gate',
              '--cuda-graphs', '--validation-rounds', '3', '--output',
              os.path.join(OUTPUT, f'reference_run_cp{world}.json'), ranks=world, port=29607)
    assert 'Validation passed' in out
