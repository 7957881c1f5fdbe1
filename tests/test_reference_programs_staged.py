"""The reference project's own acceptance drivers and benchmark harness, unmodified, against this
package on CPU ranks - and this repository's own GPU test files over the same stage.

oracle/build_ref.py stages byte-identical copies of those programs under oracle/_ref/ (a git-ignored
build output); tests/cuda_stage.py runs a program written for CUDA devices in processes without a GPU
(devices rewritten to the CPU, torch.cuda stand-ins, an emulation of CUDA-graph capture and replay)
with libfga.so replaced by tests/abi_simulator.py. What passes here is everything those programs demand
of the host layer: names and signatures, error messages, frozen configuration, cached views, "no
allocation, synchronization or group barrier after set-up", ownership of returned tensors, the
main_grad protocol, saved-tensor hooks, micro-batches of different lengths with delayed backward,
pipeline-parallel set-up order, and correct values after graph replays with changed inputs - checked
by the reference's own independent FP32 computations. It says nothing about the CUDA kernels;
tests/test_zu_reference_drivers.py runs the same programs on GPUs.

All programs are started together (they are independent processes with two threads each) - by
tests/conftest.py when the long simulated-rank tests of the suite begin, else when the first test here
asks for one - so the file costs about as long as its slowest program, or nothing. FGA_STAGED=all adds the
long ones (minutes each on eight cores).
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, 'oracle', '_ref')
STAGE = os.path.join(ROOT, 'tests', 'cuda_stage.py')
pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(STAGED, 'benchmark', 'run.py')),
                                reason='oracle/_ref/ has not been built (no reference tree at build time)')

HARNESS = ('--tokens', '512', '--hidden-size', '1024', '--heads', '8', '--iterations', '2', '--trials', '1',
           '--warmup', '1', '--graph-batch', '2', '--layers', '2', '--cuda-graphs', '--validation-rounds', '2')
BENCH = ('--steps', '2', '--warmup', '1', '--tokens', '512', '--hidden', '1024', '--heads', '8', '--min-seconds', '0.2',
         '--cpu-sample-tokens', '256')
# name: (ranks, stage flags, program, arguments, line the program prints on success, runs by default)
PROGRAMS = {
    'harness_bf16_cp2': (2, (), 'benchmark/run.py', ('--cp', '2', *HARNESS, '--bias', '--bias-in-gemm', '--gate'),
                         'Validation passed', True),
    'harness_mxfp8_cp1': (1, (), 'benchmark/run.py',
                          ('--cp', '1', '--tokens', '256', '--hidden-size', '512', '--heads', '4', '--iterations', '1',
                           '--trials', '1', '--warmup', '1', '--graph-batch', '1', '--layers', '2', '--cuda-graphs',
                           '--validation-rounds', '1', '--precision', 'mxfp8'), 'Validation passed', True),
    'pipeline_setup': (4, (), 'tests/pipeline_setup_driver.py', ('--prepare',), 'PIPELINE_SETUP_PASS', True),
    'attention_training': (1, ('--stand-in-attention',), 'tests/attention_training_driver.py', ('--tokens', '256'),
                           'checks passed with owned QKV outputs', True),
    'recv_padding': (1, (), 'tests/recv_padding_driver.py', (), 'PASS receive padding: segments=4', True),
    'mxfp8_modules': (1, (), 'tests/mxfp8_driver.py', ('--heads', '2', '--lengths', '33'), 'MXFP8_PASS', True),
    'mxfp8_local': (1, (), 'tests/mxfp8_local_driver.py', (), 'MXFP8_LOCAL_PASS', True),
    # This repository's own GPU test files (their host logic: shapes, call sequences, expectations against
    # the oracle) over the same stage, so that no GPU test meets a GPU with its own code unrun. Left out:
    # what only the real library can answer (argument validation, bounded device waits, the static
    # scratch array) and the files that start GPU processes of their own.
    'own_gpu_tests': (1, (), '-m', ('pytest', '-q', '-m', 'gpu', '-p', 'no:cacheprovider', 'tests/test_emulated_ranks.py',
                                   'tests/test_fused_modules.py', 'tests/test_gemm_local.py', 'tests/test_mxfp8_gemm.py',
                                   'tests/test_mxfp8_modules.py', 'tests/test_yb_grouped_query.py',
                                   'tests/test_zx_two_layer_training.py', 'tests/test_zy_opt_in_paths.py',
                                   'tests/test_aux_kernels.py', '-k',
                                   'not test_argument_validation and not test_argument_errors_are_reported '
                                   'and not rejects_bad_arguments'), ' passed', True),
    # bench.py's GPU code path itself (CUDA events, graphs, copy streams, the parity gate, the instrumented
    # steps, the JSON line) rather than its --device cpu harness mode.
    'bench_fused': (1, (), 'bench.py', BENCH, '"roofline"', True),
    'bench_unfused_cp2': (2, (), 'bench.py', (*BENCH, '--gpus', '2', '--impl', 'nccl', '--no-e2e'), '"parity_check"', True),
    'bench_mxfp8': (1, (), 'bench.py', ('--steps', '1', '--warmup', '1', '--tokens', '256', '--hidden', '512', '--heads', '4',
                                        '--min-seconds', '0.05', '--precision', 'mxfp8', '--no-e2e', '--no-cpu-baseline'),
                    '"roofline"', True),
    'variable_length': (1, ('--cpu-is-elsewhere',), 'tests/variable_length_driver.py',
                        ('--local-tokens', '130', '1', '257'), 'Variable-length projections', False),
    'variable_length_cp2': (2, ('--cpu-is-elsewhere',), 'tests/variable_length_driver.py',
                            ('--local-tokens', '130', '1'), 'Variable-length projections', False),
    'attention_training_cp2': (2, ('--stand-in-attention',), 'tests/attention_training_driver.py',
                               ('--tokens', '256'), 'checks passed with owned QKV outputs', False),
    'harness_bf16_cp4': (4, (), 'benchmark/run.py', ('--cp', '4', *HARNESS), 'Validation passed', False),
}
NEEDS_OUTPUT = {'benchmark/run.py', 'tests/attention_training_driver.py', 'tests/recv_padding_driver.py',
                'tests/mxfp8_driver.py', 'tests/mxfp8_local_driver.py', 'tests/variable_length_driver.py'}


def selected():
    everything = os.environ.get('FGA_STAGED', '') == 'all'
    return [name for name, spec in PROGRAMS.items() if spec[-1] or everything]


STARTED = {}      # name -> (process, path of its output file); filled once per session


def start_all():
    """Every selected program as a process tree of its own, all started now (output to files, so that
    nobody has to read a pipe while they run). tests/conftest.py calls this early, when the long
    simulated-rank tests begin, so that the programs run beside those instead of after them."""
    import tempfile
    if STARTED or not os.path.exists(os.path.join(STAGED, 'benchmark', 'run.py')):
        return STARTED
    scratch = tempfile.mkdtemp(prefix='fga-staged-')
    env = dict(os.environ, FGA_STAGE_THREADS='2')
    # The pipeline driver gives its process group 75 s per collective: it runs first, alone (seconds), so
    # that a loaded machine cannot push it over that limit; everything else then starts together.
    order = sorted(selected(), key=lambda name: name != 'pipeline_setup')
    for index, name in enumerate(order):
        ranks, flags, program, arguments, _, _ = PROGRAMS[name]
        command = [sys.executable, STAGE, '--ranks', str(ranks), '--port', str(29700 + index), *flags,
                   program if program == '-m' else os.path.join(ROOT if program == 'bench.py' else STAGED, program),
                   *arguments]
        if program in NEEDS_OUTPUT:
            command += ['--output', os.path.join(scratch, f'{name}.json')]
        log = os.path.join(scratch, f'{name}.log')
        with open(log, 'w') as sink:
            STARTED[name] = (subprocess.Popen(command, env=env, cwd=ROOT, stdout=sink, stderr=subprocess.STDOUT), log)
        if name == 'pipeline_setup':
            STARTED[name][0].wait(timeout=600)
    return STARTED


def stop_all():
    for process, _ in STARTED.values():
        if process.poll() is None:
            process.kill()
            process.wait()


@pytest.fixture(scope='module')
def running():
    yield start_all()
    stop_all()


@pytest.mark.parametrize('name', selected())
def test_reference_program_passes_on_the_cpu_stage(running, name):
    process, log = running[name]
    try:
        process.wait(timeout=3000)
    except subprocess.TimeoutExpired:
        process.kill()
        process.wait()
        with open(log) as text:
            pytest.fail(f'{name}: no end after 3000 s\n{text.read()[-3000:]}')
    with open(log) as text:
        output = text.read()
    assert process.returncode == 0, f'{name} exited {process.returncode}\n{output[-4000:]}'
    assert PROGRAMS[name][4] in output, output[-2000:]
    assert ' failed' not in output.splitlines()[-1], output[-2000:]
    if PROGRAMS[name][2] == 'bench.py':
        import json
        line = json.loads([text for text in output.splitlines() if text.startswith('{')][-1])
        assert line['parity_check']['passed'] and line['value'] > 0
        assert (line['gpu_launches'] > 0) == (line['impl'] == 'fused')   # only this repository's kernels count
        assert 'graph' in line['config']['launch'] and 'failed' not in line['config']['launch'], line['config']['launch']
        if name == 'bench_fused':
            assert line['e2e']['h2d_bytes_per_step'] > 0 and line['e2e']['d2h_bytes_per_step'] > 0
            assert line['cpu_baseline']['kind'] == 'reference' and line['roofline']['launches_timed'] > 0


def test_a_staged_program_notices_a_host_layer_without_ownership_copies(tmp_path):
    """Negative control: with results handed out as views of the shared head-side buffers
    (FGA_STAGE_SABOTAGE=shared-output breaks the package that way inside the stage), the reference's
    training driver must fail on its own ownership assertion - the staged programs are not passing by
    default."""
    result = subprocess.run(
        [sys.executable, STAGE, '--port', '29760', '--stand-in-attention',
         os.path.join(STAGED, 'tests', 'attention_training_driver.py'), '--tokens', '256',
         '--output', str(tmp_path / 'sabotaged.json')],
        env=dict(os.environ, FGA_STAGE_SABOTAGE='shared-output', FGA_STAGE_THREADS='2'), cwd=ROOT,
        capture_output=True, text=True, timeout=900)
    assert result.returncode != 0
    assert 'untyped_storage().data_ptr() != buffer.untyped_storage().data_ptr()' in result.stderr + result.stdout
