"""What can be checked of bench.py without a GPU: the algorithmic FLOP count, the clock-sample
parser, and the CPU arm (`--impl reference`), whose single JSON line must carry the keys the
benchmark contract names."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_algorithmic_flops_match_the_published_work_table():
    """131072 tokens, H=4096: QKV forward 13194.1 GFLOP and output forward 4398.0 GFLOP on one rank,
    an eighth of that per rank at CP=8; backward is twice forward (dgrad + wgrad)."""
    import bench
    one = bench.flops_per_step(131072, 4096, 3)
    assert round(one['qkv_fwd'] / 1e9, 1) == 13194.1 and round(one['out_fwd'] / 1e9, 1) == 4398.0
    assert one['qkv_bwd'] == 2 * one['qkv_fwd'] and one['out_bwd'] == 2 * one['out_fwd']
    assert one['total'] == 24.0 * 131072 * 4096 ** 2
    eighth = bench.flops_per_step(16384, 4096, 3)
    assert round(eighth['qkv_fwd'] / 1e9, 1) == 1649.3 and round(eighth['out_fwd'] / 1e9, 1) == 549.8
    gated = bench.flops_per_step(8191, 3072, 4)
    assert round(gated['qkv_fwd'] / 1e9, 1) == 618.4 and round(gated['out_fwd'] / 1e9, 1) == 154.6


def test_clock_samples_are_summarised_over_the_timed_window_only():
    import bench
    sampler = bench.ClockSampler(0)
    sampler.lines = [
        '1965, 1965, 150.00, Not Active, Not Active, Not Active, Not Active, 1000.00',    # warm-up, dropped
        '1095, 1965, 792.18, Not Active, Not Active, Not Active, Active, 1000.00',
        '1110, 1965, 801.00, Not Active, Not Active, Not Active, Active, 1000.00',
        '1305, 1965, 640.00, Not Active, Not Active, Not Active, Not Active, 1000.00',
        'unparsable',
        '1200, 1965, 900.00, Active, Not Active, Not Active, Not Active, 1000.00',         # after the region
    ]
    sampler.first, sampler.last = 1, 5
    summary = sampler.summary()
    assert summary == dict(sm_mhz=1110.0, sm_max_mhz=1965.0, power_w_max=801.0, power_limit_w=1000.0,
                           reasons=['sw_power_cap'], samples=3)
    sampler.first, sampler.last = 5, 6
    assert sampler.summary()['reasons'] == ['hw_slowdown']
    sampler.lines, sampler.first, sampler.last = [], 0, 0
    assert sampler.summary()['samples'] == 0 and sampler.summary()['sm_mhz'] is None


def test_dram_traffic_constants_come_from_the_committed_profiles():
    """The bytes-per-FLOP figures used for roofline.traffic are the two ncu captures' totals."""
    import bench
    for name, key in (('ulysses_gemm_kernel_bf16_forward_8192x12288x4096.md', 'gemm'),
                      ('ulysses_gemm_kernel_bf16_wgrad_12288x4096_k8192.md', 'wgrad')):
        with open(os.path.join(ROOT, 'profiles', name)) as f:
            text = f.read()
        megabytes = bench.DRAM_BYTES_PER_FLOP[key] * 824.6e9 / 1e6
        assert f'{megabytes:.1f} MB per launch' in text


@pytest.mark.timeout(600)
def test_cpu_arm_prints_one_contract_line():
    run = subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference', '--steps', '1',
                          '--warmup', '0', '--cpu-sample-tokens', '256'],
                         capture_output=True, text=True, timeout=580, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [line for line in run.stdout.splitlines() if line.startswith('{')]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ('metric', 'value', 'unit', 'n_gpus', 'steps', 'warmup', 'ms_per_step', 'higher_is_better',
                'scaling', 'vs_baseline', 'dtype', 'data', 'config', 'impl', 'cpu_baseline', 'e2e'):
        assert key in line, key
    assert line['impl'] == 'reference' and line['data'] == 'synthetic' and line['vs_baseline'] is None
    # the reference's own modules when the build step has staged them, else the oracle's restatement
    staged = os.path.exists(os.path.join(ROOT, 'oracle', '_ref', 'benchmark', 'reference.py'))
    assert line['cpu_baseline']['kind'] == ('reference' if staged else 'port') and line['cpu_baseline']['cores'] >= 1
    assert line['cpu_baseline']['value'] == line['value'] == line['e2e']['value'] > 0
    assert line['e2e']['h2d_bytes_per_step'] == 0 and line['e2e']['d2h_bytes_per_step'] == 0
    assert 'workload' in line['config']


def test_provenance_names_versions_tunables_and_digests(monkeypatch):
    import torch

    import bench
    monkeypatch.setenv('FGA_PUSHER_WARPS', '4')
    info = bench.provenance(torch)
    assert info['tunables'] == {k: v for k, v in os.environ.items() if k.startswith(('FGA_', 'FUSED_'))}
    assert info['tunables']['FGA_PUSHER_WARPS'] == '4'
    assert info['torch'] == torch.__version__
    for key in ('libfga_sha256', 'csrc_sha256', 'host_layer_sha256'):
        assert info[key] is None or len(info[key]) == 16
    assert info['csrc_sha256'] is not None and info['host_layer_sha256'] is not None


def test_timed_region_is_a_whole_number_of_requested_runs_and_long_enough():
    import bench
    assert bench.timed_steps(20, 52.0, 2.0) == 40          # one GPU: 20 steps of 52 ms are 1.04 s -> twice
    assert bench.timed_steps(20, 6.0, 2.0) == 340          # eight GPUs: 17 x 20 steps of 6 ms = 2.04 s
    assert bench.timed_steps(10, 500.0, 2.0) == 10         # already long enough
    assert bench.timed_steps(10, 0.0, 2.0) == 10 and bench.timed_steps(0, 5.0, 2.0) % 1 == 0
    assert bench.timed_steps(3, 1e-4, 2.0) == 3000         # capped at 1000 repeats


def test_link_bytes_follow_the_all_to_all_payload_formula():
    """A2A payload per rank per pass M*N_out*2 B*(P-1)/P: 352.3 MB (QKV) and 117.4 MB (output) at CP = 8."""
    import bench
    per_step = bench.link_bytes_per_step(16384, 4096, 3, 8)
    assert round(per_step / 1e6, 1) == round(2 * (352.3 + 117.4), 1) or abs(per_step / 1e6 - 2 * (352.3 + 117.4)) < 0.2
    assert bench.link_bytes_per_step(131072, 4096, 3, 1) == 0


@pytest.mark.timeout(600)
@pytest.mark.parametrize('extra', [[], ['--gate', '--bias', '--no-graphs']])
def test_harness_control_flow_on_two_cpu_ranks(extra):
    """`--device cpu` runs everything around the kernels - warm-up, the parity gate, the sized timed
    region, the end-to-end leg with its copies in both directions, the collective exit - on gloo ranks
    with the unfused arm, so that a run on GPUs does not meet that code for the first time."""
    port = 29790 + len(extra)
    run = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2',
                          '--master-addr', '127.0.0.1', '--master-port', str(port), os.path.join(ROOT, 'bench.py'),
                          '--gpus', '2', '--impl', 'nccl', '--device', 'cpu', '--tokens', '1024', '--hidden', '512',
                          '--heads', '4', '--steps', '3', '--warmup', '1', '--min-seconds', '0.2', *extra],
                         capture_output=True, text=True, timeout=580, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-3000:]
    lines = [line for line in run.stdout.splitlines() if line.startswith('{')]
    assert len(lines) == 1, run.stdout[-2000:]
    line = json.loads(lines[0])
    assert line['n_gpus'] == 2 and line['impl'] == 'nccl' and line['warmup'] == 3
    assert line['steps'] % 3 == 0 and line['steps'] >= 3 and line['steps_requested'] == 3
    assert line['ms_per_step'] * line['steps'] >= 200 * 0.5          # the region was sized from the probe steps
    parity = line['parity_check']
    segments = 4 if '--gate' in extra else 3
    assert parity['passed'] is True and len(parity['checked']) == segments + 1 + 2 * segments + 1 + 1 + 2
    assert parity['worst_relative_frobenius'] <= parity['tolerance']['relative_frobenius']
    m, h = 512, 512
    inputs_bytes = 4 * (m * h * 2 + (segments + 1) * m * h)          # FP32 on the host stand-in: x, dy, grads, o
    results_bytes = 4 * (3 * m * h + segments * h * h + h * h)       # y, dx, dO, dW_qkv, dW_o
    assert line['e2e']['h2d_bytes_per_step'] == inputs_bytes and line['e2e']['d2h_bytes_per_step'] == results_bytes
    assert line['e2e']['value'] > 0 and line['e2e']['steps'] == 3
    assert set(line['passes']) == {'qkv_fwd', 'qkv_bwd', 'out_fwd', 'out_bwd'}
    assert 'samples' in line['clocks'] and 'roofline' not in line    # the kernel roofline belongs to the fused arm


@pytest.mark.timeout(300)
def test_end_to_end_leg_is_skipped_not_fatal_when_its_buffers_cannot_be_pinned():
    """A host that cannot pin the staging buffers of the end-to-end leg still gets its line: the leg
    reports why it is missing, everything else is measured."""
    script = (
        'import sys, bench\n'
        'def refuse(tensor):\n'
        '    raise RuntimeError("CUDA error: out of memory (pinning refused by the test)")\n'
        'bench.HostApi.pin = staticmethod(refuse)\n'
        'sys.argv = ["bench.py", "--impl", "nccl", "--device", "cpu", "--tokens", "512", "--hidden", "512", "--heads", "4",\n'
        '            "--steps", "2", "--warmup", "1", "--min-seconds", "0.1", "--no-cpu-baseline"]\n'
        'bench.guarded_main()\n')
    run = subprocess.run([sys.executable, '-c', script], capture_output=True, text=True, timeout=280, cwd=ROOT,
                         env=dict(os.environ, MASTER_ADDR='127.0.0.1', MASTER_PORT='29796'))
    assert run.returncode == 0, run.stderr[-3000:]
    line = json.loads([text for text in run.stdout.splitlines() if text.startswith('{')][-1])
    assert line['value'] > 0 and line['parity_check']['passed']
    assert line['e2e']['value'] is None and 'pinning refused' in line['e2e']['unavailable']
    assert line['e2e']['h2d_bytes_per_step'] > 0 and line['e2e']['d2h_bytes_per_step'] > 0


def test_kernel_roofline_from_instrumented_steps():
    """The per-launch bookkeeping of the fused arm with stand-ins for the host layer: ten eager steps
    are instrumented, the first two are dropped, GEMM launches carry algorithmic FLOPs (pad rows not
    counted), everything else is summed as non-GEMM time."""
    import types

    import bench
    import torch
    api = bench.HostApi(torch, 0)
    m, hidden = 300, 512
    calls = []

    class Comm:
        def gemm(self, mode, a, b, b_is_kn, c, aux, counters, num_in, n_segment, num_segments, **kw):
            calls.append(mode)

        def barrier(self, *a, **kw):
            calls.append('barrier')

    fused = types.SimpleNamespace(
        bf16_wgrad=lambda dy, x, out, status, accumulate=False: calls.append('wgrad'),
        mxfp8_wgrad=lambda *a, **kw: None, mxfp8_quantize=lambda *a, **kw: None,
        resize_rank_rows=lambda *a, **kw: calls.append('copy'), reduce_bias_grad=lambda *a, **kw: None)
    ws = types.SimpleNamespace(comm=Comm())
    x, recv = torch.zeros(m, hidden), torch.zeros(512, 3 * hidden)
    out = torch.zeros(512, hidden)

    def eager_step():
        ws.comm.barrier()
        ws.comm.gemm('push', x, None, False, None, None, None, 0, hidden, 3, a_rows=512)
        ws.comm.barrier()
        fused.resize_rank_rows()
        ws.comm.barrier(bump=True)
        ws.comm.gemm('recv', recv, None, True, out, None, None, 3, 0, 1)
        fused.bf16_wgrad(recv[:m], x, None, None)

    original = ws.comm.gemm
    instrumented = bench.queue_instrumented_steps(api, fused, ws, eager_step, m, extra=10)
    assert ws.comm.gemm == original and calls.count('push') == 10      # wrappers are gone again
    assert len(instrumented['records']) == 30 and len(instrumented['others']) == 40
    args = bench.parse_args(['--precision', 'bf16'])
    roofline = bench.kernel_roofline(args, instrumented, lambda values: values, m, hidden, 3, 8, 1.0,
                                     bench.flops_per_step(m, hidden, 3))
    assert roofline['launches_timed'] == 24 and roofline['bound'] == 'tensor' and roofline['unit'] == 'TFLOP/s'
    per_step = 3 * 2.0 * m * hidden * 3 * hidden                      # push, recv and wgrad: 2*M*K*N each
    total_ms = roofline['avg_launch_ms'] * 24
    assert abs(roofline['achieved'] - 8 * per_step / (total_ms * 1e-3) / 1e12) <= 1e-6 * roofline['achieved']
    assert roofline['frac'] == roofline['achieved'] / roofline['peak']
    assert roofline['traffic'] > 0 and 'scaled' in roofline['traffic_source']
    assert [entry['op'].split('[')[0] for entry in roofline['launches_rank0_last_step']] == [
        'gemm_push', 'gemm_recv', 'gemm_wgrad', 'barrier', 'barrier', 'copy_rank_rows', 'barrier']
