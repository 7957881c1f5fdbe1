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
    assert line['cpu_baseline']['kind'] == 'port' and line['cpu_baseline']['cores'] >= 1
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
