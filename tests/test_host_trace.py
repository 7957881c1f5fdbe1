"""The host layer's launch plan, checked on the CPU: which C-ABI entry points the workspace and the
autograd functions call, in which order, with which sizes, strides, buffer offsets and peer tables,
for BF16 and MXFP8, QKV and QKVG, bias early / late / none, main_grad accumulation, two token counts
under one capacity, on one rank and on two gloo ranks. The device library is replaced by a recorder
(tests/host_trace.py); the expected traces are tests/golden/host_call_trace_*.json, written by
tests/golden/make_host_trace.py from the host layer whose launches were verified on B200s.
"""
import os
import sys
import tempfile

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, 'golden')
sys.path.insert(0, GOLDEN)


def _first_difference(expected, actual):
    exp, act = expected.splitlines(), actual.splitlines()
    for number, (e, a) in enumerate(zip(exp, act), 1):
        if e != a:
            return f'line {number}:\n  expected {e[:600]}\n  actual   {a[:600]}'
    return f'length differs: expected {len(exp)} lines, got {len(act)}'


@pytest.mark.parametrize('world,configs,port', [(1, (0, 1, 2, 3, 4), 29641), (2, (1, 3), 29642)])
def test_launch_plan_matches_the_recorded_one(world, configs, port):
    import make_host_trace
    with tempfile.TemporaryDirectory() as out_dir:
        make_host_trace.record(world, configs, out_dir, port)
        names = sorted(os.listdir(out_dir))
        assert len(names) == world
        for name in names:
            with open(os.path.join(GOLDEN, name)) as f:
                expected = f.read()
            with open(os.path.join(out_dir, name)) as f:
                actual = f.read()
            assert actual == expected, f'{name}: {_first_difference(expected, actual)}'


def test_trace_has_the_protocol_shape():
    """Independent of the recorded files: a push op is barrier, GEMM, barrier, row copy; a recv op is
    a counter-resetting barrier then the GEMM; weight gradients follow their dgrad."""
    import json
    with open(os.path.join(GOLDEN, 'host_call_trace_p1.json')) as f:
        calls = json.load(f)
    names = [name for name, _ in calls]
    start = names.index('tokens')
    first = names[start + 1:start + 5]
    assert first == ['barrier', 'fga_gemm_push', 'barrier', 'resize_rank_rows']
    recv = names.index('fga_gemm_recv')
    assert names[recv - 1] == 'barrier' and calls[recv - 1][1]['bump'] is True
    assert names[recv + 1] == 'bf16_wgrad'
    push = calls[names.index('fga_gemm_push')][1]
    assert push['a_rows'] == 512 and push['m'] == 300 and push['head_rows'] == 512 and push['segments'] == 3
    # every peer table entry of a single-rank group points into this rank's own slab
    assert all(entry.startswith('symm') for table in push['peer_heads'] for entry in table)
