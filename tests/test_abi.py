"""The C-ABI shared library builds for sm_100a without a GPU, loads, and exports every symbol that
include/fga.h declares. No compute entry point is called here."""
import os
import re

import _fga_native
import build_native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'fga.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(fga_\w+)\s*\(', text)))


def test_library_builds_and_exports_the_declared_abi():
    path = build_native.build()
    assert os.path.exists(path)
    lib = _fga_native.lib()
    names = declared_symbols()
    assert len(names) >= 16
    for name in names:
        assert hasattr(lib, name), f'{name} is declared in fga.h but not exported'
    assert sorted(_fga_native.EXPORTS) == names
    assert lib.fga_version() == 1


def test_argument_errors_do_not_need_a_gpu():
    lib = _fga_native.lib()
    assert lib.fga_barrier(None, None, 0, 1, 0, None, 0, None, None, 0, None) == -1
    assert b'null' in lib.fga_last_error()
    assert lib.fga_gemm_local(None, 0, None, 0, 1, 1, 1, 8, 8, None, 8, 0, 0, None, 0, None) == -1
    assert lib.fga_bias_grad_scratch_floats(1000, 512) == 4 * 512
    try:
        _fga_native.check(-1)
    except ValueError as error:
        assert 'null' in str(error)
    else:
        raise AssertionError('check() accepted a failure code')


def test_no_tma_load_fans_out_across_the_cluster():
    # TMA loads that fan one tile out to several CTAs of a cluster are banned from this code base
    # (issued on another GPU's memory they hang the GPU). The only qualifier of that family that
    # may appear is the one on tcgen05.commit, which fans out an mbarrier arrival, not data.
    needle = '::'.join(('multicast', 'cluster'))
    csrc = os.path.join(ROOT, 'fused-gemm-a2a_b200', 'csrc')
    for name in os.listdir(csrc):
        for line in open(os.path.join(csrc, name)):
            if needle in line:
                assert 'cp.async' not in line, f'{name}: {line.strip()}'
