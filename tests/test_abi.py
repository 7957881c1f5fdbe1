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


def _prototypes():
    """name -> (return type, [parameter declarations]) for every function declared in fga.h."""
    text = open(os.path.join(ROOT, 'include', 'fga.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    text = re.sub(r'#.*', '', text)
    found = {}
    for ret, name, params in re.findall(r'([\w\s\*]+?)\b(fga_\w+)\s*\(([^)]*)\)\s*;', text):
        params = [p.strip() for p in params.split(',')] if params.strip() not in ('', 'void') else []
        found[name] = (' '.join(ret.split()), params)
    return found


def test_ctypes_signatures_match_the_header():
    """Every binding in _fga_native.py has the header's parameter count, a pointer type exactly where
    the header has a pointer or array, and the header's integer width elsewhere."""
    import ctypes
    lib = _fga_native.lib()
    scalars = {'int': ctypes.c_int, 'int64_t': ctypes.c_int64, 'uint64_t': ctypes.c_uint64, 'size_t': ctypes.c_size_t}
    pointers = (ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int))
    returns = {'int': ctypes.c_int, 'int64_t': ctypes.c_int64, 'uint64_t': ctypes.c_uint64,
               'const char*': ctypes.c_char_p, 'const char *': ctypes.c_char_p}
    prototypes = _prototypes()
    assert set(prototypes) == set(_fga_native.EXPORTS)
    for name, (ret, params) in prototypes.items():
        fn = getattr(lib, name)
        assert fn.restype is returns[ret], f'{name}: return type {ret}'
        argtypes = fn.argtypes or []
        if not params:
            assert not argtypes, name
            continue
        assert len(argtypes) == len(params), f'{name}: {len(argtypes)} bound, {len(params)} declared'
        for bound, declared in zip(argtypes, params):
            if '*' in declared or '[' in declared:
                assert bound in pointers, f'{name}: `{declared}` bound as {bound}'
            else:
                base = declared.replace('const ', '').split()[0]
                assert bound is scalars[base], f'{name}: `{declared}` bound as {bound}'


def test_cpu_stand_ins_take_the_header_parameters():
    """The recorder and the simulator used by the host-layer tests restate entry points of the
    header; their parameter lists must follow it (a drifted stand-in would test a different ABI)."""
    import inspect
    import sys
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    import abi_simulator
    import host_trace
    prototypes = _prototypes()
    checked = 0
    for cls in (host_trace.FakeLib, abi_simulator.SimulatedLibrary):
        for name, member in inspect.getmembers(cls, inspect.isfunction):
            if not name.startswith('fga_') or name == 'fga_last_error':
                continue
            declared = [re.sub(r'\[.*\]', '', p).replace('*', ' ').split()[-1] for p in prototypes[name][1]]
            given = list(inspect.signature(member).parameters)[1:]
            assert len(given) == len(declared), f'{cls.__name__}.{name}: {given} vs {declared}'
            checked += 1
    assert checked >= 10
