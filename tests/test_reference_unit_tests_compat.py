"""Drop-in check on the CPU: the reference project's own GPU-free unit tests (geometry invariants,
MXFP8 main_grad validation, the padded row-block data-flow model) are loaded from the reference
checkout where it lies and run unmodified against this package, which is placed in sys.modules
under the reference's module names first. Nothing is copied; without a reference checkout (the GPU
box has none) the test is skipped.

The checkout is looked up in $FGA_REFERENCE_ROOT, else in `reference/` under the home directory.
"""
import importlib.util
import os
import sys
import unittest

import pytest

REFERENCE_ROOT = os.environ.get('FGA_REFERENCE_ROOT', os.path.join(os.path.expanduser('~'), 'reference'))
# files of the reference's tests/ that need no GPU and import the modules this package replaces
FILES = ('test_recv_plan.py', 'test_row_blocks.py')


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_ROOT, 'tests')),
                    reason='no reference checkout on this machine')
@pytest.mark.parametrize('name', FILES)
def test_reference_unit_tests_pass_against_this_package(name):
    import fused_gemm_a2a          # this package, found through the path set up by conftest.py
    import fused_gemm_a2a_kernels
    assert 'fused-gemm-a2a_b200' in fused_gemm_a2a.__file__ and 'fused-gemm-a2a_b200' in fused_gemm_a2a_kernels.__file__
    path = os.path.join(REFERENCE_ROOT, 'tests', name)
    spec = importlib.util.spec_from_file_location('reference_' + name[:-3], path)
    module = importlib.util.module_from_spec(spec)
    before = list(sys.path)
    try:
        spec.loader.exec_module(module)   # its `import fused_gemm_a2a` resolves to sys.modules: this package
        for attr in ('fused',):
            if hasattr(module, attr):
                assert getattr(module, attr) is fused_gemm_a2a
        suite = unittest.defaultTestLoader.loadTestsFromModule(module)
        assert suite.countTestCases() > 0
        result = unittest.TextTestRunner(verbosity=0).run(suite)
    finally:
        sys.path[:] = before
        for key in [k for k in sys.modules if k == 'benchmark' or k.startswith('benchmark.')]:
            del sys.modules[key]       # the reference's benchmark package must not shadow anything later
    assert result.wasSuccessful(), (result.failures, result.errors)
