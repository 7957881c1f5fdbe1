"""The reference project's two MXFP8 acceptance drivers, unmodified, against this package on one GPU.

Same mechanism as tests/test_zu_reference_drivers.py (oracle/_ref/ holds byte-identical copies, its
forwarding modules hand them this package). Their yardstick is torch's own block-scaled matmul
(torch.nn.functional.scaled_mm on the E4M3 payloads and E8M0 scales that the package's quantizer
wrote), so they compare this package's block-scaled tensor-core GEMM with cuBLAS on identical
operands:

  tests/mxfp8_local_driver.py   weight gradients, overwrite and FP32 accumulation, equal to
                                scaled_mm bit for bit (both add the 32-element blocks in ascending K
                                order into an FP32 accumulator), guard bytes around the output
                                untouched, FP32 subnormals surviving + 0, Inf / NaN visible in the
                                rows and columns they touch and gone again after a replay with
                                finite inputs
  tests/mxfp8_driver.py         the public modules with precision='mxfp8': two live forwards on one
                                workspace, reverse-order backward, main_grad accumulation, graph
                                replays with changed inputs and weights; the receive-side quantizer
                                byte-exact against the standalone one for every finite BF16
                                magnitude; non-finite inputs through the receive path

Sorted after the package's own MXFP8 tests and before the file that must run last.
"""
import os
import sys

import pytest
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_zu_reference_drivers import OUTPUT, needs_staged, run  # noqa: E402

pytestmark = [pytest.mark.gpu, needs_staged,
              pytest.mark.skipif(not hasattr(F, 'scaled_mm') or not hasattr(F, 'ScalingType'),
                                 reason="this torch has no block-scaled matmul, the drivers' yardstick")]


def test_mxfp8_local_driver(native):
    out = run('tests/mxfp8_local_driver.py', '--output', os.path.join(OUTPUT, 'reference_mxfp8_local.json'))
    assert 'MXFP8_LOCAL_PASS' in out


def test_mxfp8_driver_on_one_gpu(native):
    out = run('tests/mxfp8_driver.py', '--output', os.path.join(OUTPUT, 'reference_mxfp8_cp1.json'),
              ranks=1, port=29608)
    assert 'MXFP8_PASS' in out
