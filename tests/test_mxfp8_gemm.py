"""GPU parity of the block-scaled MXFP8 GEMM (fga_gemm_local_mx) through the C ABI.

Operands are quantized by the CUDA quantizer (itself bit-exact against the CPU oracle, see
test_aux_kernels.py); the product is compared with the oracle's exact dequantized product in
float64. The tensor core accumulates in FP32, so the result may differ by summation order only:
max error <= 1e-4 of the output scale for FP32 outputs, BF16 rounding (2^-8) on top for BF16.
"""
import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as mx

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
TIMEOUT_NS = 5_000_000_000


def _bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _operands(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g)
    a = torch.where(torch.rand(m, k, generator=g) < 0.001, a * 1e3, a)   # outlier groups
    if k >= 64:
        a[0, 32:64] = 0                                                   # an all-zero group
    b = torch.randn(n, k, generator=g) / k ** 0.5
    return a.to(torch.bfloat16).to(DEV), b.to(torch.bfloat16).to(DEV)


@pytest.mark.parametrize('m,n,k', [(256, 256, 128), (256, 128, 256), (300, 512, 1000), (1024, 768, 4096),
                                   (1, 128, 40), (2048, 2048, 2048)])
@pytest.mark.parametrize('out_f32', [True, False])
def test_block_scaled_gemm_matches_dequantized_product(native, m, n, k, out_f32):
    from fused_gemm_a2a_kernels import mxfp8_quantize
    a, b = _operands(m, n, k, seed=m + n + k)
    aq, sa = mxfp8_quantize(a)
    bq, sb = mxfp8_quantize(b)
    assert aq.shape[1] == bq.shape[1]
    c = torch.full((m, n), float('nan'), dtype=torch.float32 if out_f32 else torch.bfloat16, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    rc = native.fga_gemm_local_mx(aq.data_ptr(), sa.data_ptr(), aq.shape[0], bq.data_ptr(), sb.data_ptr(),
                                  bq.shape[0], m, n, aq.shape[1], c.data_ptr(), n, int(out_f32), 0,
                                  status.data_ptr(), TIMEOUT_NS, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    want = mx.mx_matmul(_bits(a), _bits(b))
    got = c.float().cpu().numpy().astype(np.float64)
    scale = np.abs(want).max()
    tol = (1e-4 if out_f32 else 1e-4 + 2.0 ** -8) * scale
    assert np.abs(got - want).max() <= tol


def test_accumulate_adds_in_fp32(native):
    from fused_gemm_a2a_kernels import mxfp8_quantize
    m, n, k = 512, 384, 776
    a, b = _operands(m, n, k, seed=9)
    aq, sa = mxfp8_quantize(a)
    bq, sb = mxfp8_quantize(b)
    seed = torch.randn(m, n, generator=torch.Generator().manual_seed(1)).to(DEV)
    seed[0, 0] = 1e-42   # an FP32 subnormal survives an accumulation of an exact zero product row
    a2 = a.clone(); a2[0] = 0
    aq2, sa2 = mxfp8_quantize(a2)
    c = seed.clone()
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    rc = native.fga_gemm_local_mx(aq2.data_ptr(), sa2.data_ptr(), aq2.shape[0], bq.data_ptr(), sb.data_ptr(),
                                  bq.shape[0], m, n, aq2.shape[1], c.data_ptr(), n, 1, 1,
                                  status.data_ptr(), TIMEOUT_NS, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    want = mx.mx_matmul(_bits(a2), _bits(b)) + seed.double().cpu().numpy()
    got = c.double().cpu().numpy()
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
    assert torch.equal(c[0], seed[0])          # zero product row: the seed row is untouched bit for bit
