"""GPU parity of the tcgen05 GEMM through the C ABI (fga_gemm_local) against an FP32 reference.

Tolerance (stated by the task): BF16 outputs within max relative error 1e-2 of the output scale
and Frobenius relative error <= 2e-3 of an FP32-accumulated reference; FP32 outputs differ from it
only by summation order (checked to 1e-4 of the output scale).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TIMEOUT_NS = 5_000_000_000


def _run(native, m, n, k, a_km, b_kn, out_f32=False, accumulate=False, seed=0):
    dev = torch.device('cuda', 0)
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
    b = (torch.randn(n, k, generator=g) / 8).to(torch.bfloat16).to(dev)
    a_mem = a.t().contiguous() if a_km else a
    b_mem = b.t().contiguous() if b_kn else b
    ref = a.float() @ b.float().t()
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    if out_f32:
        seed_val = torch.randn(m, n, generator=g).to(dev) if accumulate else None
        c = seed_val.clone() if accumulate else torch.full((m, n), float('nan'), device=dev)
        if accumulate:
            ref = ref + seed_val
    else:
        c = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device=dev)
    rc = native.fga_gemm_local(a_mem.data_ptr(), int(a_km), b_mem.data_ptr(), int(b_kn), m, n, k,
                               m if a_km else k, n if b_kn else k, c.data_ptr(), n, int(out_f32),
                               int(accumulate), status.data_ptr(), TIMEOUT_NS,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    return c.float(), ref


@pytest.mark.parametrize('m,n,k', [(256, 256, 64), (256, 128, 128), (512, 768, 512), (100, 256, 200),
                                   (1, 128, 64), (257, 384, 4096)])
@pytest.mark.parametrize('a_km,b_kn', [(0, 0), (0, 1)])
def test_bf16_output(native, m, n, k, a_km, b_kn):
    c, ref = _run(native, m, n, k, a_km, b_kn)
    scale = ref.abs().max()
    assert (c - ref).abs().max() <= 1e-2 * scale
    assert torch.linalg.norm(c - ref) <= 2e-3 * torch.linalg.norm(ref)


@pytest.mark.parametrize('m,n,k', [(512, 512, 512), (384, 256, 1001), (128, 128, 1), (1024, 384, 4097)])
@pytest.mark.parametrize('accumulate', [False, True])
def test_weight_gradient_layout_fp32(native, m, n, k, accumulate):
    """Both operands read transposed (dW = dY^T X), FP32 store or in-place accumulate."""
    c, ref = _run(native, m, n, k, 1, 1, out_f32=True, accumulate=accumulate)
    assert (c - ref).abs().max() <= 1e-4 * ref.abs().max()


def test_large_square_matches_reference(native):
    c, ref = _run(native, 2048, 2048, 2048, 0, 0)
    assert torch.linalg.norm(c - ref) <= 2e-3 * torch.linalg.norm(ref)


def test_argument_errors_are_reported(native):
    dev = torch.device('cuda', 0)
    t = torch.zeros(256, 256, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = native.fga_gemm_local(t.data_ptr(), 0, t.data_ptr(), 0, 256, 100, 256, 256, 256,
                               t.data_ptr(), 256, 0, 0, status.data_ptr(), TIMEOUT_NS, 0)
    assert rc == -1 and b'multiple of 128' in native.fga_last_error()
    rc = native.fga_gemm_local(t.data_ptr(), 0, t.data_ptr(), 0, 256, 256, 256, 256, 256,
                               t.data_ptr(), 256, 0, 1, status.data_ptr(), TIMEOUT_NS, 0)
    assert rc == -1 and b'FP32 output' in native.fga_last_error()
