"""The allocation-free bias-gradient entry point (collected last on purpose).

Some callers may not allocate device memory at the call site - a host whose memory budget is
planned in advance, or one that forbids cudaMalloc on its hot path - so they cannot hand the
reduction its scratch buffer. fga_bias_grad_static keeps the partial sums in an array inside the
library's own device image instead. It must give exactly the result of fga_bias_grad (same
kernels, same summation order), also when called twice in a row on the shared array, and it must
refuse problems larger than the array.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def _both(native, dy, out_dtype, accumulate, seed=None):
    rows, width = dy.shape
    stream = torch.cuda.current_stream().cuda_stream
    base = torch.zeros(width, dtype=out_dtype, device=DEV) if seed is None else seed.clone()
    want, got = base.clone(), base.clone()
    scratch = torch.empty(native.fga_bias_grad_scratch_floats(rows, width), dtype=torch.float32, device=DEV)
    is_f32 = int(out_dtype == torch.float32)
    assert native.fga_bias_grad(dy.data_ptr(), rows, width, want.data_ptr(), is_f32, int(accumulate),
                                scratch.data_ptr(), stream) == 0, native.fga_last_error()
    assert native.fga_bias_grad_static(dy.data_ptr(), rows, width, got.data_ptr(), is_f32, int(accumulate),
                                       stream) == 0, native.fga_last_error()
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row(native):
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(2024)
    first = torch.randn(4099, 520, generator=g).to(torch.bfloat16).to(DEV)
    second = torch.randn(700, 1408, generator=g).to(torch.bfloat16).to(DEV)   # other shape: stale partials
    seed = torch.randn(520, generator=g).to(DEV)
    # bit-exact: both entry points run the same two kernels in the same order
    got, want = _both(native, first, torch.float32, True, seed)
    assert torch.equal(got, want)
    got, want = _both(native, second, torch.bfloat16, False)
    assert torch.equal(got, want)
    got, want = _both(native, first, torch.float32, False)
    assert torch.equal(got, want)
    exact = first.double().sum(0)
    bound = 4 * torch.finfo(torch.float32).eps * first.double().abs().sum(0)
    assert ((got.double() - exact).abs() <= bound).all()


def test_static_scratch_rejects_problems_beyond_its_capacity(native):
    capacity = native.fga_bias_grad_static_capacity_floats()
    assert capacity == 1 << 20
    width = 4096
    rows = (capacity // width + 1) * 256          # one 256-row part too many
    dy = torch.zeros(rows, width, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(width, dtype=torch.float32, device=DEV)
    rc = native.fga_bias_grad_static(dy.data_ptr(), rows, width, out.data_ptr(), 1, 0,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and b'scratch floats' in native.fga_last_error()
    rows = capacity // width * 256                # exactly full: accepted
    rc = native.fga_bias_grad_static(dy.data_ptr(), rows, width, out.data_ptr(), 1, 0,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert not out.abs().any()
