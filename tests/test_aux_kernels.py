"""GPU parity of the auxiliary kernels (row copy, bias gradient, MXFP8 quantizer) with the CPU
oracle. Byte and index work is compared bit-exactly; FP32 sums by the reference's own bound
4 * eps * sum|x| (tests/bias_grad_driver.py:23-46 of the reference)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from oracle import mxfp8_oracle as mx
from oracle.ulysses_oracle import resize_rank_rows_ref

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


@pytest.mark.parametrize('peers,width', [(1, 128), (8, 384), (4, 640), (16, 256)])
@pytest.mark.parametrize('rows', [1, 127, 256, 257, 1031])
@pytest.mark.parametrize('segments', [1, 3, 4])
def test_resize_rank_rows_is_exact(native, peers, width, rows, segments):
    from fused_gemm_a2a_kernels import resize_rank_rows
    capacity = (rows + 255) // 256 * 256
    g = torch.Generator().manual_seed(rows * 131 + width)
    sources = tuple(torch.randn(peers * rows, width, generator=g).to(torch.bfloat16) for _ in range(segments))
    dev_sources = tuple(t.to(DEV) for t in sources)
    padded = resize_rank_rows(dev_sources, peers, capacity)
    for actual, expected in zip(padded, resize_rank_rows_ref(sources, peers, capacity)):
        assert torch.equal(actual.cpu(), expected)
    owned = resize_rank_rows(padded, peers, rows, copy=True)
    for actual, source, workspace in zip(owned, sources, padded):
        assert actual.data_ptr() != workspace.data_ptr() and actual.is_contiguous()
        assert torch.equal(actual.cpu(), source)
    keep = tuple(t.clone() for t in owned)
    for workspace in padded:
        workspace.zero_()
    for actual, wanted in zip(owned, keep):
        assert torch.equal(actual, wanted)
    if segments > 1 and width % 128 == 0:
        # Interleaved bias: only logical rows receive it, whichever side carries the padding
        # (reference tests/row_copy_driver.py:40-57).
        bias = torch.randn(peers * width // 128 * segments * 128, generator=g).to(torch.bfloat16)
        dev_sources = tuple(t.to(DEV) for t in sources)  # the zeroing above may have aliased them
        padded = resize_rank_rows(dev_sources, peers, capacity)
        for head_offset in sorted({0, (peers - 1) * width // 128}):
            for inputs, out_rows in ((dev_sources, rows), (dev_sources, capacity), (padded, rows)):
                got = resize_rank_rows(inputs, peers, out_rows, copy=True, bias=bias.to(DEV),
                                       head_dim=128, head_offset=head_offset)
                want = resize_rank_rows_ref(sources, peers, out_rows, bias=bias, head_dim=128,
                                            head_offset=head_offset)
                for a, w in zip(got, want):
                    assert torch.equal(a.cpu(), w)


def test_resize_rank_rows_rejects_bad_arguments(native):
    from fused_gemm_a2a_kernels import resize_rank_rows
    t = torch.zeros(6, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match='split evenly'):
        resize_rank_rows((t,), 4, 2)
    with pytest.raises(ValueError, match='CUDA matrices'):
        resize_rank_rows((t.cpu(),), 2, 2)
    with pytest.raises(ValueError, match='Bias must cover'):
        resize_rank_rows((t,), 2, 3, bias=torch.zeros(8, dtype=torch.bfloat16, device=DEV))
    assert resize_rank_rows((t,), 2, 3)[0] is t  # nothing to do: the input itself


@pytest.mark.parametrize('rows,width', [(1, 128), (255, 384), (256, 4096), (1000, 12288), (4099, 520)])
@pytest.mark.parametrize('out_dtype', [torch.bfloat16, torch.float32])
def test_reduce_bias_grad(native, rows, width, out_dtype):
    from fused_gemm_a2a_kernels import reduce_bias_grad
    g = torch.Generator().manual_seed(rows + width)
    dy = torch.randn(rows, width, generator=g).to(torch.bfloat16)
    out = reduce_bias_grad(dy.to(DEV), torch.empty(width, dtype=out_dtype, device=DEV))
    exact = dy.double().sum(0)
    bound = 4 * torch.finfo(torch.float32).eps * dy.double().abs().sum(0) + 1e-30
    if out_dtype == torch.float32:
        assert ((out.cpu().double() - exact).abs() <= bound).all()
        seed = torch.randn(width, generator=g)
        acc = reduce_bias_grad(dy.to(DEV), seed.to(DEV).clone(), accumulate=True)
        assert ((acc.cpu().double() - exact - seed.double()).abs() <= bound + 1e-6 * seed.abs()).all()
    else:
        # one BF16 rounding of an FP32 sum: within half a BF16 ulp of the exact value plus the sum bound
        ulp = exact.abs() * 2.0 ** -8 + bound
        assert ((out.cpu().double() - exact).abs() <= ulp).all()


def test_reduce_bias_grad_integer_sums_are_exact(native):
    from fused_gemm_a2a_kernels import reduce_bias_grad
    dy = torch.randint(-4, 5, (3000, 256)).to(torch.bfloat16)
    out = reduce_bias_grad(dy.to(DEV), torch.empty(256, dtype=torch.float32, device=DEV))
    assert torch.equal(out.cpu(), dy.float().sum(0))


# ---- the reference's own Triton kernels, recorded through Triton's CPU interpreter ----------------
@pytest.mark.parametrize('name', ['copy_grow', 'copy_shrink', 'copy_same', 'biased_grow', 'biased_shrink',
                                  'biased_same'])
def test_row_copy_equals_the_reference_kernels_recorded_output(native, name):
    """tests/golden/aux_kernels.npz (made by tests/golden/make_golden_aux.py from
    fused_gemm_a2a_kernels.py:1106-1142 of the reference): widths that are not multiples of 8, heads
    of 16, 64 and 128 columns, head offsets, growing and shrinking. Bit for bit."""
    from fused_gemm_a2a_kernels import resize_rank_rows
    from test_oracle_golden import GOLDEN, aux_copy_case
    z = np.load(os.path.join(GOLDEN, 'aux_kernels.npz'))
    sources, wanted, peers, rows, kwargs = aux_copy_case(z, name)
    if 'bias' in kwargs:
        kwargs['bias'] = kwargs['bias'].to(DEV)
    got = resize_rank_rows(tuple(t.to(DEV) for t in sources), peers, rows, copy=True, **kwargs)
    for i, (a, w) in enumerate(zip(got, wanted)):
        assert torch.equal(a.cpu().view(torch.int16), w.view(torch.int16)), f'{name} tensor {i}'


@pytest.mark.parametrize('name', ['bias_one_part_bf16', 'bias_one_part_f32_acc', 'bias_parts_bf16_acc',
                                  'bias_parts_f32', 'bias_many_parts_f32_acc'])
def test_bias_gradient_against_the_reference_kernels_recorded_output(native, name):
    """Same file, fused_gemm_a2a_kernels.py:1053-1103 of the reference. Both sides add in FP32 in
    their own order: within twice the reference's bound 4 * eps * sum|x|; a BF16 result, which the
    interpreter truncates, within one more BF16 step; the quarter-integer case bit for bit."""
    from fused_gemm_a2a_kernels import reduce_bias_grad
    from test_oracle_golden import GOLDEN, aux_tensor
    z = np.load(os.path.join(GOLDEN, 'aux_kernels.npz'))
    dy, previous, wanted = (aux_tensor(z, f'{name}.{key}') for key in ('dy', 'previous', 'out'))
    accumulate = bool(z[f'{name}.accumulate'])
    got = reduce_bias_grad(dy.to(DEV), previous.to(DEV).clone(), accumulate=accumulate).cpu()
    if name == 'bias_many_parts_f32_acc':
        assert torch.equal(got, wanted)
        return
    bound = 8 * torch.finfo(torch.float32).eps * (dy.double().abs().sum(0) + previous.double().abs() * accumulate)
    if wanted.dtype == torch.bfloat16:
        bound = bound + wanted.double().abs() * 2.0 ** -7
    assert ((got.double() - wanted.double()).abs() <= bound + 1e-30).all()


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _special_matrix(rows, k, seed):
    """N(0,1) with outlier groups (x1e3), an all-zero group, subnormals, +-Inf and NaN."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(rows, k, generator=g)
    mask = torch.rand(rows, k, generator=g) < 0.001
    a = torch.where(mask, a * 1e3, a)
    if k >= 64:
        a[0, 32:64] = 0.0
    a = a.to(torch.bfloat16)
    if rows > 3 and k > 40:
        a[1, 3] = float('inf')
        a[2, 40] = float('-inf')
        a[3, 5] = float('nan')
        a[3, 6] = 1e-40  # BF16 subnormal
    return a


@pytest.mark.parametrize('rows,k,k_multiple', [(128, 33, 256), (256, 512, 256), (300, 1000, 128), (17, 4096, 128)])
def test_mxfp8_quantize_rows_bit_exact(native, rows, k, k_multiple):
    from fused_gemm_a2a_kernels import mxfp8_quantize
    kk = (k + 7) // 8 * 8
    a = _special_matrix(rows, kk, seed=rows + k)[:, :k] if kk == k else _special_matrix(rows, kk, seed=rows + k)
    view = a.to(DEV)[:, :k]
    q, sf = mxfp8_quantize(view, k_multiple=k_multiple)
    q_ref, sf_ref = mx.quantize(_bits(view.contiguous()), k_multiple=k_multiple)
    _compare_quantized(q, sf, q_ref, sf_ref)


@pytest.mark.parametrize('rows,k', [(256, 128), (384, 1000), (512, 4099), (136, 72)])
def test_mxfp8_quantize_transposed_bit_exact(native, rows, k):
    """a.T of a row-major [k, rows] matrix: quantized along the strided axis, no transpose copy."""
    from fused_gemm_a2a_kernels import mxfp8_quantize
    base = _special_matrix(k, rows, seed=rows * 7 + k).to(DEV)   # memory layout [k, rows]
    q, sf = mxfp8_quantize(base.t())
    q_ref, sf_ref = mx.quantize(_bits(base.t().contiguous()))
    _compare_quantized(q, sf, q_ref, sf_ref)


def _compare_quantized(q, sf, q_ref, sf_ref):
    q = q.view(torch.uint8).cpu().numpy()
    sf = sf.cpu().numpy()
    assert q.shape == q_ref.shape and sf.shape == sf_ref.shape
    assert np.array_equal(sf, sf_ref), 'E8M0 scale bytes differ'
    nan_ref = (q_ref & 0x7f) == 0x7f
    nan_got = (q & 0x7f) == 0x7f
    assert np.array_equal(nan_got, nan_ref), 'NaN payload positions differ'
    assert np.array_equal(q[~nan_ref], q_ref[~nan_ref]), 'E4M3 codes differ'


def test_mxfp8_known_answers_of_the_reference_tests(native):
    """Inf groups: scale byte 255 at offsets [0, 16, 33], NaN payload at the Inf elements only
    (reference tests/mxfp8_local_driver.py:63-77)."""
    from fused_gemm_a2a_kernels import mxfp8_quantize
    a = torch.ones(128, 40, dtype=torch.bfloat16, device=DEV)[:, :33]
    a[0, 0] = float('inf')
    a[1, 31] = float('-inf')
    a[2, 32] = float('inf')
    q, sf = mxfp8_quantize(a)
    sf = sf.cpu().numpy()
    assert sorted(np.nonzero(sf == 255)[0].tolist()) == [0, 16, 33]
    payload = q.view(torch.uint8).cpu().numpy()
    nan = (payload & 0x7f) == 0x7f
    assert sorted(zip(*np.nonzero(nan))) == [(0, 0), (1, 31), (2, 32)]
