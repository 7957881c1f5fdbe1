"""The CPU oracle against golden vectors produced by the reference's own unfused Ulysses modules
(benchmark/reference.py of the reference tree, run under gloo by tests/golden/make_golden.py).
Float32 inputs, float64 accumulation in the oracle; the reference computed in float32, so outputs
agree to float32 round-off (1e-4 of each tensor's scale)."""
import os

import numpy as np
import pytest
import torch

from oracle.ulysses_oracle import UlyssesOracle, deinterleave_qkv_rows, interleave_qkv_rows
from tests.golden.make_golden import c1_inputs, sample

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def near(actual, expected, what, rel=1e-4):
    actual, expected = np.asarray(actual, dtype=np.float64), np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape, what
    assert np.abs(actual - expected).max() <= rel * max(np.abs(expected).max(), 1e-6), what


def tensors(z, p, key):
    return [torch.from_numpy(z[f'r{r}_{key}']) for r in range(p)]


@pytest.mark.parametrize('name,p,hidden,heads,segments,bias', [
    ('small_p2', 2, 32, 4, 4, True), ('small_p4', 4, 64, 8, 3, False)])
def test_oracle_reproduces_reference_modules(name, p, hidden, heads, segments, bias):
    z = np.load(os.path.join(GOLDEN, f'ulysses_{name}.npz'))
    d = hidden // heads
    wq = interleave_qkv_rows(torch.from_numpy(z['w']), heads, d)
    bq = interleave_qkv_rows(torch.from_numpy(z['b']), heads, d) if bias else None
    wo = torch.from_numpy(z['wo'])
    bo = torch.from_numpy(z['bo']) if bias else None
    oracle = UlyssesOracle(p, hidden, heads, segments, wq, bq, wo, bo, dtype=torch.float32,
                           acc_dtype=torch.float64)
    xs, os_, dys = tensors(z, p, 'x'), tensors(z, p, 'o'), tensors(z, p, 'dy')
    grads = [tuple(torch.from_numpy(z[f'r{r}_g{i}']) for i in range(segments)) for r in range(p)]
    outs = oracle.qkv_forward(xs)
    back = oracle.qkv_backward(xs, grads)
    ys = oracle.out_forward(os_)
    dos, out_params = oracle.out_backward(os_, dys)
    for r in range(p):
        for i in range(segments):
            near(outs[r][i], z[f'r{r}_out{i}'], f'rank {r} output {i}')
        dx, dw, db = back[r]
        near(dx, z[f'r{r}_dx'], f'rank {r} dx')
        # the reference holds segment-major parameter gradients, rank-local (not yet all-reduced)
        near(deinterleave_qkv_rows(dw, heads, d), z[f'r{r}_dw'], f'rank {r} dW_qkv')
        near(ys[r], z[f'r{r}_y'], f'rank {r} y')
        near(dos[r], z[f'r{r}_do'], f'rank {r} dO')
        near(out_params[r][0], z[f'r{r}_dwo'], f'rank {r} dW_o')
        if bias:
            near(deinterleave_qkv_rows(db, heads, d), z[f'r{r}_db'], f'rank {r} dbias_qkv')
            near(out_params[r][1], z[f'r{r}_dbo'], f'rank {r} dbias_o')


def test_oracle_reproduces_cpu_benchmark_configuration():
    """P=2, per-rank M=512, H=1024, 8 heads of 128, fp32, no bias: checksums and strided samples of
    every output of the reference run."""
    z = np.load(os.path.join(GOLDEN, 'ulysses_c1_p2.npz'))
    p, m, hidden, heads = 2, 512, 1024, 8
    per_rank = [c1_inputs(r, p, m, hidden, heads) for r in range(p)]
    w, wo = per_rank[0][0], per_rank[0][1]
    wq = interleave_qkv_rows(torch.cat(w), heads, hidden // heads)
    oracle = UlyssesOracle(p, hidden, heads, 3, wq, None, wo, None, dtype=torch.float32,
                           acc_dtype=torch.float64)
    xs = [t[2] for t in per_rank]
    grads = [tuple(t[3]) for t in per_rank]
    os_ = [t[4] for t in per_rank]
    dys = [t[5] for t in per_rank]
    outs, back = oracle.qkv_forward(xs), oracle.qkv_backward(xs, grads)
    ys = oracle.out_forward(os_)
    dos, out_params = oracle.out_backward(os_, dys)
    for r in range(p):
        got = {f'out{i}': outs[r][i] for i in range(3)}
        got.update(dx=back[r][0], dw=deinterleave_qkv_rows(back[r][1], heads, hidden // heads),
                   y=ys[r], do=dos[r], dwo=out_params[r][0])
        for key, value in got.items():
            value = value.float().numpy()
            near(sample(value), z[f'r{r}_{key}_sample'], f'rank {r} {key} samples', rel=2e-4)
            scale = float(z[f'r{r}_{key}_abs'])
            assert abs(np.abs(value.astype(np.float64)).sum() - scale) <= 1e-5 * scale, key
            assert abs(value.astype(np.float64).sum() - float(z[f'r{r}_{key}_sum'])) <= 1e-5 * scale, key


def test_row_interleave_round_trip():
    heads, d = 4, 8
    for s in (3, 4):
        seg = torch.randn(s * heads * d, 16)
        inter = interleave_qkv_rows(seg, heads, d)
        for h in range(heads):
            for j in range(s):
                rows = slice((h * s + j) * d, (h * s + j + 1) * d)
                assert torch.equal(inter[rows], seg[j * heads * d + h * d:j * heads * d + (h + 1) * d])
        assert torch.equal(deinterleave_qkv_rows(inter, heads, d), seg)
    with pytest.raises(ValueError):
        interleave_qkv_rows(torch.randn(5 * heads * d, 16), heads, d)


def test_padded_buffers_match_unpadded_flow():
    """The padded transport model (head-side and receive buffers with pad rows) carries exactly
    the unpadded results in its logical rows and zeros elsewhere."""
    torch.manual_seed(0)
    p, m, hidden, heads, capacity = 4, 37, 64, 8, 48
    d = hidden // heads
    wq, wo = torch.randn(3 * hidden, hidden, dtype=torch.float64), torch.randn(hidden, hidden, dtype=torch.float64)
    oracle = UlyssesOracle(p, hidden, heads, 3, wq, None, wo, None, dtype=torch.float64, acc_dtype=torch.float64)
    xs = [torch.randn(m, hidden, dtype=torch.float64) for _ in range(p)]
    outs = oracle.qkv_forward(xs)
    bufs = oracle.qkv_heads_buffers(xs, capacity)
    for dest in range(p):
        for s in range(3):
            blocks = bufs[dest][s].view(p, capacity, hidden // p)
            assert torch.equal(blocks[:, :m].reshape(p * m, heads // p, d), outs[dest][s])
            assert not blocks[:, m:].any()
    grads = [tuple(torch.randn(p * m, heads // p, d, dtype=torch.float64) for _ in range(3)) for _ in range(p)]
    for r in range(p):
        padded = oracle.qkv_recv_buffer(grads, r, capacity)
        assert torch.equal(padded[:m], oracle.qkv_recv_buffer(grads, r)) and not padded[m:].any()


@pytest.mark.parametrize('name,kv_heads,gate,bias', [('gqa_p2', 2, True, True), ('gqa_r2_p2', 4, False, False)])
def test_grouped_query_oracle_reproduces_reference_modules(name, kv_heads, gate, bias):
    """The reference's unfused modules with num_kv_heads < num_heads (benchmark/reference.py:151-163):
    8 query heads over 2 (or 4) key/value heads on two ranks. The oracle takes the weights in the
    grouped row order [q_g0..; k_g; v_g; (gate_g0..)]; parameter gradients come back in that order."""
    from oracle.ulysses_oracle import GroupedQueryOracle, deinterleave_gqa_rows, interleave_gqa_rows
    z = np.load(os.path.join(GOLDEN, f'ulysses_{name}.npz'))
    p, hidden, heads = 2, 64, 8
    d = hidden // heads
    kinds = 4 if gate else 3
    wq = interleave_gqa_rows(torch.from_numpy(z['w']), heads, kv_heads, d, gate)
    bq = interleave_gqa_rows(torch.from_numpy(z['b']), heads, kv_heads, d, gate) if bias else None
    wo = torch.from_numpy(z['wo'])
    bo = torch.from_numpy(z['bo']) if bias else None
    oracle = GroupedQueryOracle(p, hidden, heads, kv_heads, gate, weight_qkv=wq, bias_qkv=bq, weight_out=wo,
                                bias_out=bo, dtype=torch.float32, acc_dtype=torch.float64)
    xs, os_, dys = tensors(z, p, 'x'), tensors(z, p, 'o'), tensors(z, p, 'dy')
    grads = [tuple(torch.from_numpy(z[f'r{r}_g{i}']) for i in range(kinds)) for r in range(p)]
    outs = oracle.qkv_forward(xs)
    back = oracle.qkv_backward(xs, grads)
    ys = oracle.out_forward(os_)
    dos, out_params = oracle.out_backward(os_, dys)
    for r in range(p):
        assert [tuple(t.shape) for t in outs[r]] == [tuple(z[f'r{r}_out{i}'].shape) for i in range(kinds)]
        assert outs[r][1].shape[1] == kv_heads // p and outs[r][0].shape[1] == heads // p
        for i in range(kinds):
            near(outs[r][i], z[f'r{r}_out{i}'], f'rank {r} output {i}')
        dx, dw, db = back[r]
        near(dx, z[f'r{r}_dx'], f'rank {r} dx')
        near(deinterleave_gqa_rows(dw, heads, kv_heads, d, gate), z[f'r{r}_dw'], f'rank {r} dW_qkv')
        near(ys[r], z[f'r{r}_y'], f'rank {r} y')
        near(dos[r], z[f'r{r}_do'], f'rank {r} dO')
        near(out_params[r][0], z[f'r{r}_dwo'], f'rank {r} dW_o')
        if bias:
            near(deinterleave_gqa_rows(db, heads, kv_heads, d, gate), z[f'r{r}_db'], f'rank {r} dbias_qkv')
    # the padded transport buffers carry exactly the unpadded results in their logical rows
    capacity = 16
    bufs = oracle.qkv_heads_buffers(xs, capacity)
    oracle_no_late_bias = GroupedQueryOracle(p, hidden, heads, kv_heads, gate, weight_qkv=wq, weight_out=wo,
                                             dtype=torch.float32, acc_dtype=torch.float64)
    plain = oracle_no_late_bias.qkv_forward(xs)
    m = xs[0].shape[0]
    for dest in range(p):
        for kind in range(kinds):
            blocks = bufs[dest][kind].view(p, capacity, -1)
            assert torch.equal(blocks[:, :m].reshape(plain[dest][kind].shape), plain[dest][kind])
            assert not blocks[:, m:].any()
    for r in range(p):
        padded = oracle.qkv_recv_buffer(grads, r, capacity)
        assert torch.equal(padded[:m], oracle.qkv_recv_buffer(grads, r)) and not padded[m:].any()


# ---------------------------------------------------------------------- auxiliary kernels
# tests/golden/aux_kernels.npz holds inputs and outputs of the reference's own Triton row-copy and
# bias-gradient kernels (fused_gemm_a2a_kernels.py:1053-1142), executed by Triton's CPU interpreter
# (tests/golden/make_golden_aux.py). BF16 tensors are stored as their uint16 bit patterns. The
# interpreter narrows FP32 to BF16 by dropping bits where the compiled kernel rounds to nearest even,
# so bit-exact cases use values whose results are exact in BF16, and the random-valued ones allow the
# one BF16 step that the two narrowing rules can differ by.
AUX_COPY_CASES = ('copy_grow', 'copy_shrink', 'copy_same', 'biased_grow', 'biased_shrink', 'biased_same')
AUX_BIAS_CASES = ('bias_one_part_bf16', 'bias_one_part_f32_acc', 'bias_parts_bf16_acc', 'bias_parts_f32',
                  'bias_many_parts_f32_acc')


def aux_tensor(z, key):
    a = z[key]
    return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16) if a.dtype == np.uint16 else torch.from_numpy(a)


def aux_copy_case(z, name):
    count = sum(1 for key in z.files if key.startswith(f'{name}.in'))
    sources = tuple(aux_tensor(z, f'{name}.in{i}') for i in range(count))
    wanted = tuple(aux_tensor(z, f'{name}.out{i}') for i in range(count))
    kwargs = {}
    if f'{name}.bias' in z.files:
        kwargs = dict(bias=aux_tensor(z, f'{name}.bias'), head_dim=int(z[f'{name}.head_dim']),
                      head_offset=int(z[f'{name}.head_offset']))
    return sources, wanted, int(z[f'{name}.peers']), int(z[f'{name}.rows']), kwargs


@pytest.mark.parametrize('name', AUX_COPY_CASES)
def test_oracle_row_copy_is_the_reference_kernels_output_bit_for_bit(name):
    from oracle.ulysses_oracle import resize_rank_rows_ref
    z = np.load(os.path.join(GOLDEN, 'aux_kernels.npz'))
    sources, wanted, peers, rows, kwargs = aux_copy_case(z, name)
    got = resize_rank_rows_ref(sources, peers, rows, **kwargs)
    for i, (a, w) in enumerate(zip(got, wanted)):
        assert a.shape == w.shape and torch.equal(a.view(torch.int16), w.view(torch.int16)), f'{name} tensor {i}'


def test_oracle_biased_row_copy_rounds_where_the_interpreter_truncates():
    """Random values: the oracle rounds the FP32 sum to nearest even (what the reference's own check
    demands, tests/row_copy_driver.py:40-57), the interpreted kernel drops the low bits. Wherever the
    FP32 sum is exact in BF16 they are equal; elsewhere the recorded value is the next BF16 towards
    zero or the oracle's own; rows past the input are zero in both."""
    from oracle.ulysses_oracle import resize_rank_rows_ref
    z = np.load(os.path.join(GOLDEN, 'aux_kernels.npz'))
    sources, wanted, peers, rows, kwargs = aux_copy_case(z, 'biased_random')
    got = resize_rank_rows_ref(sources, peers, rows, **kwargs)
    in_rows = sources[0].shape[0] // peers
    for a, w in zip(got, wanted):
        a_bits, w_bits = a.view(torch.int16).int() & 0xffff, w.view(torch.int16).int() & 0xffff
        assert ((a_bits == w_bits) | (a_bits == w_bits + 1)).all()   # same sign, magnitude at most one step up
        assert (a_bits != w_bits).any()                              # the case does exercise the rounding
        for t in (a, w):
            assert not t.reshape(peers, rows, -1)[:, in_rows:].any()


@pytest.mark.parametrize('name', AUX_BIAS_CASES)
def test_oracle_bias_gradient_against_the_reference_kernels_output(name):
    """The reference adds in FP32, 256 rows per partial sum, the oracle in FP64: they agree within
    the reference's own bound 4 * eps * sum|x| (tests/bias_grad_driver.py:23-46 of the reference) plus,
    for a BF16 result, one rounding. The quarter-integer case has exact FP32 sums: bit-exact."""
    from oracle.ulysses_oracle import reduce_bias_grad_ref
    z = np.load(os.path.join(GOLDEN, 'aux_kernels.npz'))
    dy, previous, wanted = (aux_tensor(z, f'{name}.{key}') for key in ('dy', 'previous', 'out'))
    accumulate = bool(z[f'{name}.accumulate'])
    got = reduce_bias_grad_ref(dy, wanted.dtype, previous=previous if accumulate else None)
    if name == 'bias_many_parts_f32_acc':
        # exact column sums, then one FP32 addition of the previous value: nothing depends on the order
        assert torch.equal(wanted, dy.double().sum(0).float() + previous)
        assert torch.equal(got, wanted)
    bound = 4 * torch.finfo(torch.float32).eps * (dy.double().abs().sum(0) + previous.double().abs() * accumulate)
    if wanted.dtype == torch.bfloat16:
        bound = bound + wanted.double().abs() * 2.0 ** -7   # rounded here, truncated by the interpreter
    assert ((got.double() - wanted.double()).abs() <= bound + 1e-30).all(), name
