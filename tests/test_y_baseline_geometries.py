"""GPU parity at the geometries the benchmark configurations name, on a single-rank CP group:

  C2/C3  hidden 4096, 32 heads, 16384 local tokens, BF16, QKV and output projections
  C4     hidden 3072, 24 heads, QKVG with bias on both projections, odd token counts drawn from
         [4097, 8191] under one workspace of capacity 8192
  C5     hidden 5120, 40 heads, MXFP8, activations with 0.1 % outliers (x 1e3) and all-zero
         32-groups, FP32 main_grad (4096 local tokens here instead of 32768: the numpy MXFP8 oracle
         is the slow side)

The full-size outputs are too large for the CPU oracle to recompute in seconds, so each tensor is
compared on a sample that the oracle can afford: whole 256-row blocks of the row-wise results
(first, middle and the ragged last block) and whole 256 x 256 tiles of the weight gradients, which
sum over every token. Tolerance as everywhere: max error <= 1e-2 of the reference's largest
magnitude and relative Frobenius error <= 2e-3 for BF16 results; the MXFP8 quantized copy and its
scales bit-exact against the standalone quantizer. The same geometries at CP = 8 (4, 3 and 5 heads
per rank) go through the one-GPU rank emulation of tests/test_emulated_ranks.py at the end of this
file, and through the multi-GPU driver. Also here: the bias gradient of a matrix larger than 4 GiB.

The file sorts after the tests of the small shapes on purpose: a run that stops at the first
failure has then already been through every kernel on the sizes where a mismatch is cheap to read.
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import test_emulated_ranks as emulated  # noqa: E402

from oracle import mxfp8_oracle as mx
from oracle.ulysses_oracle import UlyssesOracle

gpu = pytest.mark.gpu
DEV = 'cuda:0'
BF = torch.bfloat16


def close(actual, expected, what):
    actual, expected = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert actual.shape == expected.shape, f'{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}'
    scale = expected.abs().max().clamp_min(1e-6)
    assert (actual - expected).abs().max() <= 1e-2 * scale, f'{what}: max error'
    assert torch.linalg.norm(actual - expected) <= 2e-3 * torch.linalg.norm(expected) + 1e-6, f'{what}: Frobenius'


def sampled_rows(tokens, block=256):
    """Row indices of the first, a middle and the last (possibly ragged) block of `block` rows."""
    last = (tokens - 1) // block * block
    starts = sorted({0, (tokens // 2) // block * block, last})
    return torch.cat([torch.arange(s, min(s + block, tokens)) for s in starts])


def sampled_tiles(rows, cols, tile=256):
    """Corners and centre of a [rows, cols] weight gradient, as (row0, col0) of 256 x 256 tiles."""
    r_last, c_last = rows - tile, cols - tile
    return [(0, 0), (r_last, c_last), ((rows // 2) // tile * tile, (cols // 2) // tile * tile), (0, c_last)]


def inputs(hidden, heads, tokens, segments, with_bias, seed, weight_scale=None):
    g = torch.Generator().manual_seed(seed)
    d = hidden // heads
    scale = hidden ** -0.5 if weight_scale is None else weight_scale
    return dict(
        x=torch.randn(tokens, hidden, generator=g).to(BF),
        wq=(torch.randn(segments * hidden, hidden, generator=g) * scale).to(BF),
        wo=(torch.randn(hidden, hidden, generator=g) * scale).to(BF),
        bq=torch.randn(segments * hidden, generator=g).mul(0.02).to(BF) if with_bias else None,
        bo=torch.randn(hidden, generator=g).mul(0.02).to(BF) if with_bias else None,
        grads=tuple(torch.randn(tokens, heads, d, generator=g).to(BF) for _ in range(segments)),
        o=torch.randn(tokens, heads, d, generator=g).to(BF),
        dy=torch.randn(tokens, hidden, generator=g).to(BF))


def run_modules(case, ws, hidden, heads, gate, bias_in_gemm, main_grad=False):
    from fused_gemm_a2a import FusedOutputProjection, FusedQKVProjection
    on_gpu = DEV != 'cpu'
    params = {name: (None if case[name] is None else torch.nn.Parameter(case[name].to(DEV)))
              for name in ('wq', 'wo', 'bq', 'bo')}
    seeds = {}
    if main_grad:
        g = torch.Generator().manual_seed(5)
        for name in ('wq', 'wo'):
            seeds[name] = torch.randn(params[name].shape, generator=g).to(DEV)
            params[name].main_grad = seeds[name].clone()
    qkv = FusedQKVProjection(hidden, heads, weight=params['wq'], bias=params['bq'], gate=gate,
                             bias_in_gemm=bias_in_gemm)
    proj = FusedOutputProjection(hidden, heads, weight=params['wo'], bias=params['bo'])
    x = case['x'].to(DEV).requires_grad_()
    outs = qkv(x, ws)
    torch.autograd.backward(list(outs), [t.to(DEV) for t in case['grads']])
    o = case['o'].to(DEV).requires_grad_()
    y = proj(o, ws)
    y.backward(case['dy'].to(DEV))
    if on_gpu:
        torch.cuda.synchronize()
    ws.comm.check_status()
    return dict(outs=outs, dx=x.grad, y=y, do=o.grad, params=params, seeds=seeds)


def check_bf16_case(case, got, hidden, heads, segments, bias_in_gemm, with_bias):
    """Row samples through the oracle's projections (rows are independent at CP = 1), weight-gradient
    tiles from the oracle's dY layout (receive-buffer column order = weight-row order)."""
    tokens = case['x'].shape[0]
    oracle = UlyssesOracle(1, hidden, heads, segments, case['wq'], case['bq'], case['wo'], case['bo'],
                           bias_in_gemm=bias_in_gemm)
    rows = sampled_rows(tokens)
    on_gpu = rows.to(DEV)
    for name, out, want in zip('qkvg', got['outs'], oracle.qkv_forward([case['x'][rows]])[0]):
        assert out.shape == (tokens, heads, hidden // heads)
        close(out[on_gpu], want, f'{name} rows')
    dx, _, _ = oracle.qkv_backward([case['x'][rows]], [tuple(g[rows] for g in case['grads'])])[0]
    close(got['dx'][on_gpu], dx, 'dx rows')
    close(got['y'][on_gpu], oracle.out_forward([case['o'][rows]])[0], 'y rows')
    dos, _ = oracle.out_backward([case['o'][rows]], [case['dy'][rows]])
    close(got['do'][on_gpu], dos[0], 'dO rows')
    dy_qkv = oracle.qkv_recv_buffer([case['grads']], 0)[:tokens].float()     # [tokens, segments*H], weight-row order
    x32, dy32, o32 = case['x'].float(), case['dy'].float(), case['o'].reshape(tokens, hidden).float()
    dwq, dwo = got['params']['wq'].grad, got['params']['wo'].grad
    for r0, c0 in sampled_tiles(segments * hidden, hidden):
        close(dwq[r0:r0 + 256, c0:c0 + 256], dy_qkv[:, r0:r0 + 256].t() @ x32[:, c0:c0 + 256], f'dW_qkv tile {r0},{c0}')
    for r0, c0 in sampled_tiles(hidden, hidden):
        close(dwo[r0:r0 + 256, c0:c0 + 256], dy32[:, r0:r0 + 256].t() @ o32[:, c0:c0 + 256], f'dW_o tile {r0},{c0}')
    if with_bias:
        close(got['params']['bq'].grad, dy_qkv.sum(0).to(BF), 'dbias_qkv')
        close(got['params']['bo'].grad, dy32.sum(0).to(BF), 'dbias_o')


@gpu
def test_c2_c3_bf16_hidden_4096_32_heads_16384_tokens(cp1):
    from fused_gemm_a2a import FusedGemmA2AWorkspace
    hidden, heads, tokens = 4096, 32, 16384
    case = inputs(hidden, heads, tokens, 3, False, seed=2, weight_scale=1 / 64)
    ws = FusedGemmA2AWorkspace(hidden, heads, tokens)
    got = run_modules(case, ws, hidden, heads, gate=False, bias_in_gemm=False)
    check_bf16_case(case, got, hidden, heads, 3, False, False)


@gpu
def test_c4_gate_and_bias_hidden_3072_24_heads_odd_token_counts(cp1):
    """Three odd token counts from [4097, 8191] (seeded draw) share one workspace of capacity 8192;
    the bias is added by the GEMM epilogue for the first count and by the copy kernel for the others."""
    from fused_gemm_a2a import FusedGemmA2AWorkspace
    hidden, heads = 3072, 24
    draw = torch.Generator().manual_seed(4)
    counts = [int(torch.randint(2048, 4096, (1,), generator=draw)) * 2 + 1 for _ in range(3)]
    assert all(4097 <= m <= 8191 and m % 2 for m in counts)
    ws = FusedGemmA2AWorkspace(hidden, heads, 8192, gate=True)
    for index, tokens in enumerate(counts):
        case = inputs(hidden, heads, tokens, 4, True, seed=40 + index, weight_scale=1 / 64)
        got = run_modules(case, ws, hidden, heads, gate=True, bias_in_gemm=index == 0)
        check_bf16_case(case, got, hidden, heads, 4, index == 0, True)


def bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def mm(a, b):
    """bf16(a @ b^T) with both operands quantized to MXFP8 along their second axis (exact products)."""
    return torch.from_numpy(mx.mx_matmul(bits(a), bits(b))).to(BF)


@gpu
def test_c5_mxfp8_hidden_5120_40_heads_outliers_zero_groups_main_grad(cp1):
    from fused_gemm_a2a import FusedGemmA2AWorkspace
    from fused_gemm_a2a_kernels import mxfp8_quantize
    hidden, heads, tokens, d = 5120, 40, 4096, 128
    case = inputs(hidden, heads, tokens, 3, False, seed=5)
    g = torch.Generator().manual_seed(55)
    x = case['x'].float()
    x = torch.where(torch.rand(tokens, hidden, generator=g) < 0.001, x * 1e3, x)
    x.view(-1, 4096)[:, 64:96] = 0                      # one all-zero 32-group per 4096 elements
    case['x'] = x.to(BF)
    ws = FusedGemmA2AWorkspace(hidden, heads, tokens, precision='mxfp8')
    got = run_modules(case, ws, hidden, heads, gate=False, bias_in_gemm=False, main_grad=True)
    # Receive-side quantizer: after the output projection's forward+backward the QKV receive buffer
    # still holds dY of the QKV backward; its quantized copy must be what the standalone quantizer writes.
    view = ws._view(tokens, 3)
    q_ref, sf_ref = mxfp8_quantize(view.recv, k_multiple=128)
    torch.cuda.synchronize()
    assert torch.equal(view.mx_recv.view(torch.uint8), q_ref.view(torch.uint8)[:view.capacity])
    assert torch.equal(view.mx_scale, sf_ref[:view.mx_scale.numel()])

    rows = sampled_rows(tokens, block=128)              # the float64 numpy product is the slow side
    on_gpu = rows.to(DEV)
    wq, wo = case['wq'], case['wo']
    full = mm(case['x'][rows], wq).view(len(rows), heads, 3, d)
    for i, out in enumerate(got['outs']):
        close(out[on_gpu], full[:, :, i, :], f'segment {i} rows')
    dyq = torch.stack(case['grads'], dim=2).reshape(tokens, 3 * hidden)      # weight-row order
    close(got['dx'][on_gpu], mm(dyq[rows], wq.t()), 'dx rows')
    o_seq = case['o'].reshape(tokens, hidden)
    close(got['y'][on_gpu], mm(o_seq[rows], wo), 'y rows')
    close(got['do'][on_gpu], mm(case['dy'][rows], wo.t()).view(len(rows), heads, d), 'dO rows')
    # weight gradients went into the FP32 main_grad (nothing else may have changed it)
    for name, left, right, shape in (('wq', dyq, case['x'], (3 * hidden, hidden)), ('wo', case['dy'], o_seq, (hidden, hidden))):
        param = got['params'][name]
        assert param.grad_added_to_main_grad
        added = (param.main_grad - got['seeds'][name]).cpu()
        for r0, c0 in sampled_tiles(*shape):
            want = torch.from_numpy(mx.mx_matmul(bits(left[:, r0:r0 + 256].t()), bits(right[:, c0:c0 + 256].t()))).float()
            tile = added[r0:r0 + 256, c0:c0 + 256]
            assert (tile - want).abs().max() <= 1e-3 * want.abs().max(), f'dW_{name} tile {r0},{c0}'


# ---- the same geometries at CP = 8 on one GPU: 4, 3 and 5 heads per rank -------------------------
@gpu
@pytest.mark.parametrize('p,hidden,heads,tokens,segments,bias_in_gemm', [
    (8, 4096, 32, 129, 3, False), (8, 3072, 24, 77, 4, True), (8, 5120, 40, 129, 3, False)])
def test_cp8_push_lands_in_the_right_peer_tiles(native, p, hidden, heads, tokens, segments, bias_in_gemm):
    emulated.test_push_lands_in_the_right_peer_tiles(native, p, hidden, heads, tokens, segments, bias_in_gemm)


@gpu
@pytest.mark.parametrize('p,hidden,heads,tokens', [(8, 4096, 32, 129), (8, 3072, 24, 77), (8, 5120, 40, 31)])
def test_cp8_output_dgrad_push_routes_columns_to_their_owner(native, p, hidden, heads, tokens):
    emulated.test_output_dgrad_push_routes_columns_to_their_owner(native, p, hidden, heads, tokens)


@gpu
@pytest.mark.parametrize('p,hidden,heads,tokens,num_in', [
    (8, 4096, 32, 129, 3), (8, 4096, 32, 129, 1), (8, 3072, 24, 77, 4), (8, 3072, 24, 77, 1),
    (8, 5120, 40, 129, 3), (8, 5120, 40, 33, 1)])
def test_cp8_receive_transport_and_gemm(native, p, hidden, heads, tokens, num_in):
    emulated.test_receive_transport_and_gemm(native, p, hidden, heads, tokens, num_in)


# ---- a matrix larger than 4 GiB -------------------------------------------------------------------
@gpu
def test_reduce_bias_grad_rows_beyond_four_gibibytes(native):
    """The last row of a [131073, 16384] BF16 matrix starts past 2^32 bytes and past 2^31 elements:
    row offsets must be 64-bit (reference tests/bias_grad_driver.py:54-59). Exact: one row of ones,
    all others zero. Also through the entry point with built-in scratch (513 x 16384 partial sums
    do not fit its array, so it must refuse rather than wrap)."""
    from fused_gemm_a2a_kernels import reduce_bias_grad
    rows, width = 131073, 16384
    dy = torch.zeros(rows, width, dtype=torch.bfloat16, device=DEV)
    dy[-1] = 1
    out = reduce_bias_grad(dy, torch.empty(width, dtype=torch.float32, device=DEV))
    assert torch.equal(out, torch.ones_like(out))
    dy[-1, 5] = 3
    dy[70000, 5] = -8
    out = reduce_bias_grad(dy, torch.zeros(width, dtype=torch.bfloat16, device=DEV))
    expected = torch.ones(width)
    expected[5] = -5
    assert torch.equal(out.float().cpu(), expected)
    rc = native.fga_bias_grad_static(dy.data_ptr(), rows, width, out.data_ptr(), 0, 0,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and b'scratch floats' in native.fga_last_error()


# ---- the checks themselves, on the CPU -----------------------------------------------------------
def _simulated_worker(queue):
    """This file's helpers (module run, row sampling, tile sampling, expected values) over the
    simulated library on one CPU rank, at a small QKVG + bias geometry with a ragged last row block:
    what the GPU tests above do, minus the GPU."""
    import torch.distributed as dist
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    for path in (here, root, os.path.join(root, 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT='29589')
    dist.init_process_group('gloo', rank=0, world_size=1)
    import abi_simulator
    import fused_gemm_a2a as fused
    import test_y_baseline_geometries as checks
    checks.DEV = 'cpu'
    _, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    problems = []
    try:
        hidden, heads = 768, 6
        ws = fused.FusedGemmA2AWorkspace(hidden, heads, 1024, gate=True)
        for index, tokens in enumerate((777, 513)):
            case = checks.inputs(hidden, heads, tokens, 4, True, seed=40 + index, weight_scale=1 / 32)
            got = checks.run_modules(case, ws, hidden, heads, gate=True, bias_in_gemm=index == 0)
            try:
                checks.check_bf16_case(case, got, hidden, heads, 4, index == 0, True)
            except AssertionError as error:
                problems.append(f'tokens={tokens}: {error}')
            # and the checker does object: a weight gradient with two head blocks swapped
            broken = got['params']['wq'].grad.clone()
            broken[:128], broken[128:256] = got['params']['wq'].grad[128:256], got['params']['wq'].grad[:128]
            got['params']['wq'].grad = broken
            try:
                checks.check_bf16_case(case, got, hidden, heads, 4, index == 0, True)
                problems.append('swapped weight-gradient blocks were accepted')
            except AssertionError:
                pass
    finally:
        undo()
    queue.put(problems)
    dist.destroy_process_group()


def test_the_sampled_checks_run_and_discriminate_on_the_simulated_library():
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    proc = ctx.Process(target=_simulated_worker, args=(queue,))
    proc.start()
    try:
        problems = queue.get(timeout=600)
    finally:
        proc.join(timeout=60)
        if proc.is_alive():
            proc.terminate()
    assert problems == []
    assert sampled_rows(8191).tolist()[::255][:3] == [0, 255, 3840 + 254] and len(sampled_rows(8191)) == 767
    assert len(sampled_rows(100)) == 100 and sampled_tiles(12288, 3072)[1] == (12032, 2816)
