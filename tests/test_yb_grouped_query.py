"""GPU parity of grouped-query attention (fewer key/value heads than query heads), an addition over
the reference's fused modules, which reject it (BF16 and MXFP8); expected values come from the grouped-query oracle,
pinned by the reference's unfused modules run with num_kv_heads < num_heads
(tests/test_oracle_golden.py).

Through the C ABI with the ranks emulated on one GPU (push launches never wait; the receive kernel
runs its pushers for every rank first, then every rank's GEMM on complete counters), and through
the public modules on a single-rank CP group. Transport bit-exact, GEMM results within max error
1e-2 of scale and Frobenius 2e-3.
"""
import pytest
import torch

import _fga_native as nat
from oracle.ulysses_oracle import GroupedQueryOracle

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
TIMEOUT_NS = 5_000_000_000
BF = torch.bfloat16


def close(actual, expected, what):
    actual, expected = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert actual.shape == expected.shape, f'{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}'
    scale = expected.abs().max().clamp_min(1e-6)
    assert (actual - expected).abs().max() <= 1e-2 * scale, f'{what}: max error'
    assert torch.linalg.norm(actual - expected) <= 2e-3 * torch.linalg.norm(expected) + 1e-6, f'{what}: Frobenius'


def table(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=DEV)


def geometry(heads, kv_heads, gate, p):
    kinds = 4 if gate else 3
    rows = (heads * (2 if gate else 1) + 2 * kv_heads) * 128
    widths = [(heads if kind in (0, 3) else kv_heads) // p * 128 for kind in range(kinds)]
    return kinds, rows, widths


@pytest.mark.parametrize('p,heads,kv_heads,gate,tokens,with_bias', [
    (1, 4, 2, False, 300, False), (2, 8, 2, True, 129, True), (4, 32, 8, False, 77, False), (8, 32, 8, False, 129, True),
    (2, 6, 2, False, 256, False)])
def test_push_lands_in_the_right_buffers_of_the_right_peers(native, p, heads, kv_heads, gate, tokens, with_bias):
    hidden = heads * 128
    kinds, rows, widths = geometry(heads, kv_heads, gate, p)
    g = torch.Generator().manual_seed(p * 1000 + tokens)
    capacity = (tokens + 255) // 256 * 256
    weight = (torch.randn(rows, hidden, generator=g) / hidden ** 0.5).to(BF)
    bias = torch.randn(rows, generator=g).to(BF) if with_bias else None
    xs = [torch.randn(tokens, hidden, generator=g).to(BF) for _ in range(p)]
    buffers = [[torch.full((p * capacity, widths[kind]), 5.0, dtype=BF, device=DEV) for kind in range(kinds)]
               for _ in range(p)]
    tables = [table([buffers[d][kind] for d in range(p)]) for kind in range(kinds)]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    w_dev = weight.to(DEV)
    b_dev = bias.to(DEV) if with_bias else None
    for r in range(p):
        x = xs[r].to(DEV)
        rc = native.fga_gemm_push_gqa(x.data_ptr(), tokens, hidden, capacity, w_dev.data_ptr(),
                                      0 if b_dev is None else b_dev.data_ptr(), kv_heads, heads // kv_heads, int(gate),
                                      nat.ptr_array([t.data_ptr() for t in tables]), capacity, r, p,
                                      status.data_ptr(), TIMEOUT_NS, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    oracle = GroupedQueryOracle(p, hidden, heads, kv_heads, gate, weight_qkv=weight, bias_qkv=bias, bias_in_gemm=with_bias)
    want = oracle.qkv_heads_buffers(xs, capacity)
    for d in range(p):
        for kind in range(kinds):
            close(buffers[d][kind], want[d][kind], f'dest {d} kind {kind}')


@pytest.mark.parametrize('p,heads,kv_heads,gate,tokens', [
    (1, 4, 2, False, 300), (2, 8, 2, True, 129), (4, 32, 8, False, 77), (8, 32, 8, True, 129), (2, 6, 2, False, 1)])
def test_receive_transport_and_dgrad(native, p, heads, kv_heads, gate, tokens):
    from fused_gemm_a2a_kernels import push_split
    hidden = heads * 128
    kinds, k, widths = geometry(heads, kv_heads, gate, p)
    g = torch.Generator().manual_seed(p * 77 + tokens)
    capacity = (tokens + 255) // 256 * 256
    weight = (torch.randn(k, hidden, generator=g) / k ** 0.5).to(BF)
    inputs = [tuple(torch.randn(p * tokens, widths[kind] // 128, 128, generator=g).to(BF) for kind in range(kinds))
              for _ in range(p)]
    recvs = [torch.full((capacity, k), 9.0, dtype=BF, device=DEV) for _ in range(p)]
    counters = [torch.zeros(capacity // 128, dtype=torch.int32, device=DEV) for _ in range(p)]
    outs = [torch.full((capacity, hidden), float('nan'), dtype=BF, device=DEV) for _ in range(p)]
    t_recv, t_cnt = table(recvs), table(counters)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    w_dev = weight.to(DEV)
    dev_inputs = [[t.to(DEV).flatten(1).contiguous() for t in inputs[r]] for r in range(p)]
    split = push_split(kinds * hidden, p, kinds)
    for roles in (2, 1):
        for r in range(p):
            rc = native.fga_gemm_recv_gqa(recvs[r].data_ptr(), capacity, w_dev.data_ptr(), hidden, outs[r].data_ptr(),
                                          t_recv.data_ptr(), t_cnt.data_ptr(), counters[r].data_ptr(),
                                          nat.ptr_array([t.data_ptr() for t in dev_inputs[r]]), kv_heads,
                                          heads // kv_heads, int(gate), tokens, split, r, p, roles, None,
                                          status.data_ptr(), TIMEOUT_NS, torch.cuda.current_stream().cuda_stream)
            assert rc == 0, native.fga_last_error()
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        if roles == 2:
            for r in range(p):
                assert counters[r].tolist() == [p * kinds * split] * (capacity // 128)
    oracle = GroupedQueryOracle(p, hidden, heads, kv_heads, gate)
    for r in range(p):
        want = oracle.qkv_recv_buffer(inputs, r, capacity)
        assert torch.equal(recvs[r].cpu(), want), f'rank {r}: receive buffer differs'
        close(outs[r], want.float() @ weight.float(), f'rank {r} dX')


@pytest.mark.parametrize('heads,kv_heads,gate,with_bias,bias_in_gemm,tokens', [
    (8, 2, False, False, False, 300), (8, 4, True, True, False, 777), (4, 1, False, True, True, 129)])
def test_modules_match_the_grouped_query_oracle(cp1, heads, kv_heads, gate, with_bias, bias_in_gemm, tokens):
    from fused_gemm_a2a import FusedGemmA2AWorkspace, FusedOutputProjection, FusedQKVProjection
    hidden = heads * 128
    kinds, rows, widths = geometry(heads, kv_heads, gate, 1)
    g = torch.Generator().manual_seed(tokens + heads)
    wq = (torch.randn(rows, hidden, generator=g) / hidden ** 0.5).to(BF)
    wo = (torch.randn(hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
    bq = torch.randn(rows, generator=g).mul(0.5).to(BF) if with_bias else None
    x = torch.randn(tokens, hidden, generator=g).to(BF)
    grads = tuple(torch.randn(tokens, widths[kind] // 128, 128, generator=g).to(BF) for kind in range(kinds))
    o = torch.randn(tokens, heads, 128, generator=g).to(BF)
    dy = torch.randn(tokens, hidden, generator=g).to(BF)
    ws = FusedGemmA2AWorkspace(hidden, heads, 1024, gate=gate, num_kv_heads=kv_heads)
    wq_p, wo_p = torch.nn.Parameter(wq.to(DEV)), torch.nn.Parameter(wo.to(DEV))
    bq_p = torch.nn.Parameter(bq.to(DEV)) if with_bias else None
    qkv = FusedQKVProjection(hidden, heads, kv_heads, weight=wq_p, bias=bq_p, gate=gate, bias_in_gemm=bias_in_gemm)
    proj = FusedOutputProjection(hidden, heads, weight=wo_p)
    x_d = x.to(DEV).requires_grad_()
    outs = qkv(x_d, ws)
    torch.autograd.backward(list(outs), [t.to(DEV) for t in grads])
    o_d = o.to(DEV).requires_grad_()
    y = proj(o_d, ws)
    y.backward(dy.to(DEV))
    torch.cuda.synchronize()
    ws.comm.check_status()
    oracle = GroupedQueryOracle(1, hidden, heads, kv_heads, gate, weight_qkv=wq, bias_qkv=bq, weight_out=wo,
                                bias_in_gemm=bias_in_gemm)
    for name, got, want in zip('qkvg', outs, oracle.qkv_forward([x])[0]):
        close(got, want, name)
    dx, dwq, dbq = oracle.qkv_backward([x], [grads])[0]
    close(x_d.grad, dx, 'dx')
    close(wq_p.grad, dwq, 'dW_qkv')
    if with_bias:
        close(bq_p.grad, dbq, 'dbias_qkv')
    close(y, oracle.out_forward([o])[0], 'y')
    dos, ((dwo, _),) = oracle.out_backward([o], [dy])
    close(o_d.grad, dos[0], 'dO')
    close(wo_p.grad, dwo, 'dW_o')
    with pytest.raises(ValueError, match='QKV/QKVG mode'):
        FusedQKVProjection(hidden, heads, weight=torch.nn.Parameter(torch.empty(3 * hidden, hidden, dtype=BF, device=DEV)))(
            x_d.detach(), ws)


# ---- MXFP8 operands with the grouped layout ------------------------------------------------------
def _mx_mm(a, b, acc_dtype):
    """The oracle's GEMM a @ b with both operands quantized to MXFP8 along the reduction axis and the
    exact dequantized values multiplied (oracle/mxfp8_oracle.py)."""
    import numpy as np
    from oracle import mxfp8_oracle as mx

    def bits(t):
        return t.to(BF).contiguous().view(torch.int16).numpy().view(np.uint16)
    return torch.from_numpy(mx.mx_matmul(bits(a), bits(b.t()))).to(acc_dtype)


@pytest.mark.parametrize('heads,kv_heads,gate,with_bias,tokens', [(4, 2, False, False, 300), (8, 2, True, True, 129)])
def test_mxfp8_modules_match_the_grouped_query_oracle(cp1, monkeypatch, heads, kv_heads, gate, with_bias, tokens):
    """precision='mxfp8' with fewer key/value heads: the grouped push and receive launches with
    block-scaled operands; the receive-side quantizer's bytes equal the standalone quantizer's."""
    from fused_gemm_a2a import FusedGemmA2AWorkspace, FusedOutputProjection, FusedQKVProjection
    from fused_gemm_a2a_kernels import mxfp8_quantize
    from oracle import ulysses_oracle
    monkeypatch.setattr(ulysses_oracle, '_mm', _mx_mm)
    hidden = heads * 128
    kinds, rows, widths = geometry(heads, kv_heads, gate, 1)
    g = torch.Generator().manual_seed(tokens + heads)
    wq = (torch.randn(rows, hidden, generator=g) / hidden ** 0.5).to(BF)
    wo = (torch.randn(hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
    bq = torch.randn(rows, generator=g).mul(0.5).to(BF) if with_bias else None
    x = torch.randn(tokens, hidden, generator=g).to(BF)
    grads = tuple(torch.randn(tokens, widths[kind] // 128, 128, generator=g).to(BF) for kind in range(kinds))
    o = torch.randn(tokens, heads, 128, generator=g).to(BF)
    dy = torch.randn(tokens, hidden, generator=g).to(BF)
    ws = FusedGemmA2AWorkspace(hidden, heads, 512, gate=gate, num_kv_heads=kv_heads, precision='mxfp8')
    wq_p, wo_p = torch.nn.Parameter(wq.to(DEV)), torch.nn.Parameter(wo.to(DEV))
    bq_p = torch.nn.Parameter(bq.to(DEV)) if with_bias else None
    qkv = FusedQKVProjection(hidden, heads, kv_heads, weight=wq_p, bias=bq_p, gate=gate)
    proj = FusedOutputProjection(hidden, heads, weight=wo_p)
    x_d = x.to(DEV).requires_grad_()
    outs = qkv(x_d, ws)
    torch.autograd.backward(list(outs), [t.to(DEV) for t in grads])
    view = ws._view(tokens, kinds)
    q_ref, sf_ref = mxfp8_quantize(view.recv, k_multiple=128)
    torch.cuda.synchronize()
    assert torch.equal(view.mx_recv.view(torch.uint8), q_ref.view(torch.uint8)[:view.capacity])
    assert torch.equal(view.mx_scale, sf_ref[:view.mx_scale.numel()])
    o_d = o.to(DEV).requires_grad_()
    y = proj(o_d, ws)
    y.backward(dy.to(DEV))
    torch.cuda.synchronize()
    ws.comm.check_status()
    oracle = GroupedQueryOracle(1, hidden, heads, kv_heads, gate, weight_qkv=wq, bias_qkv=bq, weight_out=wo)
    for name, got, want in zip('qkvg', outs, oracle.qkv_forward([x])[0]):
        close(got, want, name)
    dx, dwq, dbq = oracle.qkv_backward([x], [grads])[0]
    close(x_d.grad, dx, 'dx')
    close(wq_p.grad, dwq, 'dW_qkv')
    if with_bias:
        close(bq_p.grad, dbq, 'dbias_qkv')
    close(y, oracle.out_forward([o])[0], 'y')
    dos, ((dwo, _),) = oracle.out_backward([o], [dy])
    close(o_d.grad, dos[0], 'dO')
    close(wo_p.grad, dwo, 'dW_o')
