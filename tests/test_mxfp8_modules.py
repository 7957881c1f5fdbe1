"""GPU parity of the public modules with precision="mxfp8" on a single-rank CP group.

Expected values come from the CPU oracle: every GEMM quantizes both operands along its own
reduction axis (E4M3 + E8M0/32, oracle/mxfp8_oracle.py), multiplies the exact dequantized values
and rounds once to BF16. E8M0 scales and E4M3 codes written by the receive-side quantizer warps
are compared bit-exactly with the standalone quantizer; BF16 outputs and gradients within max
error 1e-2 of scale and Frobenius 2e-3.
"""
import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as mx

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
BF = torch.bfloat16


def bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def mm(a, b):
    """bf16(a @ b^T) with both operands quantized along their second axis."""
    return torch.from_numpy(mx.mx_matmul(bits(a), bits(b))).to(BF)


def close(actual, expected, what):
    actual, expected = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert actual.shape == expected.shape, what
    scale = expected.abs().max().clamp_min(1e-6)
    assert (actual - expected).abs().max() <= 1e-2 * scale, f'{what}: max error'
    assert torch.linalg.norm(actual - expected) <= 2e-3 * torch.linalg.norm(expected) + 1e-6, f'{what}: Frobenius'


@pytest.mark.parametrize('tokens,gate', [(300, False), (129, True), (512, False)])
def test_mxfp8_projections_match_oracle(cp1, tokens, gate):
    from fused_gemm_a2a import FusedGemmA2AWorkspace, FusedOutputProjection, FusedQKVProjection
    from fused_gemm_a2a_kernels import mxfp8_quantize
    hidden, heads, d = 512, 4, 128
    s = 4 if gate else 3
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, hidden, generator=g)
    x = torch.where(torch.rand(tokens, hidden, generator=g) < 0.001, x * 1e3, x).to(BF)
    x[0, 32:64] = 0
    wq = (torch.randn(s * hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
    wo = (torch.randn(hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
    grads = tuple(torch.randn(tokens, heads, d, generator=g).to(BF) for _ in range(s))
    o = torch.randn(tokens, heads, d, generator=g).to(BF)
    dy = torch.randn(tokens, hidden, generator=g).to(BF)

    ws = FusedGemmA2AWorkspace(hidden, heads, 512, gate=gate, precision='mxfp8')
    wq_d, wo_d = wq.to(DEV).requires_grad_(), wo.to(DEV).requires_grad_()
    qkv = FusedQKVProjection(hidden, heads, weight=wq_d, gate=gate)
    proj = FusedOutputProjection(hidden, heads, weight=wo_d)
    x_d, o_d = x.to(DEV).requires_grad_(), o.to(DEV).requires_grad_()
    outs = qkv(x_d, ws)
    dx, dwq = torch.autograd.grad(outs, [x_d, wq_d], [t.to(DEV) for t in grads])
    # the receive buffer still holds dY in BF16; the quantizer warps must have written exactly what
    # the standalone quantizer writes for the same buffer (reference tests/mxfp8_driver.py:127-135)
    view = ws._view(tokens, s)
    q_ref, sf_ref = mxfp8_quantize(view.recv, k_multiple=128)
    torch.cuda.synchronize()
    assert torch.equal(view.mx_recv.view(torch.uint8), q_ref.view(torch.uint8)[:view.capacity])
    assert torch.equal(view.mx_scale, sf_ref[:view.mx_scale.numel()])
    y = proj(o_d, ws)
    do, dwo = torch.autograd.grad(y, [o_d, wo_d], dy.to(DEV))
    torch.cuda.synchronize()
    ws.comm.check_status()

    full = mm(x, wq).view(tokens, heads, s, d)
    for i, got in enumerate(outs):
        close(got, full[:, :, i, :], f'segment {i}')
    dyq = torch.stack(grads, dim=2).reshape(tokens, s * hidden)   # [token][head][segment][d] = weight-row order
    close(dx, mm(dyq, wq.t()), 'dx')
    close(dwq, mm(dyq.t(), x.t()), 'dW_qkv')
    o_seq = o.reshape(tokens, hidden)
    close(y, mm(o_seq, wo), 'y')
    close(do, mm(dy, wo.t()).view(tokens, heads, d), 'dO')
    close(dwo, mm(dy.t(), o_seq.t()), 'dW_o')


def test_mxfp8_main_grad_accumulates_in_fp32(cp1):
    from fused_gemm_a2a import FusedGemmA2AWorkspace, FusedOutputProjection
    hidden, heads, tokens = 512, 4, 200
    g = torch.Generator().manual_seed(3)
    wo = torch.nn.Parameter((torch.randn(hidden, hidden, generator=g) / 22).to(BF).to(DEV))
    seed = torch.randn(hidden, hidden, generator=g).to(DEV)
    wo.main_grad = seed.clone()
    o = torch.randn(tokens, heads, 128, generator=g).to(BF)
    dy = torch.randn(tokens, hidden, generator=g).to(BF)
    ws = FusedGemmA2AWorkspace(hidden, heads, 256, precision='mxfp8')
    proj = FusedOutputProjection(hidden, heads, weight=wo)
    o_d = o.to(DEV).requires_grad_()
    proj(o_d, ws).backward(dy.to(DEV))
    torch.cuda.synchronize()
    ws.comm.check_status()
    want = torch.from_numpy(mx.mx_matmul(bits(dy.t()), bits(o.reshape(tokens, hidden).t()))).float()
    got = (wo.main_grad - seed).cpu()
    assert (got - want).abs().max() <= 1e-3 * want.abs().max()
    assert wo.grad_added_to_main_grad
