"""Multi-rank index mapping on ONE GPU, through the C ABI.

Kernels of different ranks must never wait on one another as separate launches on one GPU, so the
P ranks are emulated without any cross-launch wait: push GEMMs never wait, and the receive kernel
is launched twice per rank - first with only its pusher warps (roles = 2) for every rank, then with
only its GEMM roles (roles = 1), whose arrival counters are by then complete. Every "peer" buffer
is an ordinary allocation on this GPU, addressed through the same int64 peer tables the real
multi-GPU path uses. Transport is compared bit-exactly with the CPU oracle, GEMM results within
the BF16 tolerance (max error 1e-2 of scale, Frobenius <= 2e-3).
"""
import pytest
import torch

import _fga_native as nat
from oracle.ulysses_oracle import UlyssesOracle

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
TIMEOUT_NS = 5_000_000_000
BF = torch.bfloat16


def close(actual, expected, what):
    actual, expected = actual.float().cpu(), expected.float().cpu()
    scale = expected.abs().max().clamp_min(1e-6)
    assert (actual - expected).abs().max() <= 1e-2 * scale, what
    assert torch.linalg.norm(actual - expected) <= 2e-3 * torch.linalg.norm(expected) + 1e-6, what


def table(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=DEV)


@pytest.mark.parametrize('p,hidden,heads,tokens,segments,bias_in_gemm', [
    (2, 512, 4, 300, 3, False), (4, 1024, 8, 129, 4, True), (2, 256, 2, 256, 3, False), (8, 1024, 8, 77, 3, False)])
def test_push_lands_in_the_right_peer_tiles(native, p, hidden, heads, tokens, segments, bias_in_gemm):
    g = torch.Generator().manual_seed(p * 1000 + tokens)
    capacity = (tokens + 255) // 256 * 256
    weight = (torch.randn(segments * hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
    bias = torch.randn(segments * hidden, generator=g).to(BF) if bias_in_gemm else None
    xs = [torch.randn(tokens, hidden, generator=g).to(BF) for _ in range(p)]
    heads_bufs = [[torch.full((p * capacity, hidden // p), 5.0, dtype=BF, device=DEV) for _ in range(segments)]
                  for _ in range(p)]
    tables = [table([heads_bufs[d][s] for d in range(p)]) for s in range(segments)]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    w_dev = weight.to(DEV)
    b_dev = bias.to(DEV) if bias is not None else None
    for r in range(p):
        x = xs[r].to(DEV)
        rc = native.fga_gemm_push(x.data_ptr(), tokens, hidden, capacity, w_dev.data_ptr(), 0,
                                  0 if b_dev is None else b_dev.data_ptr(), segments, hidden,
                                  nat.ptr_array([t.data_ptr() for t in tables]), capacity, r, p,
                                  status.data_ptr(), TIMEOUT_NS, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    oracle = UlyssesOracle(p, hidden, heads, segments, weight, bias, bias_in_gemm=bias_in_gemm)
    want = oracle.qkv_heads_buffers(xs, capacity)
    for d in range(p):
        for s in range(segments):
            close(heads_bufs[d][s], want[d][s], f'dest {d} segment {s}')


@pytest.mark.parametrize('p,hidden,heads,tokens', [(2, 512, 4, 300), (4, 1024, 8, 256), (8, 1024, 8, 31)])
def test_output_dgrad_push_routes_columns_to_their_owner(native, p, hidden, heads, tokens):
    """segments = 1 with a [K, N] weight (dO = dY * Wo): column block d goes to peer d."""
    g = torch.Generator().manual_seed(p + tokens)
    capacity = (tokens + 255) // 256 * 256
    wo = (torch.randn(hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
    dys = [torch.randn(tokens, hidden, generator=g).to(BF) for _ in range(p)]
    bufs = [torch.full((p * capacity, hidden // p), 5.0, dtype=BF, device=DEV) for _ in range(p)]
    tab = table(bufs)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    w_dev = wo.to(DEV)
    for r in range(p):
        dy = dys[r].to(DEV)
        rc = native.fga_gemm_push(dy.data_ptr(), tokens, hidden, capacity, w_dev.data_ptr(), 1, 0, 1, hidden,
                                  nat.ptr_array([tab.data_ptr()]), capacity, r, p, status.data_ptr(),
                                  TIMEOUT_NS, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    want = UlyssesOracle(p, hidden, heads, 1, weight_out=wo).out_dhead_buffers(dys, capacity)
    for d in range(p):
        close(bufs[d], want[d], f'dest {d}')


@pytest.mark.parametrize('p,hidden,heads,tokens,num_in', [
    (2, 512, 4, 300, 1), (2, 512, 4, 300, 3), (4, 1024, 8, 129, 4), (8, 1024, 8, 256, 3), (4, 512, 4, 1, 1)])
def test_receive_transport_and_gemm(native, p, hidden, heads, tokens, num_in):
    from fused_gemm_a2a_kernels import push_split
    g = torch.Generator().manual_seed(p * 77 + tokens + num_in)
    capacity = (tokens + 255) // 256 * 256
    k = num_in * hidden
    hpr, d_head = heads // p, hidden // heads
    b_is_kn = num_in > 1
    weight = (torch.randn(k, hidden, generator=g) / k ** 0.5).to(BF) if b_is_kn else \
        (torch.randn(hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
    inputs = [tuple(torch.randn(p * tokens, hpr, d_head, generator=g).to(BF) for _ in range(num_in))
              for _ in range(p)]
    recvs = [torch.full((capacity, k), 9.0, dtype=BF, device=DEV) for _ in range(p)]
    counters = [torch.zeros(capacity // 128, dtype=torch.int32, device=DEV) for _ in range(p)]
    outs = [torch.full((capacity, hidden), float('nan'), dtype=BF, device=DEV) for _ in range(p)]
    t_recv, t_cnt = table(recvs), table(counters)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    w_dev = weight.to(DEV)
    dev_inputs = [[t.to(DEV).flatten(1).contiguous() for t in inputs[r]] for r in range(p)]
    split = push_split(k, p, num_in)
    for roles in (2, 1):
        for r in range(p):
            rc = native.fga_gemm_recv(recvs[r].data_ptr(), capacity, k, w_dev.data_ptr(), int(b_is_kn), hidden,
                                      outs[r].data_ptr(), t_recv.data_ptr(), t_cnt.data_ptr(),
                                      counters[r].data_ptr(),
                                      nat.ptr_array([t.data_ptr() for t in dev_inputs[r]]), num_in, tokens, split,
                                      r, p, roles, None, None, status.data_ptr(), TIMEOUT_NS,
                                      torch.cuda.current_stream().cuda_stream)
            assert rc == 0, native.fga_last_error()
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        if roles == 2:
            for r in range(p):
                assert counters[r].tolist() == [p * num_in * split] * (capacity // 128)
    oracle = UlyssesOracle(p, hidden, heads, max(num_in, 1))
    for r in range(p):
        want = (oracle.qkv_recv_buffer(inputs, r, capacity) if num_in > 1
                else oracle.out_recv_buffer([t[0] for t in inputs], r, capacity))
        assert torch.equal(recvs[r].cpu(), want), f'rank {r}: receive buffer differs'
        ref = want.float() @ (weight.float() if b_is_kn else weight.float().t())
        close(outs[r], ref, f'rank {r} GEMM')
