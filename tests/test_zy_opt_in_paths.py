"""GPU parity of the two opt-in schedules of the GEMM kernel, both off by default:

* FGA_WGRAD_SPLITS: an FP32 weight gradient whose token axis is cut into shares that add into the
  output with bulk reductions;
* FGA_PUSH_PAIRS: recv launches in which some CTA pairs only push while the others only compute
  after the first raster groups.

The file sorts after the tests of the default paths on purpose: these schedules are selected by
environment variables and nothing else in the suite depends on them.
"""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_emulated_ranks import test_receive_transport_and_gemm as receive_case  # noqa: E402

pytestmark = pytest.mark.gpu

TIMEOUT_NS = 5_000_000_000


@pytest.mark.parametrize('splits', ['1', '4', '8', 'auto'])
@pytest.mark.parametrize('accumulate', [False, True])
def test_weight_gradient_split_along_tokens(native, monkeypatch, splits, accumulate):
    """The output is a column window of a wider matrix: a plain store zero-fills exactly that
    window before the shares add into it, and the neighbouring columns keep their contents."""
    monkeypatch.setenv('FGA_WGRAD_SPLITS', splits)
    dev = torch.device('cuda', 0)
    m, n, k, ldc = 300, 256, 16384, 384
    g = torch.Generator().manual_seed(11)
    dy = torch.randn(k, m, generator=g).to(torch.bfloat16).to(dev)
    x = (torch.randn(k, n, generator=g) / 8).to(torch.bfloat16).to(dev)
    start = torch.randn(m, ldc, generator=g).to(dev)
    wide = start.clone()
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    # operands need 16-byte aligned rows: pad the token-major dY to a multiple of 8 columns
    lda = (m + 7) // 8 * 8
    dy_pad = torch.zeros(k, lda, dtype=torch.bfloat16, device=dev)
    dy_pad[:, :m] = dy
    rc = native.fga_gemm_local(dy_pad.data_ptr(), 1, x.data_ptr(), 1, m, n, k, lda, n,
                               wide.data_ptr() + 64 * 4, ldc, 1, int(accumulate), status.data_ptr(),
                               TIMEOUT_NS, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = dy.float().t() @ x.float()
    if accumulate:
        ref = ref + start[:, 64:64 + n]
    assert (wide[:, 64:64 + n] - ref).abs().max() <= 1e-4 * ref.abs().max()
    assert torch.equal(wide[:, :64], start[:, :64]) and torch.equal(wide[:, 64 + n:], start[:, 64 + n:])


@pytest.mark.parametrize('push_pairs', [0, 3, 200])
@pytest.mark.parametrize('p,hidden,heads,tokens,num_in', [(2, 512, 4, 1100, 3), (4, 1024, 8, 1300, 1)])
def test_receive_steady_phase_and_pushing_only_ctas(native, monkeypatch, p, hidden, heads, tokens, num_in,
                                                    push_pairs):
    """One row tile per raster group: the first phase covers two of the five or six row tiles and
    the rest goes through the steady phase, on every CTA (0) or on CTA pairs that only push
    (3; 200 is clamped so that one pair still computes). Ranks are emulated on one GPU: all the
    pushes of every rank run first, then every rank's GEMM."""
    monkeypatch.setenv('FGA_GROUP_M_RECV', '1')
    monkeypatch.setenv('FGA_PUSH_PAIRS', str(push_pairs))
    receive_case(native, p, hidden, heads, tokens, num_in)
