"""GPU parity of paths that are selected by environment variables, all off by default:

* FGA_WGRAD_SPLITS: an FP32 weight gradient whose token axis is cut into shares that add into the
  output with bulk reductions;
* FGA_GROUP_M_RECV=1: recv launches with one row tile per raster group, so that most pusher jobs go
  through the steady phase of the two-phase pusher schedule;
* the VMM-backed symmetric allocation on one device.

The file sorts after the tests of the default paths on purpose: nothing else in the suite depends
on these settings.
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


@pytest.mark.parametrize('p,hidden,heads,tokens,num_in', [(2, 512, 4, 1100, 3), (4, 1024, 8, 1300, 1)])
def test_receive_steady_phase(native, monkeypatch, p, hidden, heads, tokens, num_in):
    """One row tile per raster group: the first phase covers two of the five or six row tiles and
    the rest goes through the steady phase. Ranks are emulated on one GPU: all the pushes of every
    rank run first, then every rank's GEMM."""
    monkeypatch.setenv('FGA_GROUP_M_RECV', '1')
    receive_case(native, p, hidden, heads, tokens, num_in)


def test_vmm_allocation_is_shared_through_its_descriptor_and_outlives_the_first_mapping(native):
    """FGA_SYMM=vmm on one GPU: the allocation's file descriptor is imported again in the same
    process, which gives a second mapping of the same physical memory (what a peer process gets).
    Stores through one mapping are read through the other, and after the owner's mapping is released
    the memory is still there for the remaining one."""
    import ctypes

    from fused_gemm_a2a import _wrap
    dev = torch.device('cuda', 0)
    wanted = 3 << 20
    size = native.fga_symm_vmm_size(wanted)
    assert size >= wanted, native.fga_last_error()
    owner, alias, descriptor = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int(-1)
    assert native.fga_symm_alloc_vmm(wanted, ctypes.byref(owner), ctypes.byref(descriptor)) == 0, native.fga_last_error()
    try:
        assert native.fga_symm_open_vmm(descriptor.value, size, ctypes.byref(alias)) == 0, native.fga_last_error()
    finally:
        os.close(descriptor.value)
    assert owner.value and alias.value and owner.value != alias.value and owner.value % 256 == 0
    first, second = _wrap(owner.value, size, dev), _wrap(alias.value, size, dev)
    assert int(first.sum()) == 0                      # zero-filled
    first[:4096] = 7
    second[size - 4096:] = 9
    torch.cuda.synchronize()
    assert bool((second[:4096] == 7).all()) and bool((first[size - 4096:] == 9).all())
    del first
    assert native.fga_symm_release_vmm(owner.value, size) == 0, native.fga_last_error()
    torch.cuda.synchronize()
    assert bool((second[:4096] == 7).all()) and int(second[4096:size - 4096].sum()) == 0
    del second
    assert native.fga_symm_release_vmm(alias.value, size) == 0, native.fga_last_error()
