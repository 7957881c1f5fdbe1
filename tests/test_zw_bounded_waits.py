"""Failure detection on the GPU without a fault: a wait that nothing will ever satisfy runs into its
time limit, the kernel records {code, where, detail} in the status word and returns, the context
stays usable, and while the word holds a code the kernels return at entry without touching peer
memory. The "peer that never arrives" is a flag slot in this GPU's own memory that nobody sets.
No trap, no bad address, no endless loop: every wait used here is bounded by a 0.3 s limit.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
LIMIT_NS = 300_000_000


def test_barrier_gives_up_on_a_silent_peer_and_the_error_is_sticky(native):
    flags = torch.zeros(2, dtype=torch.int64, device=DEV)          # this rank's slots, one per peer
    silent_peer = torch.zeros(2, dtype=torch.int64, device=DEV)    # stands for rank 1's slots; nobody answers
    peer_flags = torch.tensor([flags.data_ptr(), silent_peer.data_ptr()], dtype=torch.int64, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    rc = native.fga_barrier(flags.data_ptr(), peer_flags.data_ptr(), 0, 2, 0, 0, 0, 0, status.data_ptr(), LIMIT_NS, stream)
    assert rc == 0, native.fga_last_error()
    torch.cuda.synchronize()
    code, where, detail, _ = status.tolist()
    assert (code, where, detail) == (1, 1, 1)          # barrier timeout, waiting for lane 1, epoch 1
    assert flags.tolist() == [1, 0] and silent_peer.tolist() == [1, 0]   # published to both, heard only from itself

    # Sticky: with the code still in place a GEMM returns at entry and leaves its output alone ...
    a = torch.randn(256, 256, device=DEV).to(torch.bfloat16)
    out = torch.full((256, 256), float('nan'), dtype=torch.bfloat16, device=DEV)

    def gemm():
        rc = native.fga_gemm_local(a.data_ptr(), 0, a.data_ptr(), 0, 256, 256, 256, 256, 256, out.data_ptr(), 256,
                                   0, 0, status.data_ptr(), LIMIT_NS, stream)
        assert rc == 0, native.fga_last_error()
        torch.cuda.synchronize()

    gemm()
    assert bool(torch.isnan(out).all()) and status.tolist()[0] == 1
    # ... so does the next barrier (no new publication) ...
    rc = native.fga_barrier(flags.data_ptr(), peer_flags.data_ptr(), 0, 2, 0, 0, 0, 0, status.data_ptr(), LIMIT_NS, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert flags.tolist() == [1, 0] and silent_peer.tolist() == [1, 0]
    # ... and after the host has cleared the word the same launch computes.
    status.zero_()
    gemm()
    expected = a.float() @ a.float().t()
    assert torch.linalg.norm(out.float() - expected) <= 2e-3 * torch.linalg.norm(expected)
    assert status.tolist() == [0, 0, 0, 0]


def test_check_status_reports_and_clear_status_recovers(cp1):
    from fused_gemm_a2a import FusedGemmA2AWorkspace
    ws = FusedGemmA2AWorkspace(512, 4, 256)
    ws.comm.check_status()
    try:
        ws.comm.status.copy_(torch.tensor([2, 10, 7, 0], dtype=torch.int32))  # as a kernel would leave it
        with pytest.raises(RuntimeError, match='device error 2.*where=10, detail=7'):
            ws.comm.check_status()
    finally:
        ws.comm.clear_status()      # the group's status word is shared by every later test of the session
    ws.comm.check_status()
    assert ws.comm.status.tolist() == [0, 0, 0, 0]
