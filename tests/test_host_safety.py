"""Host-side safety nets, on CPU ranks (gloo) with the simulated library where one is needed:

* the descriptor exchange behind VMM-backed symmetric memory serves only ranks of its group and
  gives up after a time limit instead of waiting forever for a rank that died;
* FGA_SYMM=auto: when any rank cannot allocate or map VMM memory, the whole group falls back to
  cudaMalloc + IPC together and this rank's partial mappings are given back;
* the device status word reaches the caller without a synchronization: posted at the end of a
  backward pass, examined at the next forward; FGA_CHECK_STATUS_EVERY adds a synchronizing check;
* the exit helpers for launch scripts.

Failures are made on the host (a rank that never connects, an error code from a fake of the failing
call, a status word written by the test): no GPU is involved.
"""
import os
import subprocess
import sys
import time
import warnings

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
PATHS = (HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), 'fused-gemm-a2a_b200'))


def _join(port, rank, world):
    for path in PATHS:
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)


def _run(worker, world, port, *args, timeout=300):
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, queue, *args)) for r in range(world)]
    for proc in procs:
        proc.start()
    try:
        results = dict(queue.get(timeout=timeout) for _ in range(world))
    finally:
        for proc in procs:
            proc.join(timeout=60)
            if proc.is_alive():
                proc.terminate()
    return [results[r] for r in range(world)]


# ------------------------------------------------------------------------- descriptor exchange
STRANGER = r'''
import socket, sys
with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
    s.settimeout(10)
    s.connect(sys.argv[1])
    try:
        message, descriptors, _, _ = socket.recv_fds(s, 16, 4)
    except OSError:
        message, descriptors = b'', []
print(len(message), len(descriptors))
'''


def _stranger_worker(rank, world, port, queue):
    _join(port, rank, world)
    import fused_gemm_a2a as fused
    mine = os.memfd_create(f'rank{rank}')
    os.write(mine, f'rank {rank}'.encode())
    gather = fused.dist.all_gather_object
    outsider = {}

    def gather_then_intrude(out, obj, group=None):
        gather(out, obj, group=group)
        if rank == 0 and isinstance(obj, tuple) and isinstance(obj[0], str):
            # a process of the same user that is not a rank of the group knocks on rank 1's socket
            outsider['run'] = subprocess.run([sys.executable, '-c', STRANGER, out[1][0]], capture_output=True,
                                             text=True, timeout=60)

    fused.dist.all_gather_object = gather_then_intrude
    try:
        received = fused.exchange_descriptors(dist.group.WORLD, rank, world, mine, timeout=30.0)
    finally:
        fused.dist.all_gather_object = gather
    contents = [os.pread(fd, 6, 0).decode() for fd in received]
    verdict = outsider['run'].stdout.split() if outsider else None
    queue.put((rank, (contents, verdict)))
    dist.barrier()
    dist.destroy_process_group()


def test_a_process_outside_the_group_gets_no_descriptor_and_uses_up_no_turn():
    results = _run(_stranger_worker, 2, 29721)
    for contents, _ in results:
        assert contents == ['rank 0', 'rank 1']
    assert results[0][1] == ['0', '0']         # the outsider was dropped: no message, no descriptor


def _silent_peer_worker(rank, world, port, queue):
    _join(port, rank, world)
    import fused_gemm_a2a as fused
    started = time.monotonic()
    if rank == 1:
        # This rank takes part in the all-gather and then dies before serving or fetching anything.
        box = [None] * world
        dist.all_gather_object(box, ('/nonexistent/fga-socket', os.getpid()))
        queue.put((rank, ('silent', 0.0)))
    else:
        mine = os.memfd_create('rank0')
        try:
            fused.exchange_descriptors(dist.group.WORLD, rank, world, mine, timeout=1.5)
            verdict = 'returned'
        except RuntimeError as error:
            verdict = str(error)
        queue.put((rank, (verdict, time.monotonic() - started)))
    dist.barrier()
    dist.destroy_process_group()


def test_a_peer_that_never_answers_ends_the_exchange_with_an_error_not_a_hang():
    results = _run(_silent_peer_worker, 2, 29722)
    verdict, elapsed = results[0]
    assert 'Descriptor exchange failed on rank 0' in verdict
    assert elapsed < 20


def test_the_exchange_leaves_no_socket_directory_behind(tmp_path, monkeypatch):
    import fused_gemm_a2a as fused
    monkeypatch.setenv('TMPDIR', str(tmp_path))
    import tempfile
    monkeypatch.setattr(tempfile, 'tempdir', None)
    monkeypatch.setattr(fused.dist, 'all_gather_object', lambda out, obj, group=None: out.__setitem__(0, obj))
    descriptor = os.memfd_create('solo')
    try:
        assert fused.exchange_descriptors(None, 0, 1, descriptor) == [descriptor]
    finally:
        os.close(descriptor)
    assert list(tmp_path.iterdir()) == []


# ------------------------------------------------------------------------- FGA_SYMM=auto
def _auto_worker(rank, world, port, queue, broken_call, broken_rank):
    _join(port, rank, world)
    import abi_simulator
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    fused.SYMM_BACKEND = 'auto'
    if broken_call and rank == broken_rank:
        setattr(sim, broken_call, lambda *args: -2)          # FGA_CUDA_ERROR from the failing driver call
    try:
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter('always')
            ws = fused.FusedGemmA2AWorkspace(512, 4, 300)
        kinds = sorted({backend for backend, *_ in ws.comm._allocations})
        x = torch.randn(129, 512).to(torch.bfloat16)
        weight = (torch.randn(1536, 512) / 32).to(torch.bfloat16)
        q, k, v = fused.FusedQKVProjection(512, 4, weight=weight)(x, ws)
        queue.put((rank, dict(backend=ws.comm.symm_backend, kinds=kinds, warned=len(caught),
                              released=[entry[0] for entry in sim.released], rows=q.shape[0])))
    finally:
        undo()
    dist.destroy_process_group()


@pytest.mark.parametrize('broken_call,broken_rank,expected', [
    (None, None, 'vmm'),
    ('fga_symm_alloc_vmm', 1, 'ipc'),          # one rank cannot allocate: nobody exchanges anything
    ('fga_symm_open_vmm', 0, 'ipc'),           # one rank cannot map a peer: everybody undoes its mappings
])
def test_auto_backend_is_decided_by_the_whole_group(broken_call, broken_rank, expected):
    results = _run(_auto_worker, 2, 29723, broken_call, broken_rank)
    for rank, report in enumerate(results):
        assert report['backend'] == expected and report['kinds'] == [expected], report
        assert report['rows'] == 2 * 129
        assert report['warned'] == (1 if expected == 'ipc' and rank == 0 else 0), report
    if broken_call == 'fga_symm_open_vmm':
        # the rank whose import failed gives back its own allocation; the other one also the peer's mapping
        assert results[0]['released'] == ['release'] and results[1]['released'] == ['release', 'release']
    if broken_call == 'fga_symm_alloc_vmm':
        assert results[0]['released'] == ['release'] and results[1]['released'] == []


def _required_vmm_worker(rank, world, port, queue):
    _join(port, rank, world)
    import abi_simulator
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    fused.SYMM_BACKEND = 'vmm'
    if rank == 1:
        sim.fga_symm_alloc_vmm = lambda *args: -2
    try:
        try:
            fused.FusedGemmA2AWorkspace(512, 4, 300)
            verdict = 'created'
        except RuntimeError as error:
            verdict = str(error)
        queue.put((rank, verdict))
    finally:
        undo(meet=False)
    dist.destroy_process_group()


def test_explicit_vmm_raises_on_every_rank_instead_of_falling_back():
    for verdict in _run(_required_vmm_worker, 2, 29724):
        assert 'FGA_SYMM=vmm' in verdict and 'every rank' in verdict


# ------------------------------------------------------------------------- status word
def _status_worker(rank, world, port, queue):
    _join(port, rank, world)
    import abi_simulator
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    report = {}
    try:
        ws = fused.FusedGemmA2AWorkspace(512, 4, 300)
        comm = ws.comm
        weight = (torch.randn(1536, 512) / 32).to(torch.bfloat16).requires_grad_()
        qkv = fused.FusedQKVProjection(512, 4, weight=weight)
        x = torch.randn(129, 512).to(torch.bfloat16).requires_grad_()
        outs = qkv(x, ws)
        comm.status.copy_(torch.tensor([2, 10, 7, 0], dtype=torch.int32))     # as a timed-out kernel leaves it
        torch.autograd.backward(list(outs), [torch.zeros_like(t) for t in outs])   # backward posts the word
        try:
            qkv(x, ws)
            report['next_forward'] = 'ran'
        except RuntimeError as error:
            report['next_forward'] = str(error)
        try:                                    # reported once; the word itself stays until it is cleared
            qkv(x.detach(), ws)
            report['forward_after_report'] = 'ran'
        except RuntimeError as error:
            report['forward_after_report'] = str(error)
        try:
            comm.check_status()
            report['check'] = 'clean'
        except RuntimeError as error:
            report['check'] = str(error)
        comm.clear_status()
        comm.check_status()
        qkv(x.detach(), ws)
        report['after_clear'] = comm.status.tolist()
        # the synchronizing variant: every second forward checks the device word itself
        fused.CHECK_STATUS_EVERY = 2
        comm._forwards = 0
        comm.status.copy_(torch.tensor([1, 3, 9, 0], dtype=torch.int32))
        qkv(x.detach(), ws)
        try:
            qkv(x.detach(), ws)
            report['every_second'] = 'ran'
        except RuntimeError as error:
            report['every_second'] = str(error)
        comm.clear_status()
        queue.put((rank, report))
    finally:
        fused.CHECK_STATUS_EVERY = 0
        undo()
    dist.destroy_process_group()


def test_a_device_error_surfaces_at_the_next_forward_without_a_synchronizing_call():
    report, = _run(_status_worker, 1, 29725)
    assert 'device error 2' in report['next_forward'] and 'where=10, detail=7' in report['next_forward']
    assert report['forward_after_report'] == 'ran'
    assert 'device error 2' in report['check']
    assert report['after_clear'] == [0, 0, 0, 0]
    assert 'device error 1' in report['every_second']


def test_mxfp8_weight_gradient_reports_into_the_groups_status_word(monkeypatch):
    import fused_gemm_a2a as fused
    seen = {}

    def fake_wgrad(dy, x, out, *, accumulate=False, status=None):
        seen.update(status=status, accumulate=accumulate)
        return out

    monkeypatch.setattr(fused, 'mxfp8_wgrad', fake_wgrad)
    weight = torch.nn.Parameter(torch.empty(384, 128, dtype=torch.bfloat16))
    dy, x = torch.empty(33, 384, dtype=torch.bfloat16), torch.empty(33, 128, dtype=torch.bfloat16)
    word = torch.zeros(4, dtype=torch.int32)
    fused._weight_grad(weight, dy, x, 'mxfp8', word)
    assert seen['status'] is word and seen['accumulate'] is False
    seen.clear()
    fused._weight_grad(weight, dy, x, 'mxfp8')           # the reference's call shape: no status argument
    assert seen['status'] is None


# ------------------------------------------------------------------------- leaving in order
def test_exit_helpers_drain_and_hold_only_when_memory_would_vanish(monkeypatch):
    import fused_gemm_a2a as fused
    import fused_gemm_a2a_kernels as kernels
    slept = []
    monkeypatch.setattr(time, 'sleep', slept.append)
    monkeypatch.setattr(kernels, 'DEVICE_TIMEOUT_NS', 7_000_000_000)

    class Runtime:
        def __init__(self, p, backend):
            self.p, self.symm_backend, self.device = p, backend, torch.device('cpu')

    monkeypatch.setattr(fused, '_live_comms', [Runtime(1, 'ipc'), Runtime(4, 'vmm')])
    fused.hold_buffers_after_failure()
    assert slept == []                           # one rank alone, or memory that outlives its owner
    monkeypatch.setattr(fused, '_live_comms', [Runtime(4, 'vmm'), Runtime(2, 'ipc')])
    fused.hold_buffers_after_failure()
    assert slept == [9.0]                        # the package's device time limit + 2 s


SIGTERM_SCRIPT = r'''
import os, signal, sys, time
sys.path[:0] = {paths!r}
import fused_gemm_a2a as fused
import torch
class Runtime:
    p, symm_backend, device = 2, 'ipc', torch.device('cpu')
fused._live_comms.append(Runtime())
drained = []
fused._drain = lambda: (drained.append(1), print('drained', flush=True))
fused.install_exit_guards()
os.kill(os.getpid(), signal.SIGTERM)
time.sleep(5)
print('survived', flush=True)
'''


def test_sigterm_drains_first_and_then_ends_the_process_by_the_same_signal():
    import signal
    result = subprocess.run([sys.executable, '-c', SIGTERM_SCRIPT.format(paths=list(PATHS))], capture_output=True,
                            text=True, timeout=120)
    assert result.stdout.split() == ['drained']
    assert result.returncode == -signal.SIGTERM


# ------------------------------------------------------------------------- MXFP8 weight cache
def _weight_cache_worker(rank, world, port, queue):
    _join(port, rank, world)
    import abi_simulator
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    counts = {}
    try:
        quantize, calls = fused.mxfp8_quantize, []

        def counting(a, *, k_multiple=256):
            calls.append(tuple(a.shape))
            return quantize(a, k_multiple=k_multiple)

        fused.mxfp8_quantize = counting
        ws = fused.FusedGemmA2AWorkspace(512, 4, 300, precision='mxfp8')
        weight = (torch.randn(1536, 512) / 32).to(torch.bfloat16).requires_grad_()
        qkv = fused.FusedQKVProjection(512, 4, weight=weight)
        x = torch.randn(129, 512).to(torch.bfloat16).requires_grad_()

        def step():
            del calls[:]
            outs = qkv(x, ws)
            torch.autograd.backward(list(outs), [torch.ones_like(t) for t in outs])
            return sum(1 for shape in calls if 1536 in shape)      # quantizer passes over the weight

        counts['off'] = [step(), step()]
        fused.MX_WEIGHT_CACHE = True
        fused._quantized_weights.clear()
        counts['on'] = [step(), step(), step()]
        with torch.no_grad():
            weight.mul_(0.5)                                       # an optimizer step: the version counter moves
        counts['after_update'] = [step(), step()]
        queue.put((rank, counts))
    finally:
        fused.MX_WEIGHT_CACHE = False
        fused._quantized_weights.clear()
        undo()
    dist.destroy_process_group()


def test_quantized_weights_are_kept_only_while_the_weight_is_unchanged():
    counts, = _run(_weight_cache_worker, 1, 29726)
    assert counts['off'] == [2, 2]                  # forward (rows) and dgrad (columns): every call, as the reference does
    assert counts['on'] == [2, 0, 0]
    assert counts['after_update'] == [2, 0]


def _resync_worker(rank, world, port, queue):
    _join(port, rank, world)
    import abi_simulator
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    try:
        ws = fused.FusedGemmA2AWorkspace(512, 4, 300)
        comm = ws.comm
        # as after a timed-out step: rank 1 skipped two barriers, so the epochs its peers wrote here are ahead
        comm.flags.copy_(torch.tensor([7, 7] if rank == 0 else [5, 7], dtype=torch.int64))
        comm.status.copy_(torch.tensor([1, 1, 6, 0], dtype=torch.int32))
        comm.clear_status()
        queue.put((rank, (comm.flags.tolist(), comm.status.tolist())))
    finally:
        undo()
    dist.destroy_process_group()


def test_clearing_the_status_word_puts_every_rank_back_on_the_same_barrier_epoch():
    for flags, status in _run(_resync_worker, 2, 29727):
        assert flags == [0, 0] and status == [0, 0, 0, 0]
