"""Fused projection GEMM + Ulysses all-to-all for context-parallel attention on B200 (sm_100a).

Drop-in for the public surface of the reference module fused_gemm_a2a.py
(FusedGemmA2AWorkspace, FusedQKVProjection, FusedOutputProjection; reference lines 475-648):

    ws = FusedGemmA2AWorkspace(H, N, max_local_tokens, cp_group=None, gate=False, precision="bf16")
    q, k, v = FusedQKVProjection(H, N, weight=Wqkv)(x, ws)     # x [M, H] -> each [P*M, N/P, D]
    y = FusedOutputProjection(H, N, weight=Wo)(o, ws)           # o [P*M, N/P, D] -> y [M, H]

Sequence side is [M, H]; head side is [P*M, heads/P, D] with rank-major rows. QKV weights and
biases use Megatron's per-head [q; k; v; (gate)] row order. All CP ranks call with equal M in the
same order. Returned activations and gradients own ordinary storage.

The host layer is plain PyTorch plumbing (validation, autograd, buffer views). All device work is
done by libfga.so through its C ABI: symmetric buffers are allocated once per geometry and mapped
into every peer (driver virtual-memory allocations shared as file descriptors, or cudaMalloc +
CUDA IPC handles), exchanged once over the CP group; the GEMMs are hand-written TMA/tcgen05
kernels whose epilogue (push) or pusher warps (receive) perform the all-to-all over NVLink. No
kernel is compiled at run time and nothing falls back to the CPU.

Layout of this file: memory (slabs of symmetric memory and their peer tables), the per-group
runtime `_Comm` (barrier, status word, GEMM launches), gradient helpers, the two autograd
functions, the buffer sets and their active-length views, and the public classes.
"""
import atexit
import os
import signal
import warnings
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
from torch import nn
from torch.profiler import record_function

import _fga_native as _native
import fused_gemm_a2a_kernels as _k
from fused_gemm_a2a_kernels import (  # noqa: F401  (re-exported: the reference's tests import them here)
    CLUSTER_MN, CTA_M, MMA_N, MMA_N_OUT_PUSH, MMA_N_RECV, MMA_TILER_MN, PUSH_SPLIT,
    bf16_wgrad, device_barrier, mxfp8_quantize, mxfp8_tile_n, mxfp8_wgrad, padded_rows, push_split,
    reduce_bias_grad, resize_rank_rows, tile_swizzle, validate_peer_count, validate_tile_n,
)

__all__ = ['FusedGemmA2AWorkspace', 'FusedQKVProjection', 'FusedOutputProjection',
           'install_exit_guards', 'hold_buffers_after_failure', 'release_all']

# The reference selects between torch's GEMM + add_ and Megatron's accumulating cuBLAS extension
# for the BF16 weight gradient (fused_gemm_a2a.py:34-40). Here both settings mean the same thing:
# the GEMM epilogue adds straight into main_grad, so no extension is imported. The variable is
# still validated so that a launch script written for the reference fails the same way.
WGRAD_BACKEND = os.environ.get('FUSED_WGRAD_BACKEND', 'torch')
if WGRAD_BACKEND not in ('torch', 'fused_accum'):
    raise ValueError('FUSED_WGRAD_BACKEND must be torch or fused_accum')

# Debug aid, off by default: with FGA_CHECK_TOKENS=1 every forward first checks on the host that all
# ranks of the CP group pass the same local token count (one small all-reduce, so not for production
# steps and skipped during graph capture). Ranks that disagree would otherwise wait, until the
# device time limit, for row blocks that never arrive.
CHECK_TOKENS = os.environ.get('FGA_CHECK_TOKENS', '0') == '1'

# How symmetric buffers are allocated and mapped into the peers: 'vmm' = the driver's virtual memory
# management API with POSIX file descriptors passed over Unix-domain sockets, 'ipc' = cudaMalloc +
# CUDA IPC memory handles. With 'vmm' every mapping holds a reference to the physical memory, so a
# rank that exits (a crash, an exception on one rank, a SIGTERM from the launcher) does not unmap
# what its peers still store into; with 'ipc' such stores are GPU memory faults. The default 'auto'
# tries 'vmm' when a group's runtime is created and, if any rank cannot allocate, export, pass or map
# the memory, the whole group falls back to 'ipc' together (one warning on rank 0).
SYMM_BACKEND = os.environ.get('FGA_SYMM', 'auto')
if SYMM_BACKEND not in ('auto', 'ipc', 'vmm'):
    raise ValueError('FGA_SYMM must be auto, ipc or vmm')

# Seconds a rank waits for a peer while file descriptors are handed around (FGA_SYMM=vmm / auto).
DESCRIPTOR_TIMEOUT_S = float(os.environ.get('FGA_DESCRIPTOR_TIMEOUT_S', 60))

# FGA_MX_WEIGHT_CACHE=1 (off by default; MXFP8 only): keep the quantized copy of a weight, per
# reduction axis, for as long as the weight tensor is unchanged (same storage, same autograd version
# counter), instead of requantizing it from BF16 on every call as the reference does. The result is
# bit-identical; it saves one pass over the weight per GEMM and holds two E4M3 copies (as many bytes
# as the BF16 weight). Never used during graph capture: a captured step quantizes inside the graph,
# because a replay must see the weights an optimizer step has written in between.
MX_WEIGHT_CACHE = os.environ.get('FGA_MX_WEIGHT_CACHE', '0') == '1'

# With FGA_CHECK_STATUS_EVERY=N every N-th forward of a group synchronizes and raises when a device
# wait has expired since the last check (never during graph capture). Off by default (0): the status
# word is then surfaced without synchronizing, see _Comm.post_status / poll_status.
CHECK_STATUS_EVERY = int(os.environ.get('FGA_CHECK_STATUS_EVERY', 0))

_ALIGN = 1024        # every region of a slab starts on a 1 KiB boundary
_HANDLE_BYTES = 64   # size of an exported memory handle (FGA_IPC_HANDLE_BYTES)
_ROW_TILE = MMA_TILER_MN[0]   # rows of a CTA pair: capacities are multiples of it


def _itemsize(dtype):
    return torch.empty(0, dtype=dtype).element_size()


def _numel(shape):
    total = 1
    for extent in shape:
        total *= extent
    return total


# ----------------------------------------------------------------------------------------------
# Symmetric memory
# ----------------------------------------------------------------------------------------------
class _DevicePointer:
    """Exposes raw device memory to torch through the CUDA array interface."""

    def __init__(self, address, nbytes):
        self.__cuda_array_interface__ = {
            'shape': (nbytes,), 'typestr': '|u1', 'data': (address, False), 'version': 3}


def _wrap(address, nbytes, device):
    return torch.as_tensor(_DevicePointer(address, nbytes), device=device)


def slab_offsets(layout):
    """Byte (offset, size) of every (name, shape, dtype) entry of a slab and the slab's total size;
    each entry starts on a 1 KiB boundary."""
    placed, cursor = [], 0
    for _, shape, dtype in layout:
        size = _numel(shape) * _itemsize(dtype)
        placed.append((cursor, size))
        cursor += -(-size // _ALIGN) * _ALIGN
    return placed, cursor


def exchange_handles(group, rank, peers, handle, local_address, open_peer):
    """All-gather one 64-byte memory handle per rank over the CP group (the only collective of a
    buffer's lifetime) and map every peer's allocation: returns the P addresses under which this
    rank reaches each rank's buffer, its own through `local_address`."""
    inbox = [None] * peers
    dist.all_gather_object(inbox, (rank, bytes(handle)), group=group)
    reachable = []
    for owner, entry in enumerate(inbox):
        sender, raw = entry
        if sender != owner or len(raw) != _HANDLE_BYTES:
            raise RuntimeError('Memory handle exchange returned a malformed entry')
        reachable.append(local_address if owner == rank else open_peer(raw))
    return reachable


def exchange_descriptors(group, rank, peers, descriptor, timeout=None):
    """Hand one open file descriptor of every rank to every other rank of the group (all on this
    host). Each rank listens on a Unix-domain socket inside a private directory (mode 0700, so only
    this user can connect), the socket paths and process ids go around with one all-gather, and every
    rank fetches its peers' descriptors as SCM_RIGHTS messages. A connection is served only when the
    kernel reports (SO_PEERCRED) the same user and the process id of a rank of this group; anything
    else is dropped without using up a peer's turn. Every accept, connect and receive is bounded by
    `timeout` seconds (default FGA_DESCRIPTOR_TIMEOUT_S), after which RuntimeError is raised instead
    of waiting forever for a rank that died. Returns P descriptors valid in this process:
    `descriptor` itself at [rank], received duplicates (which the caller closes) elsewhere."""
    import shutil
    import socket
    import struct
    import tempfile
    import threading
    import time
    timeout = DESCRIPTOR_TIMEOUT_S if timeout is None else timeout
    directory = tempfile.mkdtemp(prefix='fga-')
    path = os.path.join(directory, 'fd')
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    received, failure = [], []
    try:
        server.bind(path)
        server.listen(max(peers, 1))
        identities = [None] * peers
        dist.all_gather_object(identities, (path, os.getpid()), group=group)
        members = {pid for _, pid in identities}
        credentials = struct.Struct('3i')            # struct ucred: pid, uid, gid

        def serve():
            served, deadline = 0, time.monotonic() + timeout
            try:
                while served < peers - 1:
                    server.settimeout(max(0.05, deadline - time.monotonic()))
                    connection, _ = server.accept()
                    with connection:
                        connection.settimeout(timeout)
                        pid, uid, _ = credentials.unpack(
                            connection.getsockopt(socket.SOL_SOCKET, socket.SO_PEERCRED, credentials.size))
                        if uid != os.getuid() or pid not in members:
                            continue               # not a rank of this group: no descriptor, no turn
                        socket.send_fds(connection, [b'fd'], [descriptor])
                        served += 1
            except OSError as error:               # includes socket.timeout
                failure.append(error)

        server_thread = threading.Thread(target=serve, daemon=True)
        server_thread.start()
        try:
            for owner in range(peers):
                if owner == rank:
                    received.append(descriptor)
                    continue
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as client:
                    client.settimeout(timeout)
                    client.connect(identities[owner][0])
                    message, descriptors, _, _ = socket.recv_fds(client, 16, 1)
                if len(descriptors) != 1 or message != b'fd':
                    for extra in descriptors:
                        os.close(extra)
                    raise RuntimeError('Descriptor exchange returned a malformed message')
                received.append(descriptors[0])
        except OSError as error:
            failure.append(error)
        server_thread.join(timeout + 1.0)
        if server_thread.is_alive() and not failure:
            failure.append(TimeoutError('a peer never fetched this rank\'s descriptor'))
        if failure:
            for owner, got in enumerate(received):
                if owner != rank:
                    os.close(got)
            raise RuntimeError(f'Descriptor exchange failed on rank {rank}: {failure[0]!r}')
        return received
    finally:
        server.close()
        shutil.rmtree(directory, ignore_errors=True)


class _Slab:
    """One symmetric allocation: the local bytes and the address of the same allocation on every
    rank as seen from this one. Regions of it become tensors with their int64 peer tables."""

    def __init__(self, base, nbytes, peer_bases, device):
        self.base, self.nbytes, self.peer_bases, self.device = base, nbytes, peer_bases, device
        self.bytes = _wrap(base, nbytes, device)

    def region(self, offset, shape, dtype):
        size = _numel(shape) * _itemsize(dtype)
        tensor = self.bytes[offset:offset + size].view(dtype).view(shape)
        addresses = tuple(peer + offset for peer in self.peer_bases)
        table = torch.tensor(addresses, dtype=torch.int64, device=self.device)
        table.peer_addresses = addresses           # host copy: reading the device table would synchronize
        return tensor, table


class _RecvBuffer:
    """Receive side of one pooled geometry: the symmetric buffer, its arrival counters (one per 128
    rows), both with their peer address tables, and the device-side invocation counter."""

    def __init__(self, recv, peer_recv, counters, peer_counters, epoch):
        self.recv, self.counters, self.epoch = recv, counters, epoch
        self.peer_recv, self.peer_counters = peer_recv, peer_counters


# ----------------------------------------------------------------------------------------------
# Leaving in order
# ----------------------------------------------------------------------------------------------
_live_comms = []


def _drain():
    """Wait until this process's GPU work has finished. Every device wait of the kernels is bounded,
    so this returns; afterwards nothing of this process is still storing into a peer's memory."""
    for comm in list(_live_comms):
        try:
            if comm.device.type == 'cuda':
                torch.cuda.synchronize(comm.device)
        except Exception:                          # noqa: BLE001  (interpreter shutdown: nothing left to do)
            pass


_drain_registered = []


def _drain_at_exit(comm):
    """Register a runtime for the interpreter-exit drain (installed once)."""
    if not _drain_registered:
        atexit.register(_drain)
        _drain_registered.append(True)
    _live_comms.append(comm)


def hold_buffers_after_failure():
    """For launch scripts: call on a rank that hit an unexpected exception, before it exits. The rank's
    queued kernels finish; then, if any of its symmetric buffers would disappear with the process
    (cudaMalloc + IPC backing), it keeps them mapped until the peers' bounded device waits have run
    out (FGA_TIMEOUT_S + 2 s): by then their status words are set and their later launches return at
    entry instead of storing into freed memory. With VMM-backed buffers nothing has to be held."""
    import time
    _drain()
    if any(comm.p > 1 and comm.symm_backend != 'vmm' for comm in _live_comms):
        time.sleep(_k.DEVICE_TIMEOUT_NS / 1e9 + 2.0)


def release_all():
    """Collective, for the normal end of a run: every rank gives back the symmetric buffers of all
    its groups (see _Comm.release), in creation order, after all ranks have drained their devices."""
    for comm in list(_Comm._instances.values()):
        comm.release()


def install_exit_guards(signals=(signal.SIGTERM,)):
    """For launch scripts (call once, from the main thread): on SIGTERM - what torchrun sends to the
    surviving workers when one rank has died - first let this process's queued GPU work finish,
    then die by the same signal. Without it the context is torn down under kernels that may be in
    the middle of remote stores. The interpreter-exit drain is always installed; this adds the
    signal path, which a library must not take over on its own."""
    def handler(number, _frame):
        _drain()
        signal.signal(number, signal.SIG_DFL)
        os.kill(os.getpid(), number)

    for number in signals:
        signal.signal(number, handler)


# ----------------------------------------------------------------------------------------------
# Per-group runtime
# ----------------------------------------------------------------------------------------------
class _Comm:
    """Per (process group, device) state: rank, barrier flags, the device status word and the pool
    of symmetric allocations. Layers of equal geometry share buffers, so the footprint does not
    grow with depth (reference _Comm, fused_gemm_a2a.py:71-160)."""

    _instances = {}

    @classmethod
    def get(cls, group):
        if group is None:
            group = dist.group.WORLD      # one runtime per group, however the default group is spelled
        slot = (group, torch.cuda.current_device())
        existing = cls._instances.get(slot)
        if existing is not None:
            return existing
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError('Create FusedGemmA2AWorkspace before capture to initialize communication')
        created = cls._instances[slot] = cls(group)
        return created

    def __init__(self, group):
        self.group = group if group is not None else dist.group.WORLD
        self.p = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        validate_peer_count(self.p)
        if torch.cuda.get_device_capability()[0] != 10:
            raise ValueError('These kernels target SM100/Blackwell GPUs')
        _native.lib()  # fail here, loudly, if the CUDA library was never built
        self.device = torch.device('cuda', torch.cuda.current_device())
        self.status = self._words(4)      # {code, where, detail, 0} of the first bounded wait that expired
        self.progress = self._words(1)    # row tile the recv GEMM has reached (pusher pacing)
        self.compiled = {}                # launch plans by geometry (nothing is compiled; kept for introspection)
        self.pool = {}
        self.projection_buffers = {}
        self._allocations = []            # (backend, local address, addresses as seen from here, mapped bytes)
        self._status_host = torch.zeros(4, dtype=torch.int32)    # host mirror of the status word
        if self.status.is_cuda:
            self._status_host = self._status_host.pin_memory()
        self._status_event, self._status_posted, self._forwards = None, False, 0
        self.symm_backend = SYMM_BACKEND if SYMM_BACKEND != 'auto' else None   # None: decided by the first allocation
        self.flags, self.peer_flags = self.symmetric((self.p,), torch.int64)
        self.epoch = self._words(1)
        torch.cuda.synchronize()
        dist.barrier(self.group)
        _drain_at_exit(self)

    def _words(self, count):
        return torch.zeros(count, dtype=torch.int32, device=self.device)

    # -- symmetric memory ------------------------------------------------------------------
    def symmetric_bytes(self, nbytes):
        """Allocate `nbytes` of zeroed device memory, map it into every peer and return
        (local address, list of P addresses of the same buffer as seen from this rank). Collective."""
        backend = self.symm_backend
        if backend is None:                       # FGA_SYMM=auto: the group's first allocation decides
            mapping = self._map_everywhere_vmm(nbytes, required=False)
            backend = self.symm_backend = 'vmm' if mapping is not None else 'ipc'
            if mapping is None:
                if self.rank == 0:
                    warnings.warn('fused_gemm_a2a: symmetric memory falls back to cudaMalloc + CUDA IPC '
                                  f'({_native.lib().fga_last_error().decode(errors="replace")}); with it a '
                                  'rank that exits alone invalidates buffers its peers may still write to')
                mapping = self._map_everywhere_ipc(nbytes)
        elif backend == 'vmm':
            mapping = self._map_everywhere_vmm(nbytes, required=True)
        else:
            mapping = self._map_everywhere_ipc(nbytes)
        local, seen, mapped = mapping
        self._allocations.append((backend, local, list(seen), mapped))
        if not self._everyone(all(address and address % 16 == 0 for address in seen)):
            raise RuntimeError('Peer buffers must be aligned and GPU-addressable')
        return local, seen

    def _everyone(self, fine):
        """True when `fine` holds on every rank of the group (one small all-reduce)."""
        if self.p == 1:
            return bool(fine)
        verdict = torch.tensor(int(bool(fine)), device=self.device)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
        return bool(verdict.item())

    def _map_everywhere_ipc(self, nbytes):
        """cudaMalloc + one 64-byte CUDA IPC handle per rank."""
        lib, ct = _native.lib(), _native.ctypes
        local, handle, problem = _native.c_void_p(), ct.create_string_buffer(_HANDLE_BYTES), None
        try:
            _native.check(lib.fga_symm_alloc(nbytes, ct.byref(local)))
            if self.p > 1:
                _native.check(lib.fga_symm_export(local, handle))
        except Exception as error:                 # noqa: BLE001  (the verdict must reach the all-reduce)
            problem = error
        if not self._everyone(problem is None):    # nobody enters the exchange unless everybody can
            if local.value:
                lib.fga_symm_free(local)
            raise RuntimeError(f'Symmetric memory ({nbytes} bytes) could not be allocated on every rank '
                               f'(rank {self.rank}: {problem!r})')
        if self.p == 1:
            return local.value, [local.value], nbytes

        def open_peer(raw):
            remote = _native.c_void_p()
            _native.check(lib.fga_symm_open(raw, ct.byref(remote)))
            return remote.value

        return local.value, exchange_handles(self.group, self.rank, self.p, handle.raw, local.value, open_peer), nbytes

    def _map_everywhere_vmm(self, nbytes, required):
        """Driver VMM allocation + one POSIX file descriptor per rank; every mapping keeps the
        physical memory alive. Two collective steps, each followed by a group-wide verdict so that
        all ranks succeed or give up together: allocate and export locally; pass the descriptors
        around and map the peers' memory. On failure everything this rank mapped is released and
        the result is None, or RuntimeError when `required`."""
        lib, ct = _native.lib(), _native.ctypes
        local, descriptor, size, problem = _native.c_void_p(), ct.c_int(-1), -1, None
        try:
            size = lib.fga_symm_vmm_size(nbytes)
            if size < 0:
                _native.check(-3)
            _native.check(lib.fga_symm_alloc_vmm(nbytes, ct.byref(local), ct.byref(descriptor)))
            # The memory must also be usable as a tensor (torch looks the pointer up with the runtime
            # before it adopts it): read the zero fill back through the same wrapper the slabs use.
            if int(_wrap(local.value, min(nbytes, 4096), self.device).sum()) != 0:
                raise RuntimeError('a fresh VMM allocation did not read back as zeros')
        except Exception as error:                 # noqa: BLE001  (the verdict must reach the all-reduce)
            problem = error
        seen, opened = [local.value], []          # opened: peers' memory mapped by this rank
        allocated_everywhere = self._everyone(problem is None)
        if allocated_everywhere and self.p > 1:
            seen = []
            try:
                for owner, received in enumerate(
                        exchange_descriptors(self.group, self.rank, self.p, descriptor.value)):
                    if owner == self.rank:
                        seen.append(local.value)
                        continue
                    remote = _native.c_void_p()
                    try:
                        _native.check(lib.fga_symm_open_vmm(received, size, ct.byref(remote)))
                    finally:
                        os.close(received)
                    opened.append(remote.value)
                    seen.append(remote.value)
            except Exception as error:             # noqa: BLE001
                problem = error
            mapped_everywhere = self._everyone(problem is None)
        else:
            mapped_everywhere = allocated_everywhere
        if descriptor.value >= 0:
            os.close(descriptor.value)
        if mapped_everywhere:
            return local.value, seen, size
        for address in opened:                     # undo the partial work of this rank
            lib.fga_symm_release_vmm(address, size)
        if local.value:
            lib.fga_symm_release_vmm(local.value, size)
        if required:
            raise RuntimeError(f'FGA_SYMM=vmm: symmetric memory could not be set up on every rank ({problem!r})')
        return None

    def release(self):
        """Give every symmetric buffer of this group back. Collective: all ranks synchronize their
        device and meet first, so that nobody still stores into memory that is about to be unmapped;
        then each rank unmaps its peers' buffers and frees its own. Workspaces, views and tensors
        that came from this object must not be used afterwards; the next workspace of the group
        builds a new runtime."""
        torch.cuda.synchronize()
        dist.barrier(self.group)
        lib = _native.lib()
        for backend, local, seen, mapped in self._allocations:
            for owner, address in enumerate(seen):
                if owner == self.rank:
                    continue
                _native.check(lib.fga_symm_release_vmm(address, mapped) if backend == 'vmm'
                              else lib.fga_symm_close(address))
            _native.check(lib.fga_symm_release_vmm(local, mapped) if backend == 'vmm' else lib.fga_symm_free(local))
        self._allocations.clear()
        self.pool.clear()
        self.projection_buffers.clear()
        for slot in [slot for slot, comm in type(self)._instances.items() if comm is self]:
            del type(self)._instances[slot]
        if self in _live_comms:
            _live_comms.remove(self)
        dist.barrier(self.group)

    def _allocate(self, nbytes):
        base, peer_bases = self.symmetric_bytes(nbytes)
        return _Slab(base, nbytes, peer_bases, self.device)

    def symmetric(self, shape, dtype):
        """A zeroed symmetric tensor and the int64 device table of its address on every peer."""
        nbytes = max(16, _numel(shape) * _itemsize(dtype))
        return self._allocate(nbytes).region(0, shape, dtype)

    def slab(self, layout):
        """One symmetric allocation carved into named sub-buffers. layout: [(name, shape, dtype)].
        Returns {name: (tensor, peer address table)}; a single handle exchange serves them all."""
        placed, total = slab_offsets(layout)
        memory = self._allocate(total)
        return {name: memory.region(offset, shape, dtype)
                for (name, shape, dtype), (offset, _) in zip(layout, placed)}

    def pooled(self, key, shape, dtype):
        slot = (key, tuple(shape), dtype)
        if slot not in self.pool:
            self.pool[slot] = self.symmetric(shape, dtype)
        return self.pool[slot]

    # -- synchronization -------------------------------------------------------------------
    def barrier(self, bump=False, epoch=None, counters=None):
        """Device-side group barrier on the current stream. bump=True first zeroes `counters` and
        afterwards advances `epoch` (a receive buffer's invocation counter)."""
        advanced = None
        if bump:
            advanced = self.epoch if epoch is None else epoch
        device_barrier(self.flags, self.peer_flags, self.rank, self.p, self.status, bump=bump,
                       counters=counters, epoch=advanced)

    @staticmethod
    def _raise_for(word):
        code, where, detail = word[0], word[1], word[2]
        if code:
            reason = _native.DEVICE_ERRORS.get(code, 'unknown device error')
            raise RuntimeError(f'Fused GEMM/A2A device error {code}: {reason} (where={where}, detail={detail}). '
                               'Outputs and gradients produced since then are not valid; repair or tear down '
                               'the CP group, then call clear_status()')

    def check_status(self):
        """Synchronize and raise if any kernel of this group (or an MXFP8 weight gradient launched
        outside a group on this device) gave up on a bounded wait."""
        self._raise_for(self.status.tolist())
        local = _k._local_status.get(self.device)
        if local is not None:
            self._raise_for(local.tolist())

    def clear_status(self):
        """Zero the status word once a device error has been dealt with. The word is sticky: while
        it holds a code, barriers and fused GEMMs of this group return at entry without touching any
        peer's memory, because the peer that never answered may have unmapped it.

        Collective over the group when it has more than one rank: a barrier that returned at entry did
        not advance this rank's epoch, so the ranks' epochs may differ by the number of barriers each
        of them skipped, and a rank that is behind would sail through its next barriers on its peers'
        older, higher flags. All ranks therefore drain their devices, meet on the host, zero their
        barrier flags (every rank starts again from epoch 1) and meet again. Only meaningful while
        every rank of the group is still alive; after a rank has died the group has to be rebuilt."""
        if self.p > 1:
            torch.cuda.synchronize()
            dist.barrier(self.group)
            self.flags.zero_()
            torch.cuda.synchronize()
            dist.barrier(self.group)
        self.status.zero_()
        self._status_host.zero_()
        self._status_posted = False
        local = _k._local_status.get(self.device)
        if local is not None:
            local.zero_()

    def post_status(self):
        """Queue a copy of the status word into pinned host memory behind the work issued so far
        on the current stream (no synchronization; skipped during graph capture). Called at the end
        of every backward pass; poll_status() looks at the copy later."""
        if torch.cuda.is_current_stream_capturing():
            return
        if self._status_event is None:
            self._status_event = torch.cuda.Event()
        self._status_host.copy_(self.status, non_blocking=True)
        self._status_event.record()
        self._status_posted = True

    def poll_status(self):
        """Raise if a copy queued by post_status() has arrived and shows a device error; never
        waits. Called at the start of every forward pass, so a step that ran on after a timed-out
        wait (its kernels return at entry and leave their outputs unwritten) is reported at the next
        step at the latest. Graph replays run no Python: call check_status() once per step there."""
        self._forwards += 1
        capturing = torch.cuda.is_current_stream_capturing()
        if CHECK_STATUS_EVERY and not capturing and self._forwards % CHECK_STATUS_EVERY == 0:
            self.check_status()
        if self._status_posted and not capturing and self._status_event.query():
            self._status_posted = False
            self._raise_for(self._status_host.tolist())

    @staticmethod
    def push_split(a, num_in, p):
        return push_split(a.shape[1], p, num_in, PUSH_SPLIT)

    # -- GEMM dispatch ---------------------------------------------------------------------
    def gemm(self, mode, a, b, b_is_kn, c, aux, counters, num_in, n_segment, num_segments,
             srcs=(0, 0, 0, 0), a_rows=None, head_dim=0, bias=None, src_rows=None, scales=(),
             roles=3):
        """Launch one fused GEMM on the current stream (reference _Comm.gemm, fused_gemm_a2a.py:162-234).

        push: a [M, K] x b -> stored tile by tile into the peers' head-side buffers `aux` (one
              int64 peer table per segment); rows of a beyond M up to a_rows count as zero.
        recv: a is this rank's receive buffer [rows, K]; `srcs` are the addresses of the head-side
              inputs that this kernel's pusher warps distribute to the peers (aux = [peer receive
              buffers, peer counters]); c [rows, N] is the local output.
        b is [N, K] or, with b_is_kn, [K, N]."""
        if mode not in ('push', 'recv'):
            raise ValueError('GEMM mode must be push/recv and tile N must divide output width')
        if not all(t.is_contiguous() for t in (a, b, c)):
            raise ValueError('Fused kernels need contiguous tensors')
        rows, depth = a.shape
        padded = rows if a_rows is None else a_rows
        logical = rows if src_rows is None else src_rows
        if not 1 <= logical <= rows:
            raise ValueError('Receive source rows must be positive and fit the receive buffer')
        if scales:
            # MXFP8 (reference fused_gemm_a2a.py:163, 187-192): a and b are E4M3 payloads written by
            # mxfp8_quantize, scales = (a's scale bytes, b's); b is always [N, K] then. Quantization
            # pads b's rows, so the output width comes from the segments (push) or from c (recv).
            if b_is_kn or len(scales) != 2:
                raise ValueError('MXFP8 operands are K-major payloads with one scale tensor each')
            self._gemm_mx(mode, a, b, c, aux, counters, num_in, n_segment, num_segments, list(srcs), padded,
                          head_dim, bias, logical, scales, roles)
            return
        if padded < rows or padded % _ROW_TILE or (mode == 'recv' and padded != rows):
            raise ValueError('a_rows must be a tile multiple >= the rows of a, and equal to them in recv mode')
        width = b.shape[1] if b_is_kn else b.shape[0]
        if mode == 'push':
            tile_n = MMA_N if num_segments > 1 else MMA_N_OUT_PUSH
            routed = num_segments
        else:  # the kernel narrows its output tile when 256 does not divide the width
            tile_n = MMA_N if width % MMA_N_RECV else MMA_N_RECV
            routed = num_in
        validate_tile_n(mode, tile_n, width, self.p, n_segment, routed, head_dim)
        if bias is not None and not (mode == 'push' and tuple(bias.shape) == (width,) and bias.dtype == torch.bfloat16):
            raise ValueError('GEMM bias requires push mode and a BF16 vector of output-width entries')
        tables_ok = all(len(table) == self.p for table in aux)
        if not tables_ok or (mode == 'recv' and counters.numel() != c.shape[0] // CTA_M):
            raise ValueError('Peer pointer arrays must have P entries and counters one per row block')
        plan = (mode, tuple(a.shape), padded, tuple(b.shape), b_is_kn, tuple(c.shape), num_in, n_segment,
                num_segments, bias is not None, logical != rows)
        self.compiled.setdefault(plan, len(self.compiled))
        if mode == 'push':
            self._launch_push(a, padded, b, b_is_kn, bias, aux[:num_segments], n_segment, c.shape[0] // self.p)
        else:
            self._launch_recv(a, b, b_is_kn, width, c, aux, counters, list(srcs)[:num_in], logical, roles)

    def _gemm_mx(self, mode, aq, bq, c, aux, counters, num_in, n_segment, num_segments, srcs, a_rows,
                 head_dim, bias, src_rows, scales, roles):
        """The MXFP8 launches behind gemm(scales=...). push: aq [pad256(M), Kp] x bq [pad(N), Kp].
        recv: aq is the local E4M3 copy of the receive buffer that the kernel's quantizer warps
        fill; the BF16 receive buffer itself is this rank's entry of the peer table aux[0]."""
        lib, stream = _native.lib(), torch.cuda.current_stream().cuda_stream
        sa, sb = scales
        if mode == 'push':
            width = n_segment * num_segments
            validate_tile_n('push', MMA_N_OUT_PUSH if num_segments == 1 else MMA_N, width, self.p,
                            n_segment, num_segments, head_dim)
            if bias is not None and not (tuple(bias.shape) == (width,) and bias.dtype == torch.bfloat16):
                raise ValueError('GEMM bias requires push mode and a BF16 vector of output-width entries')
            tables = _native.ptr_array([table.data_ptr() for table in aux[:num_segments]])
            _native.check(lib.fga_gemm_push_mx(
                aq.data_ptr(), sa.data_ptr(), aq.shape[0], aq.shape[1], a_rows, bq.data_ptr(), sb.data_ptr(),
                bq.shape[0], bias.data_ptr() if bias is not None else 0, num_segments, n_segment, tables,
                c.shape[0] // self.p, self.rank, self.p, self.status.data_ptr(), _k.DEVICE_TIMEOUT_NS, stream))
            return
        if bias is not None:
            raise ValueError('GEMM bias requires push mode and a BF16 vector of output-width entries')
        peer_recv, peer_counters = aux[0], aux[1]
        rows, k = aq.shape
        if a_rows != rows or counters.numel() != c.shape[0] // CTA_M:
            raise ValueError('Peer pointer arrays must have P entries and counters one per row block')
        addresses = getattr(peer_recv, 'peer_addresses', None)
        recv_address = addresses[self.rank] if addresses is not None else int(peer_recv[self.rank])
        sources = _native.ptr_array([int(address) for address in srcs[:num_in]])
        split = push_split(k, self.p, num_in, PUSH_SPLIT)
        _native.check(lib.fga_gemm_recv_mx(
            recv_address, aq.data_ptr(), sa.data_ptr(), rows, k, bq.data_ptr(), sb.data_ptr(), bq.shape[0],
            bq.shape[1], c.shape[1], c.data_ptr(), peer_recv.data_ptr(), peer_counters.data_ptr(),
            counters.data_ptr(), sources, num_in, src_rows, split, self.rank, self.p, roles,
            self._pacing_epoch(), self.progress.data_ptr(), self.status.data_ptr(), _k.DEVICE_TIMEOUT_NS, stream))

    def push_gqa(self, a, a_rows, weight, bias, peer_tables, layout, head_rows, scales=()):
        """QKV forward with more query heads than key/value heads: `weight` rows (and `bias`) are grouped
        per key/value head, layout = (kv_heads, q_per_kv, gate); one head-side buffer per kind
        (q, k, v(, gate)), the k and v buffers 1/q_per_kv as wide as the q buffer. With `scales` both
        operands are what mxfp8_quantize made of them (E4M3 payload, padded) and scales = (sa, sb)."""
        kv_heads, q_per_kv, gate = layout
        if not (a.is_contiguous() and weight.is_contiguous()):
            raise ValueError('Fused kernels need contiguous tensors')
        if len(peer_tables) != (4 if gate else 3) or not all(len(table) == self.p for table in peer_tables):
            raise ValueError('Peer pointer arrays must have P entries and counters one per row block')
        tables = _native.ptr_array([table.data_ptr() for table in peer_tables])
        stream = torch.cuda.current_stream().cuda_stream
        bias_address = bias.data_ptr() if bias is not None else 0
        if scales:
            sa, sb = scales
            _native.check(_native.lib().fga_gemm_push_gqa_mx(
                a.data_ptr(), sa.data_ptr(), a.shape[0], a.shape[1], a_rows, weight.data_ptr(), sb.data_ptr(),
                weight.shape[0], bias_address, kv_heads, q_per_kv, int(gate), tables, head_rows, self.rank, self.p,
                self.status.data_ptr(), _k.DEVICE_TIMEOUT_NS, stream))
            return
        _native.check(_native.lib().fga_gemm_push_gqa(
            a.data_ptr(), a.shape[0], a.shape[1], a_rows, weight.data_ptr(), bias_address,
            kv_heads, q_per_kv, int(gate), tables, head_rows, self.rank, self.p, self.status.data_ptr(),
            _k.DEVICE_TIMEOUT_NS, stream))

    def recv_gqa(self, recv, weight, out, peer_recv, peer_counters, counters, inputs, src_rows, layout, roles=3,
                 scales=(), mx=None):
        """QKV dgrad for the same layout: `inputs` are the head-side gradients of q, k, v(, gate), whose
        rows are of different widths; `weight` is [rows of the grouped layout, H]. With `scales` = (sb,)
        the weight is its quantized transpose [pad(H), pad(K)] and mx = (local E4M3 copy of the receive
        buffer, its scale bytes), which the kernel's quantizer warps fill."""
        kv_heads, q_per_kv, gate = layout
        if counters.numel() != out.shape[0] // CTA_M or recv.shape[0] != out.shape[0]:
            raise ValueError('Peer pointer arrays must have P entries and counters one per row block')
        hidden = out.shape[1]
        split = push_split(len(inputs) * hidden, self.p, len(inputs), PUSH_SPLIT)   # sized by the widest input
        sources = _native.ptr_array([t.data_ptr() for t in inputs])
        stream = torch.cuda.current_stream().cuda_stream
        if scales:
            mx_recv, mx_scale = mx
            _native.check(_native.lib().fga_gemm_recv_gqa_mx(
                recv.data_ptr(), mx_recv.data_ptr(), mx_scale.data_ptr(), recv.shape[0], weight.data_ptr(),
                scales[-1].data_ptr(), weight.shape[0], weight.shape[1], out.shape[1], out.data_ptr(),
                peer_recv.data_ptr(), peer_counters.data_ptr(), counters.data_ptr(), sources, kv_heads, q_per_kv,
                int(gate), src_rows, split, self.rank, self.p, roles, self.progress.data_ptr(),
                self.status.data_ptr(), _k.DEVICE_TIMEOUT_NS, stream))
            return
        _native.check(_native.lib().fga_gemm_recv_gqa(
            recv.data_ptr(), recv.shape[0], weight.data_ptr(), out.shape[1], out.data_ptr(), peer_recv.data_ptr(),
            peer_counters.data_ptr(), counters.data_ptr(), sources, kv_heads, q_per_kv, int(gate), src_rows, split,
            self.rank, self.p, roles, self.progress.data_ptr(), self.status.data_ptr(), _k.DEVICE_TIMEOUT_NS,
            stream))

    def _launch_push(self, a, a_rows, b, b_is_kn, bias, peer_tables, n_segment, head_rows):
        tables = _native.ptr_array([table.data_ptr() for table in peer_tables])
        _native.check(_native.lib().fga_gemm_push(
            a.data_ptr(), a.shape[0], a.shape[1], a_rows, b.data_ptr(), int(b_is_kn),
            bias.data_ptr() if bias is not None else 0, len(peer_tables), n_segment, tables, head_rows,
            self.rank, self.p, self.status.data_ptr(), _k.DEVICE_TIMEOUT_NS,
            torch.cuda.current_stream().cuda_stream))

    def _launch_recv(self, recv, b, b_is_kn, width, c, aux, counters, srcs, src_rows, roles):
        peer_recv, peer_counters = aux
        sources = _native.ptr_array([int(address) for address in srcs])
        _native.check(_native.lib().fga_gemm_recv(
            recv.data_ptr(), recv.shape[0], recv.shape[1], b.data_ptr(), int(b_is_kn), width, c.data_ptr(),
            peer_recv.data_ptr(), peer_counters.data_ptr(), counters.data_ptr(), sources, len(srcs),
            src_rows, self.push_split(recv, len(srcs), self.p), self.rank, self.p, roles,
            self._pacing_epoch(), self.progress.data_ptr(), self.status.data_ptr(),
            _k.DEVICE_TIMEOUT_NS, torch.cuda.current_stream().cuda_stream))

    def _pacing_epoch(self):
        """Address of this rank's own barrier flag, a device word that grows with every barrier.
        The C ABI keeps the argument for compatibility; the kernels no longer read it."""
        return self.flags.data_ptr() + 8 * self.rank

    def recv_gemm(self, a, b, b_is_kn, c, peer_recv, peer_counters, counters, num_in, srcs,
                  head_dim=0, src_rows=None):
        """Push head-side inputs to the peers while the GEMM consumes completed row blocks."""
        self.gemm('recv', a, b, b_is_kn, c, [peer_recv, peer_counters], counters, num_in, 0, 1,
                  srcs=srcs, head_dim=head_dim, src_rows=src_rows)


# ----------------------------------------------------------------------------------------------
# Gradients of the parameters
# ----------------------------------------------------------------------------------------------
def _check(t, shape, label):
    shape = tuple(shape)
    if tuple(t.shape) != shape or t.dtype != torch.bfloat16 or not t.is_contiguous():
        raise ValueError(f'{label} must be a contiguous BF16 tensor of shape {shape}, got {tuple(t.shape)}')


_placeholder_grads = {}


def _accumulated(param):
    """Gradient already added to param.main_grad: flag it the Megatron way and hand autograd a
    shape-cached placeholder (zeroed on request) so gradient-ready hooks still fire
    (reference fused_gemm_a2a.py:281-294)."""
    param.grad_added_to_main_grad = True
    slot = (param.device, param.dtype, tuple(param.shape))
    if slot not in _placeholder_grads:
        _placeholder_grads[slot] = torch.empty(param.shape, device=param.device, dtype=param.dtype)
    placeholder = _placeholder_grads[slot]
    if getattr(param, 'zero_out_wgrad', False):
        placeholder.zero_()
    return placeholder.detach()


def _usable_main_grad(main_grad, weight, *, same_device):
    """The accumulating epilogue writes FP32 rows of the weight's shape through 16-byte bulk
    reductions: anything else would be silently truncated or misaligned."""
    return (main_grad.shape == weight.shape and main_grad.dtype == torch.float32
            and main_grad.is_contiguous() and main_grad.data_ptr() % 16 == 0
            and (not same_device or main_grad.device == weight.device))


def _weight_grad(weight, a, b, precision='bf16', status=None):
    """dW = a^T b for a [T, N_out] (dY) and b [T, K]. With a Megatron FP32 `main_grad` the GEMM
    epilogue accumulates straight into it; otherwise a BF16 gradient is returned
    (reference fused_gemm_a2a.py:249-275)."""
    main_grad = getattr(weight, 'main_grad', None)
    into_main_grad = main_grad is not None
    if precision == 'mxfp8':
        if into_main_grad and not _usable_main_grad(main_grad, weight, same_device=True):
            raise ValueError('MXFP8 main_grad must match the weight shape and device, '
                             'with contiguous FP32 storage and 16-byte alignment')
        target = main_grad if into_main_grad else torch.empty_like(weight)
        # Bounded-wait reports go to the group's status word when the caller has one.
        report = {} if status is None else {'status': status}
        mxfp8_wgrad(a, b, target, accumulate=into_main_grad, **report)
        return _accumulated(weight) if into_main_grad else target
    if status is None:
        if dist.is_initialized():
            status = _Comm.get(None).status
        else:
            status = torch.zeros(4, dtype=torch.int32, device=a.device)
    if not into_main_grad:
        return bf16_wgrad(a, b, torch.empty(weight.shape, device=a.device, dtype=a.dtype), status)
    if not _usable_main_grad(main_grad, weight, same_device=False):
        raise ValueError('main_grad must match the weight shape with contiguous, 16-byte aligned FP32 storage')
    bf16_wgrad(a, b, main_grad, status, accumulate=True)
    return _accumulated(weight)


def _bias_grad(bias, dy_rows, accumulate=True, *, use_cute=False):
    """FP32 column sums of the logical rows; written into main_grad when the parameter has one and
    accumulate is set, else returned in the parameter dtype (reference fused_gemm_a2a.py:297-309)."""
    if bias is None:
        return None
    main_grad = getattr(bias, 'main_grad', None) if accumulate else None
    if main_grad is not None:
        reduce_bias_grad(dy_rows, main_grad, accumulate=True)
        return _accumulated(bias)
    return reduce_bias_grad(dy_rows, torch.empty_like(bias))


# ----------------------------------------------------------------------------------------------
# Autograd
# ----------------------------------------------------------------------------------------------
def _as_heads(matrix, head_dim):
    """[rows, heads*D] -> [rows, heads, D] without copying."""
    return matrix.view(-1, matrix.shape[1] // head_dim, head_dim)


def _kind_units(layout):
    """(first unit, units) of q, k, v(, gate) inside one key/value group of a grouped layout."""
    _, q_per_kv, gate = layout
    return [(0, q_per_kv), (q_per_kv, 1), (q_per_kv + 1, 1)] + ([(q_per_kv + 2, q_per_kv)] if gate else [])


def _own_grouped(workspace, comm, tokens, late_bias, head_dim):
    """Ownership copy of the grouped-query head buffers: q (and gate) are wider than k and v, so the
    buffers are copied per width class; a late bias is first gathered, per kind, into the contiguous
    order of this rank's heads of that kind (a few kilobytes), which the copy kernel then adds."""
    kv_heads, q_per_kv, gate = workspace.layout
    kinds = _kind_units(workspace.layout)
    groups = kv_heads // comm.p
    if late_bias is None:
        wide = [0] + ([3] if gate else [])
        owned = {}
        for members in (wide, [1, 2]):
            copies = resize_rank_rows([workspace.heads[kind] for kind in members], comm.p, tokens, copy=True)
            owned.update(zip(members, copies))
        return [owned[kind] for kind in range(len(kinds))]
    per_group = kinds[-1][0] + kinds[-1][1]
    grouped = late_bias.view(kv_heads, per_group, head_dim)[comm.rank * groups:(comm.rank + 1) * groups]
    owned = []
    for kind, (first, units) in enumerate(kinds):
        mine = grouped[:, first:first + units].reshape(-1)
        owned.append(resize_rank_rows([workspace.heads[kind]], comm.p, tokens, copy=True, bias=mine,
                                      head_dim=head_dim, head_offset=0)[0])
    return owned


class _FusedQKV(torch.autograd.Function):
    """x [M, H] -> q, k, v(, gate) each [P*M, N/P, D] (reference fused_gemm_a2a.py:312-353)."""

    @staticmethod
    @record_function('fused_qkv_forward')
    def forward(ctx, x, weight, bias, module, workspace):
        comm = workspace.comm
        early_bias = bias if module.bias_in_gemm else None
        late_bias = bias if (module.apply_bias and not module.bias_in_gemm) else None
        comm.barrier()                      # every rank is done reading the head-side buffers
        workspace.run_push(x, weight, False, module.segments, bias=early_bias)
        comm.barrier()                      # every incoming tile has landed
        ctx.module, ctx.workspace, ctx.tokens, ctx.has_bias = module, workspace, x.shape[0], bias is not None
        ctx.save_for_backward(x, weight, *(() if bias is None else (bias,)))
        # One pass strips the tile padding, applies a late bias and gives the caller storage of its
        # own: the shared buffers are overwritten by the next call of this geometry.
        if workspace.layout is None:
            owned = resize_rank_rows(workspace.heads, comm.p, x.shape[0], copy=True, bias=late_bias,
                                     head_dim=module.head_dim,
                                     head_offset=comm.rank * module.num_heads // comm.p)
        else:
            owned = _own_grouped(workspace, comm, x.shape[0], late_bias, module.head_dim)
        return tuple(_as_heads(t, module.head_dim) for t in owned)

    @staticmethod
    @record_function('fused_qkv_backward')
    def backward(ctx, *head_grads):
        x, weight = ctx.saved_tensors[:2]
        workspace, tokens, module = ctx.workspace, ctx.tokens, ctx.module
        workspace.begin_recv()
        dx = torch.empty(workspace.capacity, x.shape[1], device=x.device, dtype=x.dtype)
        workspace.run_recv([g.contiguous().flatten(1) for g in head_grads], weight, True, dx)
        # The receive buffer now holds this rank's dY in weight-row order; pad rows are not read.
        # Saved-tensor hooks may hand back a plain tensor for the weight, so main_grad and the
        # other parameter metadata are taken from the module's own Parameter.
        dy = workspace.recv[:tokens]
        dw = _weight_grad(module.weight, dy, x, workspace.precision, workspace.comm.status)
        db = _bias_grad(module.bias, dy, module.accumulate_bias_grad) if ctx.has_bias else None
        workspace.comm.post_status()
        return dx[:tokens], dw, db, None, None


class _FusedOutput(torch.autograd.Function):
    """o [P*M, N/P, D] -> y [M, H] (reference fused_gemm_a2a.py:356-392)."""

    @staticmethod
    @record_function('fused_out_forward')
    def forward(ctx, o, weight, bias, module, workspace, tokens):
        workspace.begin_recv()
        y = torch.empty(workspace.capacity, weight.shape[0], device=o.device, dtype=o.dtype)
        workspace.run_recv([o.flatten(1)], weight, False, y)
        ctx.module, ctx.workspace, ctx.tokens, ctx.has_bias = module, workspace, tokens, bias is not None
        # The sequence-side O lives in the shared receive buffer, which the next call of this
        # geometry overwrites; backward needs it for dW, so keep a private copy of the logical rows.
        ctx.save_for_backward(weight, workspace.recv[:tokens].clone())
        y = y[:tokens]
        if module.apply_bias and bias is not None:
            y.add_(bias.view(1, -1))
        return y

    @staticmethod
    @record_function('fused_out_backward')
    def backward(ctx, dy):
        weight, o_seq = ctx.saved_tensors
        workspace, tokens, module = ctx.workspace, ctx.tokens, ctx.module
        comm = workspace.comm
        dy = dy.contiguous()
        comm.barrier()
        workspace.run_push(dy, weight, True, 1)
        # The weight and bias gradients need nothing from the peers: they run between the push and
        # the barrier that waits for everybody's tiles, so a rank that finished its push early
        # computes instead of idling and the remote stores have landed by the time it arrives.
        dw = _weight_grad(module.weight, dy, o_seq, workspace.precision, comm.status)
        db = _bias_grad(module.bias, dy, module.accumulate_bias_grad) if ctx.has_bias else None
        comm.barrier()
        do, = resize_rank_rows(workspace.heads, comm.p, tokens, copy=True)
        comm.post_status()
        return _as_heads(do, module.head_dim), dw, db, None, None, None


# ----------------------------------------------------------------------------------------------
# Buffer sets and their active-length views
# ----------------------------------------------------------------------------------------------
class _ProjectionBuffers:
    """Maximum-capacity buffers of one (capacity, hidden, head_dim, segments) geometry: `segments`
    head-side buffers [P*capacity, H/P], a receive buffer [capacity, segments*H] and its counters,
    all carved from one symmetric slab (reference fused_gemm_a2a.py:395-421)."""

    def __init__(self, comm, capacity, hidden_size, head_dim, segments, kv_hidden=None):
        self.comm, self.capacity, self.head_dim = comm, capacity, head_dim
        self.workspaces = {}              # active-length views by (capacity, precision)
        self.mx_recv = self.mx_scale = None
        # Grouped-query attention (kv_hidden < hidden_size): the k and v buffers are narrower than the
        # q (and gate) buffers, and the receive buffer is as wide as all kinds together.
        grouped = kv_hidden is not None and kv_hidden != hidden_size and segments > 1
        self.layout = (kv_hidden // head_dim, hidden_size // kv_hidden, segments == 4) if grouped else None
        widths = [kv_hidden if grouped and index in (1, 2) else hidden_size for index in range(segments)]
        head_names = [f'head{index}' for index in range(segments)]
        regions = comm.slab([(name, (comm.p * capacity, width // comm.p), torch.bfloat16)
                             for name, width in zip(head_names, widths)] + [
            ('recv', (capacity, sum(widths)), torch.bfloat16),
            ('counters', (capacity // CTA_M,), torch.int32)])
        self.heads, self.peer_heads = map(list, zip(*(regions[name] for name in head_names)))
        self.recv, self.peer_recv = regions['recv']
        self.counters, self.peer_counters = regions['counters']
        self.epoch = torch.zeros(1, dtype=torch.int32, device=comm.device)
        torch.cuda.synchronize()
        dist.barrier(comm.group)

    def init_mxfp8(self):
        """Local (not symmetric) E4M3 copy of the receive buffer and its scale bytes: only BF16
        crosses the links, the quantized operand is produced where it is consumed."""
        if self.mx_recv is not None:
            return
        rows, k = self.recv.shape
        device = self.recv.device
        self.mx_recv = torch.empty((rows, k), device=device, dtype=torch.float8_e4m3fn)
        self.mx_scale = torch.empty((rows * k // 32,), device=device, dtype=torch.uint8)


_quantized_weights = {}


def _quantized_weight(weight, transposed):
    """mxfp8_quantize(weight.T if transposed else weight), through the opt-in cache (see MX_WEIGHT_CACHE)."""
    view = weight.T if transposed else weight
    if not MX_WEIGHT_CACHE or torch.cuda.is_current_stream_capturing():
        return mxfp8_quantize(view)
    slot = (weight.data_ptr(), tuple(weight.shape), transposed)
    version = weight._version
    cached = _quantized_weights.get(slot)
    if cached is None or cached[0] != version:
        cached = _quantized_weights[slot] = (version, mxfp8_quantize(view))
    return cached[1]


class _ProjectionWorkspace:
    """Views of the fixed allocation sized for one invocation's active capacity
    (reference fused_gemm_a2a.py:424-473)."""

    def __init__(self, buffers, capacity, precision):
        comm = buffers.comm
        self.comm, self.capacity, self.precision = comm, capacity, precision
        self.head_dim, self.epoch, self.layout = buffers.head_dim, buffers.epoch, buffers.layout
        blocks = capacity // CTA_M
        self.heads = [head[:comm.p * capacity] for head in buffers.heads]
        self.recv, self.counters = buffers.recv[:capacity], buffers.counters[:blocks]
        self.peer_heads, self.peer_recv, self.peer_counters = (
            buffers.peer_heads, buffers.peer_recv, buffers.peer_counters)
        if precision == 'mxfp8':
            self.mx_recv = buffers.mx_recv[:capacity]
            self.mx_scale = buffers.mx_scale[:capacity * self.recv.shape[1] // 32]

    def run_push(self, a, weight, b_is_kn, segments, bias=None):
        comm = self.comm
        if self.layout is not None and segments > 1:
            if b_is_kn:
                raise ValueError('The grouped-query push takes the weight as [rows, K]')
            if self.precision == 'mxfp8':
                aq, sa = mxfp8_quantize(a)
                wq, sb = _quantized_weight(weight, False)
                comm.push_gqa(aq, self.capacity, wq, bias, self.peer_heads, self.layout, self.capacity, scales=(sa, sb))
                return
            comm.push_gqa(a, self.capacity, weight, bias, self.peer_heads, self.layout, self.capacity)
            return
        width = weight.shape[1] if b_is_kn else weight.shape[0]
        n_segment = width // segments
        if self.precision != 'mxfp8':
            comm.gemm('push', a, weight, b_is_kn, self.heads[0], self.peer_heads, self.counters, 0,
                      n_segment, segments, a_rows=self.capacity, head_dim=self.head_dim, bias=bias)
            return
        # MXFP8: both operands are requantized from BF16 on every call, each along this GEMM's
        # reduction axis (reference fused_gemm_a2a.py:439-448).
        aq, sa = mxfp8_quantize(a)
        wq, sb = _quantized_weight(weight, b_is_kn)
        comm.gemm('push', aq, wq, False, self.heads[0], self.peer_heads, self.counters, 0, n_segment,
                  segments, a_rows=self.capacity, head_dim=self.head_dim, bias=bias, scales=(sa, sb))

    def begin_recv(self):
        self.comm.barrier(bump=True, epoch=self.epoch, counters=self.counters)

    def run_recv(self, inputs, weight, b_is_kn, out, roles=3):
        comm = self.comm
        rows_in = inputs[0].shape[0]
        grouped = self.layout is not None and len(inputs) > 1
        if any(t.shape != inputs[0].shape for t in inputs) and not (
                grouped and all(t.shape[0] == rows_in and t.is_contiguous() for t in inputs)):
            raise ValueError('All head-side inputs must have the same shape')
        if rows_in % comm.p:
            raise ValueError('Head-side rows must divide evenly over CP ranks')
        src_rows = rows_in // comm.p
        if grouped:
            if not b_is_kn:
                raise ValueError('The grouped-query dgrad takes the weight as [K, N]')
            if self.precision == 'mxfp8':
                wq, sb = _quantized_weight(weight, True)
                comm.recv_gqa(self.recv, wq, out, self.peer_recv, self.peer_counters, self.counters, inputs, src_rows,
                              self.layout, roles=roles, scales=(sb,), mx=(self.mx_recv, self.mx_scale))
                return
            comm.recv_gqa(self.recv, weight, out, self.peer_recv, self.peer_counters, self.counters, inputs, src_rows,
                          self.layout, roles=roles)
            return
        if self.precision != 'mxfp8':
            comm.gemm('recv', self.recv, weight, b_is_kn, out, [self.peer_recv, self.peer_counters],
                      self.counters, len(inputs), 0, 1, srcs=[t.data_ptr() for t in inputs],
                      head_dim=self.head_dim, src_rows=src_rows, roles=roles)
            return
        # MXFP8: only BF16 crosses the links; quantizer warps inside the kernel convert each arrived
        # row block into the local E4M3 copy that the GEMM reads (reference fused_gemm_a2a.py:465-470).
        wq, sb = _quantized_weight(weight, b_is_kn)
        comm.gemm('recv', self.mx_recv, wq, False, out, [self.peer_recv, self.peer_counters],
                  self.counters, len(inputs), 0, 1, srcs=[t.data_ptr() for t in inputs],
                  head_dim=self.head_dim, src_rows=src_rows, scales=(self.mx_scale, sb), roles=roles)


# ----------------------------------------------------------------------------------------------
# Public classes
# ----------------------------------------------------------------------------------------------
def _head_dim(hidden_size, num_heads):
    if num_heads <= 0 or hidden_size <= 0 or hidden_size % num_heads:
        raise ValueError('hidden_size must be positive and divisible by num_heads')
    return hidden_size // num_heads


def _one_tile_per_head(head_dim, tile_n):
    """The QKV push routes whole heads: one 128-column tile is one (head, q|k|v|gate) unit."""
    if head_dim != tile_n:
        raise ValueError(f'QKV needs one N tile per head: set FUSED_MMA_N={head_dim}')


@dataclass(frozen=True, eq=False)
class FusedGemmA2AWorkspace:
    """Caller-owned, fixed-capacity communication workspace for the QKV(/gate) and output
    projections. Create it after the CP process group exists and before pipeline receives are
    posted or a CUDA graph is captured; pass the same object to every layer of matching geometry."""

    hidden_size: int
    num_heads: int
    max_local_tokens: int
    cp_group: object = None
    gate: bool = False
    precision: str = "bf16"
    num_kv_heads: int = None          # fewer than num_heads: grouped-query attention (an addition to the reference)
    comm: object = field(init=False, repr=False)
    _buffers: dict = field(init=False, repr=False)

    def __post_init__(self):
        quantized = self.precision == 'mxfp8'
        if not quantized and self.precision != 'bf16':
            raise ValueError('precision must be bf16 or mxfp8')
        if quantized and self.hidden_size != 128 * self.num_heads:
            raise ValueError('Experimental MXFP8 requires head_dim=128')
        capacity = padded_rows(self.max_local_tokens, _ROW_TILE)
        head_dim = _head_dim(self.hidden_size, self.num_heads)
        if not dist.is_initialized():
            raise RuntimeError('Initialize the CP process group before creating FusedGemmA2AWorkspace')
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError('Create FusedGemmA2AWorkspace before CUDA Graph capture')
        group = self.cp_group if self.cp_group is not None else dist.group.WORLD
        peers = dist.get_world_size(group)
        validate_peer_count(peers)
        per_rank_width = self.hidden_size // peers
        if self.num_heads % peers or per_rank_width % MMA_N or per_rank_width % MMA_N_OUT_PUSH:
            raise ValueError('Heads must split over CP with tile-aligned per-rank width')
        _one_tile_per_head(head_dim, MMA_N)
        kv_heads = self.num_kv_heads or self.num_heads
        if kv_heads != self.num_heads:
            if kv_heads < 1 or self.num_heads % kv_heads or kv_heads % peers:
                raise ValueError('Query heads must be a multiple of key/value heads, which must split over CP')
        comm = _Comm.get(group)
        # One buffer set for the QKV(/gate) side and one for the output side, shared by every
        # workspace handle and layer of the same geometry on this group.
        sets = {}
        for segments in (4 if self.gate else 3, 1):
            geometry = (capacity, self.hidden_size, head_dim, segments)
            if segments > 1 and kv_heads != self.num_heads:
                geometry += (kv_heads * head_dim,)
            if geometry not in comm.projection_buffers:
                comm.projection_buffers[geometry] = _ProjectionBuffers(comm, *geometry)
            sets[segments] = comm.projection_buffers[geometry]
            if quantized:
                sets[segments].init_mxfp8()
        for name, value in (('cp_group', group), ('comm', comm), ('_buffers', sets)):
            object.__setattr__(self, name, value)   # the dataclass is frozen for its users

    def _validate(self, module, tensor):
        device = self.comm.device
        weight, bias = module.weight, module.bias
        if self.precision == 'mxfp8' and type(weight) not in (torch.Tensor, nn.Parameter):
            raise TypeError('MXFP8 currently takes BF16 master weights, not quantized Parameter subclasses')
        same_geometry = (weight.shape[1] == self.hidden_size and module.num_heads == self.num_heads
                         and module.segments in self._buffers
                         and getattr(module, 'num_kv_heads', None) in (None, self.num_kv_heads or self.num_heads))
        if not same_geometry:
            raise ValueError('Workspace hidden size, head count and QKV/QKVG mode must match the projection')
        if weight.device != device or torch.cuda.current_device() != device.index:
            raise ValueError('Workspace and projection must use the current CUDA device')
        if tensor.device != device:
            raise ValueError('Input and workspace must use the same CUDA device')
        if bias is not None and not (bias.device == device and bias.is_contiguous()):
            raise ValueError('Bias must be contiguous and on the workspace CUDA device')

    def _view(self, local_tokens, segments):
        """The cached active-length view for `local_tokens`; never allocates device memory."""
        if local_tokens > self.max_local_tokens:
            raise ValueError(f'local_tokens={local_tokens} exceeds max_local_tokens={self.max_local_tokens}')
        buffers = self._buffers[segments]
        active = (padded_rows(local_tokens, _ROW_TILE), self.precision)
        if active not in buffers.workspaces:
            buffers.workspaces[active] = _ProjectionWorkspace(buffers, *active)
        return buffers.workspaces[active]


def _check_workspace(workspace, module, tensor):
    if not isinstance(workspace, FusedGemmA2AWorkspace):
        raise TypeError('Pass an explicitly created FusedGemmA2AWorkspace to forward')
    workspace._validate(module, tensor)


def _agree_on_tokens(comm, tokens):
    """All ranks of the group must call with the same local token count (reference README: equal M
    on every rank). Collective; raises the same ValueError on every rank when they differ."""
    if comm.p == 1 or torch.cuda.is_current_stream_capturing():
        return
    span = torch.tensor([tokens, -tokens], dtype=torch.int64, device=comm.device)
    dist.all_reduce(span, op=dist.ReduceOp.MIN, group=comm.group)
    fewest, most = int(span[0]), -int(span[1])
    if fewest != most:
        raise ValueError(f'All CP ranks must pass the same number of local tokens; this group has {fewest} to {most}')


class _CallerOwnedProjection(nn.Module):
    """What both projections share: weight and bias are caller-owned tensors kept by reference
    (never copied, never initialised), checked once at construction."""

    def _adopt(self, hidden_size, num_heads, weight, bias, apply_bias, accumulate_bias_grad):
        if not isinstance(weight, torch.Tensor):
            raise TypeError('weight must be a caller-provided tensor')
        if not (bias is None or isinstance(bias, torch.Tensor)):
            raise TypeError('bias must be a caller-provided tensor or None')
        self.head_dim = _head_dim(hidden_size, num_heads)
        self.num_heads = num_heads
        self.apply_bias, self.accumulate_bias_grad = apply_bias, accumulate_bias_grad

    def _keep(self, weight, bias, out_rows, hidden_size):
        _check(weight.data, (out_rows, hidden_size), 'weight')
        if bias is not None and (tuple(bias.shape) != (out_rows,) or bias.dtype != torch.bfloat16):
            raise ValueError(f'bias must be a BF16 vector of {out_rows} entries')
        self.weight, self.bias = weight, bias


class FusedQKVProjection(_CallerOwnedProjection):
    """[T/P, H] -> q, k, v [T, heads/P, D] (and gate with gate=True). `weight` is
    [(3 + gate) * H, H] in per-head [q; k; v; gate] row order, `bias` likewise; both are
    caller-owned and kept by reference. apply_bias=False leaves the add to the consumer (dbias is
    still produced); bias_in_gemm=True adds the bias to the FP32 accumulator before the BF16
    rounding; accumulate_bias_grad=False returns dbias in the parameter dtype even when the bias
    has a main_grad (reference fused_gemm_a2a.py:559-607)."""

    weight_layout = 'head_qkvg'

    def __init__(self, hidden_size, num_heads, num_kv_heads=None, *, weight, gate=False, bias=None,
                 apply_bias=True, bias_in_gemm=False, accumulate_bias_grad=True):
        super().__init__()
        if bias_in_gemm and not apply_bias:
            raise ValueError('bias_in_gemm requires apply_bias=True; the consumer must not add bias again')
        self._adopt(hidden_size, num_heads, weight, bias, apply_bias, accumulate_bias_grad)
        self.bias_in_gemm = bias_in_gemm
        self.segments = 4 if gate else 3
        self.num_kv_heads = num_kv_heads or num_heads
        self.n_q = num_heads * self.head_dim
        self.n_kv = self.num_kv_heads * self.head_dim
        if self.n_kv != self.n_q:
            # Grouped-query attention (rejected by the reference's fused modules, fused_gemm_a2a.py:592-593;
            # its unfused baseline supports it): weight rows grouped per key/value head,
            # [q_g0 .. q_g(r-1); k_g; v_g; (gate_g0 .. gate_g(r-1))], Megatron's order of a fused QKV weight.
            if self.num_kv_heads < 1 or num_heads % self.num_kv_heads:
                raise ValueError('Query heads must be a multiple of key/value heads')
            self.weight_layout = 'group_qkvg'
        _one_tile_per_head(self.head_dim, MMA_TILER_MN[1])
        self._keep(weight, bias, self.n_q * (2 if gate else 1) + 2 * self.n_kv, hidden_size)

    def forward(self, x, workspace):
        _check_workspace(workspace, self, x)
        _check(x, (x.shape[0], self.weight.shape[1]), 'x')
        workspace.comm.poll_status()
        if CHECK_TOKENS:
            _agree_on_tokens(workspace.comm, x.shape[0])
        return _FusedQKV.apply(x, self.weight, self.bias, self, workspace._view(x.shape[0], self.segments))


class FusedOutputProjection(_CallerOwnedProjection):
    """[T, heads/P, D] -> [T/P, H] with weight [H, H] (reference fused_gemm_a2a.py:610-648).
    apply_bias=False returns y without the bias (the caller fuses it elsewhere) while dbias is
    still produced."""

    def __init__(self, hidden_size, num_heads, *, weight, bias=None, apply_bias=True,
                 accumulate_bias_grad=True):
        super().__init__()
        self._adopt(hidden_size, num_heads, weight, bias, apply_bias, accumulate_bias_grad)
        self.segments = 1
        self._keep(weight, bias, hidden_size, hidden_size)

    def forward(self, o, workspace):
        _check_workspace(workspace, self, o)
        peers = workspace.comm.p
        local_heads = self.weight.shape[0] // peers // self.head_dim
        _check(o, (o.shape[0], local_heads, self.head_dim), 'o')
        if o.shape[0] % peers:
            raise ValueError('Token count must be divisible by CP')
        tokens = o.shape[0] // peers
        workspace.comm.poll_status()
        if CHECK_TOKENS:
            _agree_on_tokens(workspace.comm, tokens)
        return _FusedOutput.apply(o, self.weight, self.bias, self, workspace._view(tokens, 1), tokens)
