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
done by libfga.so through its C ABI: symmetric buffers are cudaMalloc'ed once per geometry and
mapped into every peer with CUDA IPC handles exchanged once over the CP group; the GEMMs are
hand-written TMA/tcgen05 kernels whose epilogue (push) or pusher warps (receive) perform the
all-to-all over NVLink. No kernel is compiled at run time and nothing falls back to the CPU.
"""
import os
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

__all__ = ['FusedGemmA2AWorkspace', 'FusedQKVProjection', 'FusedOutputProjection']

# The reference selects between torch's GEMM + add_ and Megatron's accumulating cuBLAS extension
# for the BF16 weight gradient (fused_gemm_a2a.py:34-40). Here both settings mean the same thing:
# the GEMM epilogue adds straight into main_grad, so no extension is imported. The variable is
# still validated so that a launch script written for the reference fails the same way.
WGRAD_BACKEND = os.environ.get('FUSED_WGRAD_BACKEND', 'torch')
if WGRAD_BACKEND not in ('torch', 'fused_accum'):
    raise ValueError('FUSED_WGRAD_BACKEND must be torch or fused_accum')

_ALIGN = 1024  # every sub-buffer of a symmetric slab starts on a 1 KiB boundary


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
    offsets, total = [], 0
    for _, shape, dtype in layout:
        count = 1
        for extent in shape:
            count *= extent
        nbytes = count * torch.empty(0, dtype=dtype).element_size()
        offsets.append((total, nbytes))
        total += (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
    return offsets, total


def exchange_handles(group, rank, peers, handle, local_address, open_peer):
    """All-gather one 64-byte memory handle per rank over the CP group (the only collective of a
    buffer's lifetime) and map every peer's allocation: returns the P addresses under which this
    rank reaches each rank's buffer, its own through `local_address`."""
    gathered = [None] * peers
    dist.all_gather_object(gathered, (rank, bytes(handle)), group=group)
    addresses = []
    for peer, (sender, raw) in enumerate(gathered):
        if sender != peer or len(raw) != 64:
            raise RuntimeError('Memory handle exchange returned a malformed entry')
        addresses.append(local_address if peer == rank else open_peer(raw))
    return addresses


class _RecvBuffer:
    """Receive side of one pooled geometry: the symmetric buffer, its arrival counters (one per 128
    rows), both with their peer address tables, and the device-side invocation counter."""

    def __init__(self, recv, peer_recv, counters, peer_counters, epoch):
        self.recv, self.peer_recv = recv, peer_recv
        self.counters, self.peer_counters, self.epoch = counters, peer_counters, epoch


class _Comm:
    """Per (process group, device) state: rank, barrier flags, the device status word and the pool
    of symmetric allocations. Layers of equal geometry share buffers, so the footprint does not
    grow with depth (reference _Comm, fused_gemm_a2a.py:71-160)."""

    _instances = {}

    @classmethod
    def get(cls, group):
        key = (group, torch.cuda.current_device())
        if key not in cls._instances:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError('Create FusedGemmA2AWorkspace before capture to initialize communication')
            cls._instances[key] = cls(group)
        return cls._instances[key]

    def __init__(self, group):
        self.group = dist.group.WORLD if group is None else group
        self.rank, self.p = dist.get_rank(self.group), dist.get_world_size(self.group)
        validate_peer_count(self.p)
        if torch.cuda.get_device_capability()[0] != 10:
            raise ValueError('These kernels target SM100/Blackwell GPUs')
        _native.lib()  # fail here, loudly, if the CUDA library was never built
        self.device = torch.device('cuda', torch.cuda.current_device())
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.progress = torch.zeros(1, dtype=torch.int32, device=self.device)  # GEMM progress for pusher pacing
        self.compiled = {}   # launch plans by geometry (nothing is compiled; kept for introspection)
        self.pool = {}
        self.projection_buffers = {}
        self._allocations = []
        self.flags, self.peer_flags = self.symmetric((self.p,), torch.int64)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize()
        dist.barrier(self.group)

    # -- symmetric memory ------------------------------------------------------------------
    def symmetric_bytes(self, nbytes):
        """Allocate `nbytes` of zeroed device memory, map it into every peer and return
        (local address, list of P addresses of the same buffer as seen from this rank)."""
        lib = _native.lib()
        base = _native.c_void_p()
        _native.check(lib.fga_symm_alloc(nbytes, _native.ctypes.byref(base)))
        self._allocations.append(base.value)
        addresses = [base.value] * self.p
        if self.p > 1:
            handle = _native.ctypes.create_string_buffer(64)
            _native.check(lib.fga_symm_export(base, handle))

            def open_peer(raw):
                mapped = _native.c_void_p()
                _native.check(lib.fga_symm_open(raw, _native.ctypes.byref(mapped)))
                return mapped.value

            addresses = exchange_handles(self.group, self.rank, self.p, handle.raw, base.value, open_peer)
        valid = torch.tensor(int(all(a and a % 16 == 0 for a in addresses)), device=self.device)
        if self.p > 1:
            dist.all_reduce(valid, op=dist.ReduceOp.MIN, group=self.group)
        if not valid.item():
            raise RuntimeError('Peer buffers must be aligned and GPU-addressable')
        return base.value, addresses

    def symmetric(self, shape, dtype):
        """A zeroed symmetric tensor and the int64 device table of its address on every peer."""
        count = 1
        for extent in shape:
            count *= extent
        nbytes = max(16, count * torch.empty(0, dtype=dtype).element_size())
        base, addresses = self.symmetric_bytes(nbytes)
        tensor = _wrap(base, nbytes, self.device)[:count * torch.empty(0, dtype=dtype).element_size()]
        tensor = tensor.view(dtype).view(shape)
        return tensor, torch.tensor(addresses, dtype=torch.int64, device=self.device)

    def slab(self, layout):
        """One symmetric allocation carved into named sub-buffers. layout: [(name, shape, dtype)].
        Returns {name: (tensor, peer address table)}; a single handle exchange serves them all."""
        offsets, total = slab_offsets(layout)
        base, addresses = self.symmetric_bytes(total)
        whole = _wrap(base, total, self.device)
        views = {}
        for (name, shape, dtype), (offset, nbytes) in zip(layout, offsets):
            tensor = whole[offset:offset + nbytes].view(dtype).view(shape)
            table = torch.tensor([a + offset for a in addresses], dtype=torch.int64, device=self.device)
            views[name] = (tensor, table)
        return views

    def pooled(self, key, shape, dtype):
        k = (key, tuple(shape), dtype)
        if k not in self.pool:
            self.pool[k] = self.symmetric(shape, dtype)
        return self.pool[k]

    # -- synchronization -------------------------------------------------------------------
    def barrier(self, bump=False, epoch=None, counters=None):
        """Device-side group barrier on the current stream. bump=True first zeroes `counters` and
        afterwards advances `epoch` (a receive buffer's invocation counter)."""
        device_barrier(self.flags, self.peer_flags, self.rank, self.p, self.status, bump=bump,
                       counters=counters, epoch=(self.epoch if epoch is None else epoch) if bump else None)

    def check_status(self):
        """Synchronize and raise if any kernel of this group gave up on a bounded wait."""
        code, where, detail, _ = self.status.tolist()
        if code:
            reason = _native.DEVICE_ERRORS.get(code, 'unknown device error')
            raise RuntimeError(f'Fused GEMM/A2A device error {code}: {reason} (where={where}, detail={detail})')

    def clear_status(self):
        """Zero the status word once a device error has been dealt with. The word is sticky: while
        it holds a code, barriers and fused GEMMs of this group return at entry without touching any
        peer's memory, because the peer that never answered may have unmapped it."""
        self.status.zero_()

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
        if scales:
            raise NotImplementedError('The block-scaled MXFP8 GEMM is not part of this build yet')
        if mode not in ('push', 'recv'):
            raise ValueError('GEMM mode must be push/recv and tile N must divide output width')
        if not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
            raise ValueError('Fused kernels need contiguous tensors')
        a_rows = a.shape[0] if a_rows is None else a_rows
        src_rows = a.shape[0] if src_rows is None else src_rows
        if src_rows < 1 or src_rows > a.shape[0]:
            raise ValueError('Receive source rows must be positive and fit the receive buffer')
        if a_rows < a.shape[0] or a_rows % MMA_TILER_MN[0] or (mode == 'recv' and a_rows != a.shape[0]):
            raise ValueError('a_rows must be a tile multiple >= the rows of a, and equal to them in recv mode')
        output_width = b.shape[1] if b_is_kn else b.shape[0]
        if mode == 'recv':  # the kernel narrows its output tile when 256 does not divide the width
            tile_n = MMA_N_RECV if output_width % MMA_N_RECV == 0 else MMA_N
        else:
            tile_n = MMA_N_OUT_PUSH if num_segments == 1 else MMA_N
        validate_tile_n(mode, tile_n, output_width, self.p, n_segment,
                        num_segments if mode == 'push' else num_in, head_dim)
        if bias is not None and (mode != 'push' or tuple(bias.shape) != (output_width,)
                                 or bias.dtype != torch.bfloat16):
            raise ValueError('GEMM bias requires push mode and a BF16 vector of output-width entries')
        if any(len(x) != self.p for x in aux) or (mode == 'recv' and counters.numel() != c.shape[0] // CTA_M):
            raise ValueError('Peer pointer arrays must have P entries and counters one per row block')
        key = (mode, tuple(a.shape), a_rows, tuple(b.shape), b_is_kn, tuple(c.shape), num_in, n_segment,
               num_segments, bias is not None, src_rows != a.shape[0])
        self.compiled.setdefault(key, len(self.compiled))
        lib, stream = _native.lib(), torch.cuda.current_stream().cuda_stream
        if mode == 'push':
            tables = _native.ptr_array([t.data_ptr() for t in aux[:num_segments]])
            _native.check(lib.fga_gemm_push(
                a.data_ptr(), a.shape[0], a.shape[1], a_rows, b.data_ptr(), int(b_is_kn),
                0 if bias is None else bias.data_ptr(), num_segments, n_segment, tables,
                c.shape[0] // self.p, self.rank, self.p, self.status.data_ptr(),
                _k.DEVICE_TIMEOUT_NS, stream))
        else:
            split = self.push_split(a, num_in, self.p)
            sources = _native.ptr_array([int(s) for s in list(srcs)[:num_in]])
            _native.check(lib.fga_gemm_recv(
                a.data_ptr(), a.shape[0], a.shape[1], b.data_ptr(), int(b_is_kn), output_width,
                c.data_ptr(), aux[0].data_ptr(), aux[1].data_ptr(), counters.data_ptr(), sources,
                num_in, src_rows, split, self.rank, self.p, roles,
                self.flags.data_ptr() + 8 * self.rank, self.progress.data_ptr(), self.status.data_ptr(),
                _k.DEVICE_TIMEOUT_NS, stream))

    def recv_gemm(self, a, b, b_is_kn, c, peer_recv, peer_counters, counters, num_in, srcs,
                  head_dim=0, src_rows=None):
        """Push head-side inputs to the peers while the GEMM consumes completed row blocks."""
        self.gemm('recv', a, b, b_is_kn, c, [peer_recv, peer_counters], counters, num_in, 0, 1,
                  srcs=srcs, head_dim=head_dim, src_rows=src_rows)


def _check(t, shape, label):
    if tuple(t.shape) != tuple(shape) or t.dtype != torch.bfloat16 or not t.is_contiguous():
        raise ValueError(f'{label} must be a contiguous BF16 tensor of shape {tuple(shape)}, got {tuple(t.shape)}')


_placeholder_grads = {}


def _accumulated(param):
    """Gradient already added to param.main_grad: flag it the Megatron way and hand autograd a
    shape-cached placeholder (zeroed on request) so gradient-ready hooks still fire
    (reference fused_gemm_a2a.py:281-294)."""
    param.grad_added_to_main_grad = True
    key = (param.device, param.dtype, tuple(param.shape))
    dummy = _placeholder_grads.get(key)
    if dummy is None:
        dummy = _placeholder_grads[key] = torch.empty(param.shape, device=param.device, dtype=param.dtype)
    if getattr(param, 'zero_out_wgrad', False):
        dummy.zero_()
    return dummy.detach()


def _weight_grad(weight, a, b, precision='bf16', status=None):
    """dW = a^T b for a [T, N_out] (dY) and b [T, K]. With a Megatron FP32 `main_grad` the GEMM
    epilogue accumulates straight into it; otherwise a BF16 gradient is returned
    (reference fused_gemm_a2a.py:249-275)."""
    main_grad = getattr(weight, 'main_grad', None)
    if precision == 'mxfp8':
        if main_grad is not None and (
                main_grad.shape != weight.shape or main_grad.device != weight.device
                or main_grad.dtype != torch.float32 or not main_grad.is_contiguous()
                or main_grad.data_ptr() % 16):
            raise ValueError('MXFP8 main_grad must match the weight shape and device, '
                             'with contiguous FP32 storage and 16-byte alignment')
        out = torch.empty_like(weight) if main_grad is None else main_grad
        mxfp8_wgrad(a, b, out, accumulate=main_grad is not None)
        return out if main_grad is None else _accumulated(weight)
    if status is None:
        status = _Comm.get(None).status if dist.is_initialized() else torch.zeros(
            4, dtype=torch.int32, device=a.device)
    if main_grad is None:
        return bf16_wgrad(a, b, torch.empty(weight.shape, device=a.device, dtype=a.dtype), status)
    if (main_grad.shape != weight.shape or main_grad.dtype != torch.float32
            or not main_grad.is_contiguous() or main_grad.data_ptr() % 16):
        raise ValueError('main_grad must match the weight shape with contiguous, 16-byte aligned FP32 storage')
    bf16_wgrad(a, b, main_grad, status, accumulate=True)
    return _accumulated(weight)


def _bias_grad(bias, dy_rows, accumulate=True, *, use_cute=False):
    """FP32 column sums of the logical rows; written into main_grad when the parameter has one and
    accumulate is set, else returned in the parameter dtype (reference fused_gemm_a2a.py:297-309)."""
    if bias is None:
        return None
    main_grad = getattr(bias, 'main_grad', None)
    if main_grad is None or not accumulate:
        return reduce_bias_grad(dy_rows, torch.empty_like(bias))
    reduce_bias_grad(dy_rows, main_grad, accumulate=True)
    return _accumulated(bias)


class _FusedQKV(torch.autograd.Function):
    """x [M, H] -> q, k, v(, gate) each [P*M, N/P, D] (reference fused_gemm_a2a.py:312-353)."""

    @staticmethod
    @record_function('fused_qkv_forward')
    def forward(ctx, x, weight, bias, module, workspace):
        comm, tokens = workspace.comm, x.shape[0]
        comm.barrier()                      # every rank is done reading the head-side buffers
        workspace.run_push(x, weight, False, module.segments,
                           bias=bias if module.bias_in_gemm else None)
        comm.barrier()                      # every incoming tile has landed
        ctx.module, ctx.workspace, ctx.tokens = module, workspace, tokens
        ctx.has_bias = bias is not None
        ctx.save_for_backward(*((x, weight) if bias is None else (x, weight, bias)))
        late_bias = bias if (module.apply_bias and not module.bias_in_gemm) else None
        owned = resize_rank_rows(workspace.heads, comm.p, tokens, copy=True, bias=late_bias,
                                 head_dim=module.head_dim,
                                 head_offset=comm.rank * module.num_heads // comm.p)
        return tuple(t.view(-1, t.shape[1] // module.head_dim, module.head_dim) for t in owned)

    @staticmethod
    @record_function('fused_qkv_backward')
    def backward(ctx, *head_grads):
        saved = ctx.saved_tensors
        x, weight = saved[0], saved[1]
        workspace, tokens, module = ctx.workspace, ctx.tokens, ctx.module
        sources = [g.contiguous().flatten(1) for g in head_grads]
        workspace.begin_recv()
        dx = torch.empty(workspace.capacity, x.shape[1], device=x.device, dtype=x.dtype)
        workspace.run_recv(sources, weight, True, dx)
        # The receive buffer now holds this rank's dY in weight-row order; pad rows are not read.
        dy = workspace.recv[:tokens]
        dw = _weight_grad(module.weight, dy, x, workspace.precision, workspace.comm.status)
        db = _bias_grad(module.bias if ctx.has_bias else None, dy, module.accumulate_bias_grad)
        return dx[:tokens], dw, db, None, None


class _FusedOutput(torch.autograd.Function):
    """o [P*M, N/P, D] -> y [M, H] (reference fused_gemm_a2a.py:356-392)."""

    @staticmethod
    @record_function('fused_out_forward')
    def forward(ctx, o, weight, bias, module, workspace, tokens):
        workspace.begin_recv()
        y = torch.empty(workspace.capacity, weight.shape[0], device=o.device, dtype=o.dtype)
        workspace.run_recv([o.flatten(1)], weight, False, y)
        ctx.module, ctx.workspace, ctx.tokens = module, workspace, tokens
        ctx.has_bias = bias is not None
        # The sequence-side O lives in the shared receive buffer, which the next call of this
        # geometry overwrites; backward needs it for dW, so keep a private copy of the logical rows.
        ctx.save_for_backward(weight, workspace.recv[:tokens].clone())
        y = y[:tokens]
        if bias is not None and module.apply_bias:
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
        return do.view(-1, do.shape[1] // module.head_dim, module.head_dim), dw, db, None, None, None


class _ProjectionBuffers:
    """Maximum-capacity buffers of one (capacity, hidden, head_dim, segments) geometry: `segments`
    head-side buffers [P*capacity, H/P], a receive buffer [capacity, segments*H] and its counters,
    all carved from one symmetric slab (reference fused_gemm_a2a.py:395-421)."""

    def __init__(self, comm, capacity, hidden_size, head_dim, segments):
        self.comm, self.capacity, self.head_dim = comm, capacity, head_dim
        self.workspaces = {}
        self.mx_recv = self.mx_scale = None
        layout = [(f'head{i}', (comm.p * capacity, hidden_size // comm.p), torch.bfloat16)
                  for i in range(segments)]
        layout += [('recv', (capacity, segments * hidden_size), torch.bfloat16),
                   ('counters', (capacity // CTA_M,), torch.int32)]
        views = comm.slab(layout)
        self.heads = [views[f'head{i}'][0] for i in range(segments)]
        self.peer_heads = [views[f'head{i}'][1] for i in range(segments)]
        self.recv, self.peer_recv = views['recv']
        self.counters, self.peer_counters = views['counters']
        self.epoch = torch.zeros(1, dtype=torch.int32, device=comm.device)
        torch.cuda.synchronize()
        dist.barrier(comm.group)

    def init_mxfp8(self):
        if self.mx_recv is None:
            rows, k = self.recv.shape
            self.mx_recv = torch.empty((rows, k), device=self.recv.device, dtype=torch.float8_e4m3fn)
            self.mx_scale = torch.empty((rows * k // 32,), device=self.recv.device, dtype=torch.uint8)


class _ProjectionWorkspace:
    """Views of the fixed allocation sized for one invocation's active capacity
    (reference fused_gemm_a2a.py:424-473)."""

    def __init__(self, buffers, capacity, precision):
        comm = buffers.comm
        self.comm, self.capacity, self.head_dim, self.precision = comm, capacity, buffers.head_dim, precision
        self.heads = [buf[:comm.p * capacity] for buf in buffers.heads]
        self.peer_heads = buffers.peer_heads
        self.recv, self.peer_recv = buffers.recv[:capacity], buffers.peer_recv
        self.counters, self.peer_counters = buffers.counters[:capacity // CTA_M], buffers.peer_counters
        self.epoch = buffers.epoch
        if precision == 'mxfp8':
            self.mx_recv = buffers.mx_recv[:capacity]
            self.mx_scale = buffers.mx_scale[:capacity * self.recv.shape[1] // 32]

    def run_push(self, a, weight, b_is_kn, segments, bias=None):
        width = weight.shape[1] if b_is_kn else weight.shape[0]
        if self.precision == 'mxfp8':
            # Both operands are requantized from BF16 on every call, each along this GEMM's
            # reduction axis (reference fused_gemm_a2a.py:439-448).
            aq, sa = mxfp8_quantize(a)
            wq, sb = mxfp8_quantize(weight.T if b_is_kn else weight)
            comm = self.comm
            validate_tile_n('push', MMA_N_OUT_PUSH if segments == 1 else MMA_N, width, comm.p,
                            width // segments, segments, self.head_dim)
            tables = _native.ptr_array([t.data_ptr() for t in self.peer_heads[:segments]])
            _native.check(_native.lib().fga_gemm_push_mx(
                aq.data_ptr(), sa.data_ptr(), aq.shape[0], aq.shape[1], self.capacity, wq.data_ptr(),
                sb.data_ptr(), wq.shape[0], 0 if bias is None else bias.data_ptr(), segments,
                width // segments, tables, self.capacity, comm.rank, comm.p, comm.status.data_ptr(),
                _k.DEVICE_TIMEOUT_NS, torch.cuda.current_stream().cuda_stream))
            return
        self.comm.gemm('push', a, weight, b_is_kn, self.heads[0], self.peer_heads, self.counters, 0,
                       width // segments, segments, a_rows=self.capacity, head_dim=self.head_dim,
                       bias=bias)

    def begin_recv(self):
        self.comm.barrier(bump=True, epoch=self.epoch, counters=self.counters)

    def run_recv(self, inputs, weight, b_is_kn, out, roles=3):
        shape = inputs[0].shape
        if any(t.shape != shape for t in inputs):
            raise ValueError('All head-side inputs must have the same shape')
        if shape[0] % self.comm.p:
            raise ValueError('Head-side rows must divide evenly over CP ranks')
        if self.precision == 'mxfp8':
            # Only BF16 crosses the links; quantizer warps inside the kernel convert each arrived
            # row block into the local E4M3 copy that the GEMM reads (reference fused_gemm_a2a.py:465-470).
            comm = self.comm
            wq, sb = mxfp8_quantize(weight.T if b_is_kn else weight)
            k = self.recv.shape[1]
            split = comm.push_split(self.recv, len(inputs), comm.p)
            sources = _native.ptr_array([t.data_ptr() for t in inputs])
            _native.check(_native.lib().fga_gemm_recv_mx(
                self.recv.data_ptr(), self.mx_recv.data_ptr(), self.mx_scale.data_ptr(), self.capacity, k,
                wq.data_ptr(), sb.data_ptr(), wq.shape[0], wq.shape[1], out.shape[1], out.data_ptr(),
                self.peer_recv.data_ptr(), self.peer_counters.data_ptr(), self.counters.data_ptr(), sources,
                len(inputs), shape[0] // comm.p, split, comm.rank, comm.p, roles,
                comm.flags.data_ptr() + 8 * comm.rank, comm.progress.data_ptr(), comm.status.data_ptr(),
                _k.DEVICE_TIMEOUT_NS, torch.cuda.current_stream().cuda_stream))
            return
        self.comm.gemm('recv', self.recv, weight, b_is_kn, out, [self.peer_recv, self.peer_counters],
                       self.counters, len(inputs), 0, 1, srcs=[t.data_ptr() for t in inputs],
                       head_dim=self.head_dim, src_rows=shape[0] // self.comm.p, roles=roles)


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
    comm: object = field(init=False, repr=False)
    _buffers: dict = field(init=False, repr=False)

    def __post_init__(self):
        if self.precision not in ('bf16', 'mxfp8'):
            raise ValueError('precision must be bf16 or mxfp8')
        if self.precision == 'mxfp8' and self.hidden_size != 128 * self.num_heads:
            raise ValueError('Experimental MXFP8 requires head_dim=128')
        capacity = padded_rows(self.max_local_tokens, MMA_TILER_MN[0])
        if self.num_heads <= 0 or self.hidden_size <= 0 or self.hidden_size % self.num_heads:
            raise ValueError('hidden_size must be positive and divisible by num_heads')
        if not dist.is_initialized():
            raise RuntimeError('Initialize the CP process group before creating FusedGemmA2AWorkspace')
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError('Create FusedGemmA2AWorkspace before CUDA Graph capture')
        group = dist.group.WORLD if self.cp_group is None else self.cp_group
        peers = dist.get_world_size(group)
        validate_peer_count(peers)
        if self.num_heads % peers or (self.hidden_size // peers) % MMA_N or (self.hidden_size // peers) % MMA_N_OUT_PUSH:
            raise ValueError('Heads must split over CP with tile-aligned per-rank width')
        head_dim = self.hidden_size // self.num_heads
        if head_dim != MMA_N:
            raise ValueError(f'QKV needs one N tile per head: set FUSED_MMA_N={head_dim}')
        comm = _Comm.get(group)
        buffers = {}
        for segments in (3 + bool(self.gate), 1):
            key = (capacity, self.hidden_size, head_dim, segments)
            if key not in comm.projection_buffers:
                comm.projection_buffers[key] = _ProjectionBuffers(comm, *key)
            buffers[segments] = comm.projection_buffers[key]
            if self.precision == 'mxfp8':
                buffers[segments].init_mxfp8()
        object.__setattr__(self, 'cp_group', group)
        object.__setattr__(self, 'comm', comm)
        object.__setattr__(self, '_buffers', buffers)

    def _validate(self, module, tensor):
        if self.precision == 'mxfp8' and type(module.weight) not in (torch.Tensor, nn.Parameter):
            raise TypeError('MXFP8 currently takes BF16 master weights, not quantized Parameter subclasses')
        if (module.weight.shape[1] != self.hidden_size or module.num_heads != self.num_heads
                or module.segments not in self._buffers):
            raise ValueError('Workspace hidden size, head count and QKV/QKVG mode must match the projection')
        if module.weight.device != self.comm.device or torch.cuda.current_device() != self.comm.device.index:
            raise ValueError('Workspace and projection must use the current CUDA device')
        if tensor.device != self.comm.device:
            raise ValueError('Input and workspace must use the same CUDA device')
        if module.bias is not None and (module.bias.device != self.comm.device or not module.bias.is_contiguous()):
            raise ValueError('Bias must be contiguous and on the workspace CUDA device')

    def _view(self, local_tokens, segments):
        """The cached active-length view for `local_tokens`; never allocates device memory."""
        if local_tokens > self.max_local_tokens:
            raise ValueError(f'local_tokens={local_tokens} exceeds max_local_tokens={self.max_local_tokens}')
        capacity = padded_rows(local_tokens, MMA_TILER_MN[0])
        buffers = self._buffers[segments]
        key = (capacity, self.precision)
        view = buffers.workspaces.get(key)
        if view is None:
            view = buffers.workspaces[key] = _ProjectionWorkspace(buffers, capacity, self.precision)
        return view


def _check_workspace(workspace, module, tensor):
    if not isinstance(workspace, FusedGemmA2AWorkspace):
        raise TypeError('Pass an explicitly created FusedGemmA2AWorkspace to forward')
    workspace._validate(module, tensor)


class FusedQKVProjection(nn.Module):
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
        if not isinstance(weight, torch.Tensor):
            raise TypeError('weight must be a caller-provided tensor')
        if bias is not None and not isinstance(bias, torch.Tensor):
            raise TypeError('bias must be a caller-provided tensor or None')
        if bias_in_gemm and not apply_bias:
            raise ValueError('bias_in_gemm requires apply_bias=True; the consumer must not add bias again')
        if num_heads <= 0 or hidden_size <= 0 or hidden_size % num_heads:
            raise ValueError('hidden_size must be positive and divisible by num_heads')
        self.apply_bias, self.bias_in_gemm = apply_bias, bias_in_gemm
        self.accumulate_bias_grad = accumulate_bias_grad
        self.segments = 4 if gate else 3
        self.num_heads = num_heads
        self.head_dim = hidden_size // num_heads
        kv_heads = num_kv_heads or num_heads
        self.n_q, self.n_kv = num_heads * self.head_dim, kv_heads * self.head_dim
        if self.n_kv != self.n_q:
            raise NotImplementedError('GQA is not supported yet; Q, K and V must have equal widths')
        if self.head_dim != MMA_TILER_MN[1]:
            raise ValueError(f'QKV needs one N tile per head: set FUSED_MMA_N={self.head_dim}')
        rows = self.segments * self.n_q
        _check(weight.data, (rows, hidden_size), 'weight')
        if bias is not None and (tuple(bias.shape) != (rows,) or bias.dtype != torch.bfloat16):
            raise ValueError(f'bias must be a BF16 vector of {rows} entries')
        self.weight, self.bias = weight, bias

    def forward(self, x, workspace):
        _check_workspace(workspace, self, x)
        _check(x, (x.shape[0], self.weight.shape[1]), 'x')
        return _FusedQKV.apply(x, self.weight, self.bias, self, workspace._view(x.shape[0], self.segments))


class FusedOutputProjection(nn.Module):
    """[T, heads/P, D] -> [T/P, H] with weight [H, H] (reference fused_gemm_a2a.py:610-648).
    apply_bias=False returns y without the bias (the caller fuses it elsewhere) while dbias is
    still produced."""

    def __init__(self, hidden_size, num_heads, *, weight, bias=None, apply_bias=True,
                 accumulate_bias_grad=True):
        super().__init__()
        if not isinstance(weight, torch.Tensor):
            raise TypeError('weight must be a caller-provided tensor')
        if bias is not None and not isinstance(bias, torch.Tensor):
            raise TypeError('bias must be a caller-provided tensor or None')
        if num_heads <= 0 or hidden_size <= 0 or hidden_size % num_heads:
            raise ValueError('hidden_size must be positive and divisible by num_heads')
        self.apply_bias, self.accumulate_bias_grad = apply_bias, accumulate_bias_grad
        self.segments, self.num_heads = 1, num_heads
        self.head_dim = hidden_size // num_heads
        _check(weight.data, (hidden_size, hidden_size), 'weight')
        if bias is not None and (tuple(bias.shape) != (hidden_size,) or bias.dtype != torch.bfloat16):
            raise ValueError(f'bias must be a BF16 vector of {hidden_size} entries')
        self.weight, self.bias = weight, bias

    def forward(self, o, workspace):
        _check_workspace(workspace, self, o)
        hidden, p = self.weight.shape[0], workspace.comm.p
        _check(o, (o.shape[0], hidden // p // self.head_dim, self.head_dim), 'o')
        if o.shape[0] % p:
            raise ValueError('Token count must be divisible by CP')
        tokens = o.shape[0] // p
        return _FusedOutput.apply(o, self.weight, self.bias, self, workspace._view(tokens, 1), tokens)
