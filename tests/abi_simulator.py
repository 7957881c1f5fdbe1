"""A CPU stand-in for libfga.so, for host-layer tests only.

TEST INFRASTRUCTURE. The library has no CPU path and the package never imports this file. It lets
the Python layer (workspace, views, autograd functions) run end to end on CPU ranks under gloo, so
that what the layer does with the C ABI - buffer carving, peer tables, call order, bias placement,
padding, ownership copies, main_grad protocol - can be checked numerically against the oracle
without a GPU, for one rank and for several.

How: every entry point of include/fga.h that the layer reaches is restated here with plain torch
on host memory, following the header's contract (not the CUDA sources):
  * symmetric memory is POSIX shared memory; the 64-byte handle carries its name, so a peer's
    allocation is really mapped into this process and remote stores really land there;
  * a group barrier is a gloo barrier; the recv GEMM's wait for arrival counters is a gloo barrier
    between its pushing half and its computing half (each simulated "kernel" runs to completion
    on the host, so this is the only point where ranks must meet);
  * GEMMs accumulate in FP32 from the BF16 values and round once, the arithmetic of the oracle.
  * MXFP8: the quantizer wrapper remembers which BF16 matrix every quantized operand came from, and
    the block-scaled GEMMs multiply the exact dequantized values of both operands, each quantized
    along the GEMM's reduction axis (oracle/mxfp8_oracle.py); the receive GEMM quantizes what is in
    the receive buffer once all arrivals are in, as the quantizer warps do.
"""
import ctypes
import mmap
import os
from multiprocessing import shared_memory

import torch
import torch.distributed as dist

from host_trace import _TorchShim   # torch as seen from inside the package: the CPU is "the device"

BF16 = torch.bfloat16

# When set (tests/cuda_stage.py sets it while it emulates the capture of a CUDA graph), every simulated
# kernel launch goes through it as launch_hook(function, args, kwargs): a launch is one node of the
# recorded graph and is run again, with the same raw arguments, on every replay.
launch_hook = None


def _meet():
    """Where the simulated ranks must meet. A single process that plays every rank in turn (the
    one-device rank emulation of the GPU tests) has nobody to wait for."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def _as_launch(function):
    def call(*args, **kwargs):
        if launch_hook is not None:
            return launch_hook(function, args, kwargs)
        return function(*args, **kwargs)
    call.__name__ = getattr(function, '__name__', 'launch')
    call.__wrapped__ = function
    return call


def _bytes_at(address, nbytes):
    return (ctypes.c_char * nbytes).from_address(int(address))


def matrix(address, rows, cols, dtype=BF16):
    """A [rows, cols] tensor over raw host memory."""
    itemsize = torch.empty(0, dtype=dtype).element_size()
    return torch.frombuffer(_bytes_at(address, rows * cols * itemsize), dtype=dtype).view(rows, cols)


def table(address, entries):
    return list((ctypes.c_int64 * entries).from_address(int(address)))


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view('uint16')


def mx_product(a, b):
    """a [M, K] x b [N, K]^T with both operands quantized to MXFP8 along K, exact products, FP32 result."""
    from oracle import mxfp8_oracle
    return torch.from_numpy(mxfp8_oracle.mx_matmul(bf16_bits(a), bf16_bits(b))).float()


class SimulatedLibrary:
    def __init__(self, tag):
        self.tag = tag                    # unique per test run: names of the shared segments
        self.segments = []                # SharedMemory objects this process created or opened
        self.created = []
        self.launches = 0
        self.quantized = []               # (payload tensor, BF16 matrix it was quantized from), kept alive
        self.mappings = []                # memory-mapped descriptors of the VMM flavour
        self.released = []                # what the host layer gave back, in order

    @property
    def rank(self):
        return dist.get_rank()            # asked late: the library may be installed before the group exists

    def source_of(self, address):
        for payload, source in reversed(self.quantized):
            if payload.data_ptr() == address:
                return source
        raise KeyError('operand was not produced by the quantizer wrapper')

    def fga_launch_count(self):
        return self.launches

    def fga_last_error(self):
        return b'simulated library: a receive row block did not collect all of its arrivals'

    # ---- symmetric memory
    def _map(self, segment):
        self.segments.append(segment)
        return ctypes.addressof(ctypes.c_char.from_buffer(segment.buf))

    def fga_symm_alloc(self, nbytes, out):
        name = f'{self.tag}_{self.rank}_{len(self.created)}'
        segment = shared_memory.SharedMemory(name=name, create=True, size=max(int(nbytes), 16))
        segment.buf[:] = bytes(len(segment.buf))
        self.created.append(segment)
        out._obj.value = self._map(segment)
        return 0

    def fga_symm_export(self, base, handle):
        index = [ctypes.addressof(ctypes.c_char.from_buffer(s.buf)) for s in self.created].index(base.value)
        name = self.created[index].name.encode()
        ctypes.memmove(handle, name + bytes(64 - len(name)), 64)
        return 0

    def fga_symm_open(self, raw, out):
        out._obj.value = self._map(shared_memory.SharedMemory(name=raw.rstrip(b'\0').decode()))
        return 0

    # The virtual-memory-management flavour: an anonymous memory file per allocation, whose descriptor
    # the host layer passes to the peers exactly as it passes a CUDA shareable handle; each side maps it.
    def fga_symm_vmm_size(self, nbytes):
        return -(-int(nbytes) // mmap.PAGESIZE) * mmap.PAGESIZE

    def _map_descriptor(self, descriptor, size):
        mapping = mmap.mmap(descriptor, size)
        self.mappings.append(mapping)
        return ctypes.addressof(ctypes.c_char.from_buffer(mapping))

    def fga_symm_alloc_vmm(self, nbytes, out, descriptor_out):
        size = self.fga_symm_vmm_size(nbytes)
        descriptor = os.memfd_create(f'{self.tag}_{self.rank}_{len(self.mappings)}')
        os.ftruncate(descriptor, size)
        out._obj.value = self._map_descriptor(descriptor, size)
        descriptor_out._obj.value = descriptor
        return 0

    def fga_symm_open_vmm(self, descriptor, size, out):
        out._obj.value = self._map_descriptor(descriptor, size)
        return 0

    def fga_symm_close(self, address):
        self.released.append(('close', int(address)))
        return 0

    def fga_symm_free(self, address):
        self.released.append(('free', int(address)))
        return 0

    def fga_symm_release_vmm(self, address, size):
        self.released.append(('release', int(address), int(size)))
        return 0

    def close(self, meet=True):
        if meet:
            _meet()             # nobody unmaps while a peer may still store into the segment
        self.segments.clear()
        import gc
        gc.collect()
        for segment in self.created:
            try:
                segment.close()
            except BufferError:        # a tensor still views the mapping; the name is removed all the same
                pass
            try:
                segment.unlink()
            except FileNotFoundError:
                pass

    # ---- kernels without an exchange, on the raw bytes the header describes. The host layer's
    # projections reach these through wrappers that install() replaces wholesale; a program that
    # imports the wrappers from fused_gemm_a2a_kernels itself (tests/cuda_stage.py) lands here.
    @staticmethod
    def _strided(address, rows, cols, pitch, dtype):
        itemsize = torch.empty(0, dtype=dtype).element_size()
        flat = torch.frombuffer(_bytes_at(address, ((rows - 1) * pitch + cols) * itemsize), dtype=dtype)
        return torch.as_strided(flat, (rows, cols), (pitch, 1))

    @_as_launch
    def fga_mx_quantize(self, a, rows, k, stride_row, stride_k, q, sf, rows_padded, k_padded, stream):
        from oracle import mxfp8_oracle
        self.launches += 1
        extent = (rows - 1) * stride_row + (k - 1) * stride_k + 1
        logical = torch.as_strided(torch.frombuffer(_bytes_at(a, extent * 2), dtype=BF16), (rows, k),
                                   (stride_row, stride_k))
        payload, scales = mxfp8_oracle.quantize(bf16_bits(logical), k_multiple=k_padded, row_multiple=rows_padded)
        assert payload.shape == (rows_padded, k_padded)
        torch.frombuffer(_bytes_at(q, rows_padded * k_padded), dtype=torch.uint8).copy_(
            torch.from_numpy(payload).reshape(-1))
        torch.frombuffer(_bytes_at(sf, rows_padded * k_padded // 32), dtype=torch.uint8).copy_(torch.from_numpy(scales))
        return 0

    @_as_launch
    def fga_gemm_local_mx(self, aq, sfa, a_rows_padded, bq, sfb, b_rows_padded, m, n, kp, c, ldc, out_f32, accumulate,
                          status, timeout, stream):
        from oracle import mxfp8_oracle
        self.launches += 1

        def values(payload, scales, rows):
            raw = torch.frombuffer(_bytes_at(payload, rows * kp), dtype=torch.uint8).numpy().reshape(rows, kp)
            factors = torch.frombuffer(_bytes_at(scales, rows * kp // 32), dtype=torch.uint8).numpy()
            return torch.from_numpy(mxfp8_oracle.dequantize(raw, factors, rows, kp).reshape(rows, kp))

        product = (values(aq, sfa, a_rows_padded)[:m] @ values(bq, sfb, b_rows_padded)[:n].t()).float()
        out = self._strided(c, m, n, ldc, torch.float32 if out_f32 else BF16)
        out.copy_(out + product if accumulate else product)
        return 0

    @_as_launch
    def fga_gemm_local(self, a, a_is_km, b, b_is_kn, m, n, k, lda, ldb, c, ldc, out_f32, accumulate, status, timeout,
                       stream):
        self.launches += 1
        left = self._strided(a, k, m, lda, BF16).t() if a_is_km else self._strided(a, m, k, lda, BF16)
        right = self._strided(b, k, n, ldb, BF16).t() if b_is_kn else self._strided(b, n, k, ldb, BF16)
        product = left.float() @ right.float().t()
        out = self._strided(c, m, n, ldc, torch.float32 if out_f32 else BF16)
        out.copy_(out + product if accumulate else product)
        return 0

    @_as_launch
    def fga_copy_rank_rows(self, sources, outputs, segments, peers, rows_in, rows_out, width, bias, head_dim,
                           head_offset, stream):
        from oracle.ulysses_oracle import resize_rank_rows_ref
        self.launches += 1
        tensors = tuple(matrix(sources[i], peers * rows_in, width) for i in range(segments))
        covered = (head_offset * head_dim + width) * segments
        results = resize_rank_rows_ref(tensors, peers, rows_out, head_dim=head_dim, head_offset=head_offset,
                                       bias=matrix(bias, 1, covered)[0] if bias else None)
        for i, result in enumerate(results):
            matrix(outputs[i], peers * rows_out, width).copy_(result)
        return 0

    def fga_bias_grad_scratch_floats(self, rows, width):
        return -(-rows // 256) * width

    @_as_launch
    def fga_bias_grad(self, dy, rows, width, out, out_is_f32, accumulate, scratch, stream):
        from oracle.ulysses_oracle import reduce_bias_grad_ref
        self.launches += 1
        target = matrix(out, 1, width, torch.float32 if out_is_f32 else BF16)[0]
        target.copy_(reduce_bias_grad_ref(matrix(dy, rows, width), target.dtype, previous=target if accumulate else None))
        return 0

    # ---- fused GEMMs (contract: include/fga.h)
    def _route_push(self, product, a_rows, segments, n_segment, tables, head_rows, rank, p):
        """Store a [a_rows, segments*n_segment] BF16 result unit by unit (128 columns = one head of one
        segment) into the head-side buffers of the peers that own the heads."""
        heads_per_rank = n_segment // p // 128
        for unit in range(segments * n_segment // 128):
            head, segment = (unit // segments, unit % segments) if segments > 1 else (unit, 0)
            dest, within = head // heads_per_rank, head % heads_per_rank
            target = matrix(table(tables[segment], p)[dest], p * head_rows, n_segment // p)
            target[rank * head_rows:rank * head_rows + a_rows, within * 128:(within + 1) * 128] = \
                product[:, unit * 128:(unit + 1) * 128]

    @_as_launch
    def fga_gemm_push(self, a, m, k, a_rows, b, b_is_kn, bias, segments, n_segment, tables, head_rows,
                      rank, p, status, timeout, stream):
        self.launches += 1
        n = segments * n_segment
        padded = torch.zeros(a_rows, k, dtype=BF16)
        padded[:m] = matrix(a, m, k)
        weight = matrix(b, k, n).t() if b_is_kn else matrix(b, n, k)
        product = padded.float() @ weight.float().t()
        if bias:
            product = product + matrix(bias, 1, n).float()
        self._route_push(product.to(BF16), a_rows, segments, n_segment, tables, head_rows, rank, p)
        return 0

    @_as_launch
    def fga_gemm_push_mx(self, aq, sfa, a_rows_padded, kp, a_rows, bq, sfb, b_rows_padded, bias, segments,
                         n_segment, tables, head_rows, rank, p, status, timeout, stream):
        self.launches += 1
        n = segments * n_segment
        activations, weight = self.source_of(aq), self.source_of(bq)     # [m, k] and [n, k]
        assert weight.shape[0] == n and activations.shape[1] == weight.shape[1]
        assert a_rows_padded >= a_rows >= activations.shape[0] and b_rows_padded >= n and kp >= weight.shape[1]
        product = torch.zeros(a_rows, n)
        product[:activations.shape[0]] = mx_product(activations, weight)
        if bias:
            product = product + matrix(bias, 1, n).float()
        self._route_push(product.to(BF16), a_rows, segments, n_segment, tables, head_rows, rank, p)
        return 0

    def _push_inputs(self, recv_rows, k, peer_recv, peer_counters, srcs, num_in, src_rows, split, rank, p, roles):
        heads_per_rank = k // (p * num_in * 128)
        for turn in range(p if roles & 2 else 0):
            # One rank pushes at a time: the counter increments below are plain read-modify-writes
            # on memory that every rank maps (the GPU uses atomic reductions).
            if turn != rank:
                _meet()
                continue
            for dest in range(p):
                target = matrix(table(peer_recv, p)[dest], recv_rows, k)
                arrivals = torch.frombuffer(_bytes_at(table(peer_counters, p)[dest], 4 * (recv_rows // 128)),
                                            dtype=torch.int32)
                for t in range(num_in):
                    source = matrix(srcs[t], p * src_rows, heads_per_rank * 128)[dest * src_rows:(dest + 1) * src_rows]
                    for unit in range(heads_per_rank):
                        column = ((rank * heads_per_rank + unit) * num_in + t) * 128
                        target[:src_rows, column:column + 128] = source[:, unit * 128:(unit + 1) * 128]
                        target[src_rows:, column:column + 128] = 0
                    arrivals += split          # `split` jobs per (row block, source, destination)
            _meet()                     # after the last turn: every row block has all its arrivals
        if not roles & 2:
            _meet()

    def _arrived(self, counters, recv_rows, expected, roles):
        own = torch.frombuffer(_bytes_at(counters, 4 * (recv_rows // 128)), dtype=torch.int32)
        return not roles & 2 or bool((own == expected).all())

    @_as_launch
    def fga_gemm_recv(self, recv, recv_rows, k, b, b_is_kn, n, c, peer_recv, peer_counters, counters,
                      srcs, num_in, src_rows, split, rank, p, roles, epoch, progress, status, timeout, stream):
        self.launches += 1
        self._push_inputs(recv_rows, k, peer_recv, peer_counters, srcs, num_in, src_rows, split, rank, p, roles)
        if roles & 1:
            if not self._arrived(counters, recv_rows, p * num_in * split, roles):
                return -2
            weight = matrix(b, k, n).t() if b_is_kn else matrix(b, n, k)
            matrix(c, recv_rows, n)[:] = (matrix(recv, recv_rows, k).float() @ weight.float().t()).to(BF16)
        return 0

    # ---- grouped-query attention (contract: the grouped-query section of include/fga.h)
    @staticmethod
    def _kinds(q_per_kv, gate):
        """(first unit, units) of q, k, v(, gate) inside one key/value group."""
        return [(0, q_per_kv), (q_per_kv, 1), (q_per_kv + 1, 1)] + ([(q_per_kv + 2, q_per_kv)] if gate else [])

    def _route_push_gqa(self, product, a_rows, kv_heads, q_per_kv, gate, tables, head_rows, rank, p):
        kinds = self._kinds(q_per_kv, gate)
        per_group, groups = kinds[-1][0] + kinds[-1][1], kv_heads // p
        for unit in range(kv_heads * per_group):
            group, position = divmod(unit, per_group)
            kind = max(index for index, (first, _) in enumerate(kinds) if position >= first)
            first, units = kinds[kind]
            dest, local = divmod(group, groups)
            column = (local * units + position - first) * 128
            target = matrix(table(tables[kind], p)[dest], p * head_rows, groups * units * 128)
            target[rank * head_rows:rank * head_rows + a_rows, column:column + 128] = product[:, unit * 128:(unit + 1) * 128]

    @_as_launch
    def fga_gemm_push_gqa(self, a, m, k, a_rows, b, bias, kv_heads, q_per_kv, gate, tables, head_rows, rank, p,
                          status, timeout, stream):
        self.launches += 1
        kinds = self._kinds(q_per_kv, gate)
        n = kv_heads * (kinds[-1][0] + kinds[-1][1]) * 128
        padded = torch.zeros(a_rows, k, dtype=BF16)
        padded[:m] = matrix(a, m, k)
        product = padded.float() @ matrix(b, n, k).float().t()
        if bias:
            product = product + matrix(bias, 1, n).float()
        self._route_push_gqa(product.to(BF16), a_rows, kv_heads, q_per_kv, gate, tables, head_rows, rank, p)
        return 0

    @_as_launch
    def fga_gemm_push_gqa_mx(self, aq, sfa, a_rows_padded, kp, a_rows, bq, sfb, b_rows_padded, bias, kv_heads, q_per_kv,
                             gate, tables, head_rows, rank, p, status, timeout, stream):
        self.launches += 1
        kinds = self._kinds(q_per_kv, gate)
        n = kv_heads * (kinds[-1][0] + kinds[-1][1]) * 128
        activations, weight = self.source_of(aq), self.source_of(bq)     # [m, k] and [n, k]
        assert weight.shape[0] == n and activations.shape[1] == weight.shape[1]
        assert a_rows_padded >= a_rows >= activations.shape[0] and b_rows_padded >= n and kp >= weight.shape[1]
        product = torch.zeros(a_rows, n)
        product[:activations.shape[0]] = mx_product(activations, weight)
        if bias:
            product = product + matrix(bias, 1, n).float()
        self._route_push_gqa(product.to(BF16), a_rows, kv_heads, q_per_kv, gate, tables, head_rows, rank, p)
        return 0

    def _push_inputs_gqa(self, recv_rows, peer_recv, peer_counters, srcs, kv_heads, q_per_kv, gate, src_rows, split,
                         rank, p, roles):
        kinds = self._kinds(q_per_kv, gate)
        per_group, groups = kinds[-1][0] + kinds[-1][1], kv_heads // p
        k = kv_heads * per_group * 128
        for turn in range(p if roles & 2 else 0):
            if turn != rank:
                _meet()
                continue
            for dest in range(p):
                target = matrix(table(peer_recv, p)[dest], recv_rows, k)
                arrivals = torch.frombuffer(_bytes_at(table(peer_counters, p)[dest], 4 * (recv_rows // 128)),
                                            dtype=torch.int32)
                for kind, (first, units) in enumerate(kinds):
                    width = groups * units * 128
                    source = matrix(srcs[kind], p * src_rows, width)[dest * src_rows:(dest + 1) * src_rows]
                    for unit in range(groups * units):
                        local, within = divmod(unit, units)
                        column = ((rank * groups + local) * per_group + first + within) * 128
                        target[:src_rows, column:column + 128] = source[:, unit * 128:(unit + 1) * 128]
                        target[src_rows:, column:column + 128] = 0
                    arrivals += split
            _meet()
        if not roles & 2:
            _meet()
        return k, len(kinds)

    @_as_launch
    def fga_gemm_recv_gqa(self, recv, recv_rows, b, n, c, peer_recv, peer_counters, counters, srcs, kv_heads, q_per_kv,
                          gate, src_rows, split, rank, p, roles, progress, status, timeout, stream):
        self.launches += 1
        k, num_in = self._push_inputs_gqa(recv_rows, peer_recv, peer_counters, srcs, kv_heads, q_per_kv, gate, src_rows,
                                          split, rank, p, roles)
        if roles & 1:
            if not self._arrived(counters, recv_rows, p * num_in * split, roles):
                return -2
            matrix(c, recv_rows, n)[:] = (matrix(recv, recv_rows, k).float() @ matrix(b, k, n).float()).to(BF16)
        return 0

    def _quantize_received(self, recv, mx_recv, mx_scale, counters, recv_rows, k):
        """What the quantizer warps leave behind: the E4M3 copy of the receive buffer and its scales (K
        padded to 128), and their 16 completions per row block on the arrival counters."""
        from oracle import mxfp8_oracle
        received = matrix(recv, recv_rows, k)
        payload, scales = mxfp8_oracle.quantize(bf16_bits(received), k_multiple=128)
        torch.frombuffer(_bytes_at(mx_recv, recv_rows * k), dtype=torch.uint8).copy_(
            torch.from_numpy(payload[:recv_rows, :k].copy()).reshape(-1))
        torch.frombuffer(_bytes_at(mx_scale, recv_rows * k // 32), dtype=torch.uint8).copy_(
            torch.from_numpy(scales[:recv_rows * k // 32].copy()))
        own = torch.frombuffer(_bytes_at(counters, 4 * (recv_rows // 128)), dtype=torch.int32)
        own += 16
        return received

    @_as_launch
    def fga_gemm_recv_gqa_mx(self, recv, mx_recv, mx_scale, recv_rows, bq, sfb, b_rows_padded, b_kp, n, c, peer_recv,
                             peer_counters, counters, srcs, kv_heads, q_per_kv, gate, src_rows, split, rank, p, roles,
                             progress, status, timeout, stream):
        self.launches += 1
        k, num_in = self._push_inputs_gqa(recv_rows, peer_recv, peer_counters, srcs, kv_heads, q_per_kv, gate, src_rows,
                                          split, rank, p, roles)
        if roles & 1:
            if not self._arrived(counters, recv_rows, p * num_in * split, roles):
                return -2
            received = self._quantize_received(recv, mx_recv, mx_scale, counters, recv_rows, k)
            weight = self.source_of(bq)
            assert weight.shape == (n, k) and b_rows_padded >= n and b_kp >= k
            matrix(c, recv_rows, n)[:] = mx_product(received, weight).to(BF16)
        return 0

    @_as_launch
    def fga_gemm_recv_mx(self, recv, mx_recv, mx_scale, recv_rows, k, bq, sfb, b_rows_padded, b_kp, n, c,
                         peer_recv, peer_counters, counters, srcs, num_in, src_rows, split, rank, p, roles,
                         epoch, progress, status, timeout, stream):
        from oracle import mxfp8_oracle
        self.launches += 1
        self._push_inputs(recv_rows, k, peer_recv, peer_counters, srcs, num_in, src_rows, split, rank, p, roles)
        if roles & 1:
            if not self._arrived(counters, recv_rows, p * num_in * split, roles):
                return -2
            received = matrix(recv, recv_rows, k)
            # what the quantizer warps leave behind: the E4M3 copy and its scales (K padded to 128)
            payload, scales = mxfp8_oracle.quantize(bf16_bits(received), k_multiple=128)
            torch.frombuffer(_bytes_at(mx_recv, recv_rows * k), dtype=torch.uint8).copy_(
                torch.from_numpy(payload[:recv_rows, :k].copy()).reshape(-1))
            torch.frombuffer(_bytes_at(mx_scale, recv_rows * k // 32), dtype=torch.uint8).copy_(
                torch.from_numpy(scales[:recv_rows * k // 32].copy()))
            own = torch.frombuffer(_bytes_at(counters, 4 * (recv_rows // 128)), dtype=torch.int32)
            own += 16                      # the quantizer warps' completions, 8 rows per job
            weight = self.source_of(bq)
            assert weight.shape == (n, k) and b_rows_padded >= n and b_kp >= k
            matrix(c, recv_rows, n)[:] = mx_product(received, weight).to(BF16)
        return 0


def install(fused, tag):
    """Patch the package to run on the simulated library; returns (library, undo)."""
    import _fga_native
    from oracle.ulysses_oracle import reduce_bias_grad_ref, resize_rank_rows_ref
    sim = SimulatedLibrary(tag)
    names = ('device_barrier', 'resize_rank_rows', 'reduce_bias_grad', 'bf16_wgrad', 'mxfp8_quantize', 'mxfp8_wgrad')
    saved = {name: getattr(fused, name) for name in names}
    saved.update(lib=_fga_native.lib, torch=fused.torch, wrap=fused._wrap)
    _fga_native.lib = lambda: sim
    fused.torch = _TorchShim()
    fused._wrap = lambda address, nbytes, _device: torch.frombuffer(_bytes_at(address, nbytes), dtype=torch.uint8)

    def device_barrier(flags, peer_flags, rank, peers, status, *, bump=False, counters=None, epoch=None):
        sim.launches += 1
        if bump and counters is not None:
            counters.zero_()               # before publishing: nobody can have incremented them yet
        dist.barrier()
        if bump and epoch is not None:
            epoch += 1

    def resize_rank_rows(tensors, peers, rows, *, copy=False, bias=None, head_dim=128, head_offset=0, use_cute=False):
        sim.launches += 1
        return resize_rank_rows_ref(tuple(tensors), peers, rows, bias=bias, head_dim=head_dim, head_offset=head_offset)

    def reduce_bias_grad(dy, out, *, accumulate=False, use_cute=False):
        sim.launches += 1
        out.copy_(reduce_bias_grad_ref(dy, out.dtype, previous=out if accumulate else None))
        return out

    def bf16_wgrad(dy, x, out, status, *, accumulate=False):
        sim.launches += 1
        product = dy.float().t() @ x.float()
        out.copy_((out.float() + product) if accumulate else product)
        return out

    def mxfp8_quantize(a, *, k_multiple=256):
        sim.launches += 1
        rows, k = a.shape
        rp, kp = -(-rows // 256) * 256, -(-k // k_multiple) * k_multiple
        payload = torch.zeros(rp, kp, dtype=torch.float8_e4m3fn)
        sim.quantized.append((payload, a.detach().contiguous().clone()))     # the logical [rows, k] matrix
        return payload, torch.zeros(rp * kp // 32, dtype=torch.uint8)

    def mxfp8_wgrad(dy, x, out, *, accumulate=False, status=None):
        sim.launches += 3                  # two transposing quantizer passes and the GEMM
        product = mx_product(dy.t(), x.t())           # both operands quantized along the token axis
        out.copy_((out.float() + product) if accumulate else product)
        return out

    def requantized(old_outputs, new_outputs):
        # A replayed quantizer launch: its payload tensor stays the one recorded, so the BF16 matrix that
        # the later GEMM launches look up by that address takes the new values.
        _, fresh = sim.quantized.pop()
        for payload, source in sim.quantized:
            if payload.data_ptr() == old_outputs[0].data_ptr():
                source.copy_(fresh)
    mxfp8_quantize.after_replay = requantized

    for fn in (device_barrier, resize_rank_rows, reduce_bias_grad, bf16_wgrad, mxfp8_quantize, mxfp8_wgrad):
        launch = _as_launch(fn)
        if hasattr(fn, 'after_replay'):
            launch.after_replay = fn.after_replay
        setattr(fused, fn.__name__, launch)

    def undo(meet=True):
        sim.close(meet)
        _fga_native.lib = saved['lib']
        fused.torch, fused._wrap = saved['torch'], saved['wrap']
        for name in names:
            setattr(fused, name, saved[name])
        fused._Comm._instances.clear()
        fused._placeholder_grads.clear()

    return sim, undo


def unique_tag():
    return f'fga{os.getpid() % 100000}'
