"""Host-layer call tracing on the CPU.

The Python layer of the package (workspace, buffer views, autograd functions) decides which C-ABI
entry points run, in which order and with which pointers and sizes. This module runs that layer
without a GPU and writes down every call it makes:

* `_fga_native.lib()` is replaced by a recorder. Its symmetric allocator hands out host memory, so
  the layer's slab carving and peer tables are real arithmetic on real addresses, and every pointer
  argument is resolved to "<allocation>+<offset>" (peer tables are read and resolved entry by
  entry).
* the thin kernel wrappers the layer imports (barrier, row copy, bias reduction, quantizer, weight
  gradients) are replaced by recorders that return tensors of the right shape.
* `torch.cuda` and `torch.device` are shimmed inside the package so that "the current CUDA device"
  is the CPU.

Nothing here computes a projection: the trace pins the launch plan, not the numerics (the GPU tests
and the oracle do that). tests/test_host_trace.py compares the trace of a fixed scenario with the
committed one in tests/golden/host_call_trace.json.
"""
import ctypes
import types

import torch
import torch.distributed as dist

PEER_BASE = 1 << 60   # fake addresses of peers' allocations (above any host address): base + (rank << 36) + (index << 28)


class Recorder:
    def __init__(self, rank, peers):
        self.rank, self.peers = rank, peers
        self.calls = []
        self.allocations = []      # (address, size, buffer) of the fake symmetric allocator
        self.named = []            # (address, size, label, tensor) of tensors the scenario registered; the
                                   # reference keeps them alive so that no address is ever reused

    # ---- pointer resolution
    def register(self, label, tensor):
        self.named.append((tensor.data_ptr(), tensor.numel() * tensor.element_size(), label, tensor))
        return tensor

    def resolve(self, address):
        address = int(address or 0)
        if address == 0:
            return 'null'
        for index, (start, size, _) in enumerate(self.allocations):
            if start <= address < start + size:
                return f'symm{index}+{address - start}'
        if address >= PEER_BASE:
            rel = address - PEER_BASE
            return f'peer{rel >> 36}.symm{(rel >> 28) & 0xff}+{rel & 0xfffffff}'
        for start, size, label, _ in self.named:
            if start <= address < start + max(size, 1):
                return f'{label}+{address - start}'
        return 'anon'

    def table(self, address, entries):
        """Contents of an int64 device table (here: host memory), resolved entry by entry."""
        values = (ctypes.c_int64 * entries).from_address(int(address))
        return [self.resolve(v) for v in values]

    def tensor(self, t):
        if t is None:
            return None
        return dict(ptr=self.resolve(t.data_ptr()), shape=list(t.shape), stride=list(t.stride()),
                    dtype=str(t.dtype).replace('torch.', ''))

    def log(self, name, **fields):
        self.calls.append([name, fields])


class FakeLib:
    """Stands in for the ctypes library object: every entry point the host layer calls directly."""

    def __init__(self, rec):
        self.rec = rec

    def fga_symm_alloc(self, nbytes, out):
        buffer = ctypes.create_string_buffer(int(nbytes) + 64)
        address = (ctypes.addressof(buffer) + 63) // 64 * 64
        self.rec.allocations.append((address, int(nbytes), buffer))
        out._obj.value = address
        self.rec.log('fga_symm_alloc', bytes=int(nbytes))
        return 0

    def fga_symm_export(self, base, handle):
        index = [a for a, _, _ in self.rec.allocations].index(base.value)
        payload = bytes([self.rec.rank, index]) + bytes(62)
        ctypes.memmove(handle, payload, 64)
        self.rec.log('fga_symm_export', ptr=self.rec.resolve(base.value))
        return 0

    def fga_symm_open(self, raw, out):
        owner, index = raw[0], raw[1]
        out._obj.value = PEER_BASE + (owner << 36) + (index << 28)
        self.rec.log('fga_symm_open', owner=owner, index=index)
        return 0

    def fga_gemm_push(self, a, m, k, a_rows, b, b_is_kn, bias, segments, n_segment, tables, head_rows,
                      rank, p, status, timeout, stream):
        r = self.rec
        r.log('fga_gemm_push', a=r.resolve(a), m=m, k=k, a_rows=a_rows, b=r.resolve(b), b_is_kn=b_is_kn,
              bias=r.resolve(bias), segments=segments, n_segment=n_segment,
              peer_heads=[r.table(tables[s], p) for s in range(segments)], head_rows=head_rows,
              rank=rank, p=p, status=r.resolve(status))
        return 0

    def fga_gemm_recv(self, recv, recv_rows, k, b, b_is_kn, n, c, peer_recv, peer_counters, counters,
                      srcs, num_in, src_rows, split, rank, p, roles, epoch, progress, status, timeout, stream):
        r = self.rec
        r.log('fga_gemm_recv', recv=r.resolve(recv), recv_rows=recv_rows, k=k, b=r.resolve(b),
              b_is_kn=b_is_kn, n=n, c=r.resolve(c), peer_recv=r.table(peer_recv, p),
              peer_counters=r.table(peer_counters, p), counters=r.resolve(counters),
              srcs=[r.resolve(srcs[t]) for t in range(num_in)], num_in=num_in, src_rows=src_rows,
              split=split, rank=rank, p=p, roles=roles, epoch=r.resolve(epoch),
              progress=r.resolve(progress), status=r.resolve(status))
        return 0

    def fga_gemm_push_mx(self, aq, sfa, a_rows_padded, kp, a_rows, bq, sfb, b_rows_padded, bias, segments,
                         n_segment, tables, head_rows, rank, p, status, timeout, stream):
        r = self.rec
        r.log('fga_gemm_push_mx', a_rows_padded=a_rows_padded, kp=kp, a_rows=a_rows,
              b_rows_padded=b_rows_padded, bias=r.resolve(bias), segments=segments, n_segment=n_segment,
              peer_heads=[r.table(tables[s], p) for s in range(segments)], head_rows=head_rows,
              rank=rank, p=p, status=r.resolve(status))
        return 0

    def fga_gemm_recv_mx(self, recv, mx_recv, mx_scale, recv_rows, k, bq, sfb, b_rows_padded, b_kp, n, c,
                         peer_recv, peer_counters, counters, srcs, num_in, src_rows, split, rank, p, roles,
                         epoch, progress, status, timeout, stream):
        r = self.rec
        r.log('fga_gemm_recv_mx', recv=r.resolve(recv), mx_recv=r.resolve(mx_recv), mx_scale=r.resolve(mx_scale),
              recv_rows=recv_rows, k=k, b_rows_padded=b_rows_padded, b_kp=b_kp, n=n, c=r.resolve(c),
              peer_recv=r.table(peer_recv, p), peer_counters=r.table(peer_counters, p),
              counters=r.resolve(counters), srcs=[r.resolve(srcs[t]) for t in range(num_in)],
              num_in=num_in, src_rows=src_rows, split=split, rank=rank, p=p, roles=roles,
              epoch=r.resolve(epoch), progress=r.resolve(progress), status=r.resolve(status))
        return 0


class _FakeCuda:
    """What the host layer asks torch.cuda: there is one device, it is a B200, nothing captures."""

    @staticmethod
    def current_device():
        return None      # the index of torch.device('cpu')

    @staticmethod
    def get_device_capability(*_):
        return (10, 0)

    @staticmethod
    def is_current_stream_capturing():
        return False

    @staticmethod
    def synchronize(*_):
        return None

    @staticmethod
    def current_stream(*_):
        return types.SimpleNamespace(cuda_stream=0)

    class Event:
        """Host work is done when it returns: a recorded event has always completed."""

        def record(self, *_):
            return None

        @staticmethod
        def query():
            return True


class _TorchShim:
    """`torch` as seen from inside the package: the real module except for cuda and device."""

    cuda = _FakeCuda()

    @staticmethod
    def device(*_args, **_kwargs):
        return torch.device('cpu')

    def __getattr__(self, name):
        return getattr(torch, name)


def _host_tensor(address, nbytes, _device):
    return torch.frombuffer((ctypes.c_char * nbytes).from_address(address), dtype=torch.uint8)


def install(fused, rec):
    """Patch the package for tracing; returns a callable that undoes everything."""
    import _fga_native
    saved = dict(lib=_fga_native.lib, torch=fused.torch, wrap=fused._wrap, backend=fused.SYMM_BACKEND)
    names = ('device_barrier', 'resize_rank_rows', 'reduce_bias_grad', 'bf16_wgrad', 'mxfp8_wgrad', 'mxfp8_quantize')
    saved.update({name: getattr(fused, name) for name in names})
    fake = FakeLib(rec)
    fused.SYMM_BACKEND = 'ipc'      # the recorder's allocator speaks the 64-byte-handle flavour only
    _fga_native.lib = lambda: fake
    fused.torch = _TorchShim()
    fused._wrap = _host_tensor

    def device_barrier(flags, peer_flags, rank, peers, status, *, bump=False, counters=None, epoch=None):
        rec.log('barrier', flags=rec.resolve(flags.data_ptr()), peer_flags=rec.table(peer_flags.data_ptr(), peers),
                rank=rank, p=peers, bump=bool(bump), counters=rec.tensor(counters),
                epoch=None if epoch is None else rec.resolve(epoch.data_ptr()), status=rec.resolve(status.data_ptr()))

    def resize_rank_rows(tensors, peers, rows, *, copy=False, bias=None, head_dim=128, head_offset=0, use_cute=False):
        tensors = tuple(tensors)
        rec.log('resize_rank_rows', inputs=[rec.tensor(t) for t in tensors], peers=peers, rows=rows, copy=bool(copy),
                bias=rec.tensor(bias), head_dim=head_dim, head_offset=head_offset)
        return tuple(torch.zeros(peers * rows, t.shape[1], dtype=t.dtype) for t in tensors)

    def reduce_bias_grad(dy, out, *, accumulate=False, use_cute=False):
        rec.log('reduce_bias_grad', dy=rec.tensor(dy), out=rec.tensor(out), accumulate=bool(accumulate))
        return out

    def bf16_wgrad(dy, x, out, status, *, accumulate=False):
        rec.log('bf16_wgrad', dy=rec.tensor(dy), x=rec.tensor(x), out=rec.tensor(out),
                status=rec.resolve(status.data_ptr()), accumulate=bool(accumulate))
        return out

    def mxfp8_wgrad(dy, x, out, *, accumulate=False, status=None):
        rec.log('mxfp8_wgrad', dy=rec.tensor(dy), x=rec.tensor(x), out=rec.tensor(out), accumulate=bool(accumulate))
        return out

    def mxfp8_quantize(a, *, k_multiple=256):
        rec.log('mxfp8_quantize', a=rec.tensor(a), k_multiple=k_multiple)
        rows, k = a.shape
        rp, kp = (rows + 255) // 256 * 256, (k + k_multiple - 1) // k_multiple * k_multiple
        return torch.zeros(rp, kp, dtype=torch.float8_e4m3fn), torch.zeros(rp * kp // 32, dtype=torch.uint8)

    for fn in (device_barrier, resize_rank_rows, reduce_bias_grad, bf16_wgrad, mxfp8_wgrad, mxfp8_quantize):
        setattr(fused, fn.__name__, fn)

    def undo():
        _fga_native.lib = saved['lib']
        fused.torch, fused._wrap, fused.SYMM_BACKEND = saved['torch'], saved['wrap'], saved['backend']
        for name in names:
            setattr(fused, name, saved[name])
        fused._Comm._instances.clear()
        fused._placeholder_grads.clear()

    return undo


CONFIGS = (dict(gate=False, bias=False, bias_in_gemm=False, main_grad=False, precision='bf16', tokens=(300, 129)),
           dict(gate=True, bias=True, bias_in_gemm=False, main_grad=False, precision='bf16', tokens=(300,)),
           dict(gate=False, bias=True, bias_in_gemm=True, main_grad=True, precision='bf16', tokens=(129,)),
           dict(gate=False, bias=True, bias_in_gemm=False, main_grad=True, precision='mxfp8', tokens=(300,)),
           dict(gate=False, bias=False, bias_in_gemm=False, main_grad=False, precision='mxfp8', tokens=(129,)))


def scenario(rec, fused, configs, hidden=512, heads=4, capacity_tokens=300):
    """Workspace creation plus forward and backward of both projections, per configuration."""
    p = dist.get_world_size()
    d = hidden // heads
    bf = torch.bfloat16
    for index in configs:
        cfg = CONFIGS[index]
        segments = 4 if cfg['gate'] else 3
        rec.log('config', index=index, **{k: v for k, v in cfg.items() if k != 'tokens'})
        ws = fused.FusedGemmA2AWorkspace(hidden, heads, capacity_tokens, gate=cfg['gate'], precision=cfg['precision'])
        if not any(label == 'status' for _, _, label, _ in rec.named):
            rec.register('status', ws.comm.status)
        wq = rec.register(f'wq{index}', torch.zeros(segments * hidden, hidden, dtype=bf)).requires_grad_()
        wo = rec.register(f'wo{index}', torch.zeros(hidden, hidden, dtype=bf)).requires_grad_()
        bq = rec.register(f'bq{index}', torch.zeros(segments * hidden, dtype=bf)).requires_grad_() if cfg['bias'] else None
        bo = rec.register(f'bo{index}', torch.zeros(hidden, dtype=bf)).requires_grad_() if cfg['bias'] else None
        if cfg['main_grad']:
            for name, param in (('wq', wq), ('wo', wo), ('bq', bq), ('bo', bo)):
                if param is not None:
                    param.main_grad = rec.register(f'{name}{index}.main_grad', torch.zeros(param.shape, dtype=torch.float32))
        qkv = fused.FusedQKVProjection(hidden, heads, weight=wq, bias=bq, gate=cfg['gate'], bias_in_gemm=cfg['bias_in_gemm'])
        proj = fused.FusedOutputProjection(hidden, heads, weight=wo, bias=bo)
        for tokens in cfg['tokens']:
            rec.log('tokens', tokens=tokens)
            x = rec.register(f'x{index}.{tokens}', torch.zeros(tokens, hidden, dtype=bf)).requires_grad_()
            grads = [rec.register(f'g{index}.{tokens}.{s}', torch.zeros(p * tokens, heads // p, d, dtype=bf))
                     for s in range(segments)]
            o = rec.register(f'o{index}.{tokens}', torch.zeros(p * tokens, heads // p, d, dtype=bf)).requires_grad_()
            dy = rec.register(f'dy{index}.{tokens}', torch.zeros(tokens, hidden, dtype=bf))
            outs = qkv(x, ws)
            rec.log('qkv outputs', shapes=[list(t.shape) for t in outs])
            got = torch.autograd.grad(outs, [x, wq] + ([bq] if cfg['bias'] else []), grads)
            rec.log('qkv grads', shapes=[list(t.shape) for t in got], dtypes=[str(t.dtype) for t in got],
                    flagged=bool(getattr(wq, 'grad_added_to_main_grad', False)))
            y = proj(o, ws)
            rec.log('out output', shape=list(y.shape))
            got = torch.autograd.grad(y, [o, wo] + ([bo] if cfg['bias'] else []), dy)
            rec.log('out grads', shapes=[list(t.shape) for t in got], dtypes=[str(t.dtype) for t in got],
                    flagged=bool(getattr(wo, 'grad_added_to_main_grad', False)))
        rec.log('launch plans', count=len(ws.comm.compiled))
    return rec.calls


def trace(configs=(0, 1, 2, 3, 4)):
    """The scenario's trace on this rank of an initialised (gloo) process group."""
    import fused_gemm_a2a as fused
    rec = Recorder(dist.get_rank(), dist.get_world_size())
    undo = install(fused, rec)
    try:
        return scenario(rec, fused, configs)
    finally:
        undo()


def dump(calls):
    """One call per line, so that a changed launch plan shows up as a readable diff."""
    import json
    return '[\n' + ',\n'.join(json.dumps(call, sort_keys=True) for call in calls) + '\n]\n'
