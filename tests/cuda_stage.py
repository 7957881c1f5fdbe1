"""Run an unmodified program that was written for CUDA devices on CPU ranks.

TEST INFRASTRUCTURE for the host layer. The reference project's acceptance drivers and benchmark
harness say `device='cuda'`, `torch.cuda.graph(...)`, `init_process_group('nccl')` throughout; this
module lets exactly those files run in a process that has no GPU, against this package on the
simulated library (tests/abi_simulator.py), so that everything they demand of the *host* side -
names, arguments, error messages, caching, "no allocation after set-up", ownership of results,
behaviour under graph replay with changed inputs - is exercised before a GPU ever sees it. Nothing
here says anything about the kernels.

    python tests/cuda_stage.py [--ranks N] [--port P] [--cpu-is-elsewhere] [--stand-in-attention] [--real-library]
                               (<script.py> | -m <module>) [arguments...]

One process per rank: with --ranks N this file starts N copies of itself with RANK / LOCAL_RANK /
WORLD_SIZE / MASTER_ADDR / MASTER_PORT set (a launcher may also set them itself). What the stage
provides:

  * devices: a torch-function mode rewrites every `device=cuda...` argument (and `.to(cuda)`,
    `.cuda()`, `.pin_memory()`) to the CPU. With --cpu-is-elsewhere `.cpu()` moves a tensor to the
    meta device instead, so that a check for "tensor on another device" has another device to meet.
    With --stand-in-attention the flash-attention function one test program imports is torch's math
    attention. torch's block-scaled matmul, which the reference's MXFP8 checks multiply with, is an
    exact product of the values the quantized bytes stand for.
  * --real-library keeps libfga.so itself instead of the simulated library: whatever it answers before it
    touches a device - its argument validation - then works in a process without a GPU.
  * torch.cuda: the handful of calls these programs make (streams, events, synchronize, memory
    statistics, device queries) as host stand-ins; `init_process_group('nccl')` becomes gloo.
  * CUDA graphs: during a capture, what a real capture refuses is refused here too (synchronizing
    the device, a stream or an event; reading a tensor from the host with .item(), .tolist(), .cpu(),
    bool() and the like). `torch.cuda.graph` records what runs inside it - every ATen operation (a
    torch-dispatch mode sees forward and backward alike) and every simulated kernel launch, each with
    the very tensors and raw arguments it ran on - and `CUDAGraph.replay()` runs the recording again
    in order, writing results into the recorded output tensors. Host decisions taken during capture
    are frozen, values flow through the same memory: the semantics of a real graph.
"""
import contextlib
import os
import runpy
import sys
import types

# Ranks share the host's cores: OpenMP workers sleep between parallel regions instead of spinning
# (read when the OpenMP runtime starts, hence before torch is imported).
os.environ.setdefault('OMP_WAIT_POLICY', 'PASSIVE')
os.environ.setdefault('GOMP_SPINCOUNT', '0')

import torch
import torch.distributed as dist
from torch.overrides import TorchFunctionMode
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_flatten

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
STATE = types.SimpleNamespace(recording=None, cpu_is_elsewhere=False, program=None)


def _not_while_capturing(what):
    """A real capture fails on anything that waits for the device or reads device memory from the
    host; the emulation refuses the same, outside the simulated launches (which are host code here)."""
    recording = STATE.recording
    if recording is not None and not recording.inside_launch:
        raise RuntimeError(f'{what}: operation not permitted while a stream is capturing (emulated capture)')


# ---------------------------------------------------------------------------------------- devices
def _is_cuda(value):
    if isinstance(value, torch.device):
        return value.type == 'cuda'
    return isinstance(value, str) and value.startswith('cuda')


HOST_READS = {torch.Tensor.item, torch.Tensor.tolist, torch.Tensor.numpy, torch.Tensor.__bool__, torch.Tensor.__int__,
              torch.Tensor.__float__, torch.Tensor.__index__, torch.Tensor.cpu}


class OnHost(TorchFunctionMode):
    """Every tensor that the program asks to have on a CUDA device lives on the CPU."""

    def __torch_function__(self, func, types_, args=(), kwargs=None):
        kwargs = dict(kwargs or {})
        if _is_cuda(kwargs.get('device')):
            kwargs['device'] = 'cpu'
        if func is torch.Tensor.cuda:
            return args[0]
        if func is torch.Tensor.pin_memory:
            return args[0]
        if func is torch.Tensor.record_stream:
            return None
        if func is torch.Tensor.cpu and STATE.cpu_is_elsewhere and \
                os.path.abspath(sys._getframe(1).f_code.co_filename) == STATE.program:
            return args[0].to('meta')      # only where the program itself says .cpu(), not in libraries
        if getattr(func, '__self__', None) is torch.Tensor.is_cuda:   # the property's getter
            return args[0].device.type == 'cpu'
        if func in HOST_READS and isinstance(args[0], torch.Tensor) and args[0].device.type == 'cpu':
            _not_while_capturing(f'Tensor.{func.__name__}')
        if func is torch.Tensor.to:
            args = tuple('cpu' if _is_cuda(a) else a for a in args)
            kwargs.pop('non_blocking', None)
        return func(*args, **kwargs)


# ------------------------------------------------------------------------------------ CUDA graphs
class Recording(TorchDispatchMode):
    """The nodes of one emulated graph: ATen calls and simulated launches, in issue order."""

    SKIP_COPY = ('aten.empty', 'aten.empty_like', 'aten.empty_strided', 'aten.new_empty')

    def __init__(self):
        super().__init__()
        self.nodes = []
        self.inside_launch = False

    def __torch_dispatch__(self, func, types_, args=(), kwargs=None):
        kwargs = kwargs or {}
        result = func(*args, **kwargs)
        if not self.inside_launch:
            self.nodes.append(('op', func, args, kwargs, result))
        return result

    def launch(self, function, args, kwargs):
        previous, self.inside_launch = self.inside_launch, True
        try:
            result = function(*args, **kwargs)
        finally:
            self.inside_launch = previous
        if not previous:
            self.nodes.append(('launch', function, args, kwargs, result))
        return result

    @staticmethod
    def _write_back(recorded, fresh, skip):
        old, _ = tree_flatten(recorded)
        new, _ = tree_flatten(fresh)
        for before, after in zip(old, new):
            if hasattr(after, 'wait') and not isinstance(after, torch.Tensor):
                after.wait()                                   # an asynchronous collective's handle
            if not isinstance(before, torch.Tensor) or skip:
                continue
            if before.device.type == 'meta' or before.data_ptr() == after.data_ptr():
                continue                                       # a view of, or the very, memory it was given
            before.detach().copy_(after)

    @torch.no_grad()
    def replay(self):
        for kind, function, args, kwargs, recorded in self.nodes:
            fresh = function(*args, **kwargs)
            if kind == 'op':
                self._write_back(recorded, fresh, any(str(function).startswith(name) for name in self.SKIP_COPY))
            else:
                self._write_back(recorded, fresh, False)
                follow_up = getattr(function, 'after_replay', None) or getattr(
                    getattr(function, '__wrapped__', None), 'after_replay', None)
                if follow_up is not None:
                    follow_up(tree_flatten(recorded)[0], tree_flatten(fresh)[0])


class Graph:
    def __init__(self, *_, **__):
        self.recording = None

    def replay(self):
        if self.recording is None:
            raise RuntimeError('replay of a graph that captured nothing')
        self.recording.replay()

    def reset(self):
        self.recording = None

    def pool(self):
        return (0, id(self))

    def enable_debug_mode(self):
        return None


@contextlib.contextmanager
def capture(graph, pool=None, stream=None, capture_error_mode='global'):
    import abi_simulator
    if STATE.recording is not None:
        raise RuntimeError('a capture is already under way')
    graph.recording = STATE.recording = Recording()
    abi_simulator.launch_hook = graph.recording.launch
    try:
        with graph.recording:
            yield
    finally:
        abi_simulator.launch_hook = None
        STATE.recording = None


# ------------------------------------------------------------------------------------- torch.cuda
class Stream:
    cuda_stream = 0
    stream_id = 0
    device_index = 0
    device = torch.device('cpu')

    def __init__(self, *_, **__):
        pass

    def wait_stream(self, other):
        return None

    def wait_event(self, event):
        return None

    def synchronize(self):
        _not_while_capturing('Stream.synchronize')

    def query(self):
        return True

    def record_event(self, event=None):
        return event or Event()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        return False


class Event:
    """Host work is complete when it returns; elapsed time is wall-clock time between the records."""

    def __init__(self, *_, **__):
        self.at = None

    def record(self, stream=None):
        import time
        self.at = time.perf_counter()

    def synchronize(self):
        _not_while_capturing('Event.synchronize')

    def wait(self, stream=None):
        return None

    def query(self):
        _not_while_capturing('Event.query')
        return True

    def elapsed_time(self, end):
        return max((end.at - self.at) * 1e3, 1e-6)


_CURRENT = Stream()


def _current_stream(device=None):
    return _CURRENT


@contextlib.contextmanager
def _stream_context(stream):
    yield


def _properties(device=None):
    return types.SimpleNamespace(name='simulated device', multi_processor_count=148, major=10, minor=0,
                                 total_memory=180 << 30, L2_cache_size=126 << 20)


CUDA_STAND_INS = dict(
    is_available=lambda: True, device_count=lambda: 1, set_device=lambda device: None, current_device=lambda: 0,
    synchronize=lambda device=None: _not_while_capturing('torch.cuda.synchronize'), Stream=Stream, Event=Event, stream=_stream_context,
    current_stream=_current_stream, default_stream=_current_stream, set_stream=lambda stream: None,
    CUDAGraph=Graph, graph=capture, is_current_stream_capturing=lambda: STATE.recording is not None,
    memory_allocated=lambda device=None: 0, max_memory_allocated=lambda device=None: 0,
    memory_reserved=lambda device=None: 0, reset_peak_memory_stats=lambda device=None: None,
    empty_cache=lambda: None, _sleep=lambda cycles: None, get_device_name=lambda device=None: 'simulated device',
    get_device_capability=lambda device=None: (10, 0), get_device_properties=_properties,
    manual_seed=lambda seed: None, manual_seed_all=lambda seed: None, graph_pool_handle=lambda: (0, 0),
    mem_get_info=lambda device=None: (170 << 30, 180 << 30))


class _HostGenerator(torch.Generator):
    """torch.Generator is a class, so the function mode never sees its constructor's device."""

    def __new__(cls, device='cpu'):
        return super().__new__(cls, 'cpu')


class _PackageCuda:
    @staticmethod
    def current_device():
        return None

    def __getattr__(self, name):
        return getattr(torch.cuda, name)


class _PackageTorch:
    cuda = _PackageCuda()

    @staticmethod
    def device(*_, **__):
        return torch.device('cpu')

    def __getattr__(self, name):
        return getattr(torch, name)


def _init_process_group(original):
    def init(backend=None, *args, **kwargs):
        kwargs.pop('device_id', None)
        return original('gloo', *args, **kwargs)
    return init


def install(cpu_is_elsewhere=False, real_library=False):
    """Patch this process; returns nothing - the process is the stage's for the rest of its life."""
    for path in (os.path.join(ROOT, 'fused-gemm-a2a_b200'), HERE, ROOT):
        if path not in sys.path:
            sys.path.insert(0, path)
    import abi_simulator
    import fused_gemm_a2a as fused
    STATE.cpu_is_elsewhere = cpu_is_elsewhere
    for name, stand_in in CUDA_STAND_INS.items():
        setattr(torch.cuda, name, stand_in)
    dist.init_process_group = _init_process_group(dist.init_process_group)
    torch.Generator = _HostGenerator
    if real_library:
        # libfga.so itself: only what it answers before it touches a device can work here, i.e. its
        # argument validation (tests that expect a rejection and its message).
        fused.torch = _PackageTorch()
        OnHost().__enter__()
        return None
    _, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    # The package's own view of torch: the CPU is "the device" (its index is None), and every torch.cuda
    # call goes to the stand-ins above through the real module, so that a program which patches
    # torch.cuda.synchronize to catch a forbidden call also catches the package's.
    fused.torch = _PackageTorch()
    _sabotage(fused, os.environ.get('FGA_STAGE_SABOTAGE', ''))
    OnHost().__enter__()
    return undo


def _sabotage(fused, what):
    """Negative controls: break the host layer in a known way, so that a test can show that the staged
    programs notice (tests/test_reference_programs_staged.py).
      shared-output   results that need no resizing are handed out as views of the shared head-side
                      buffers instead of owned copies (the next forward overwrites them)"""
    if what == 'shared-output':
        owned = fused.resize_rank_rows

        def resize_rank_rows(tensors, peers, rows, *, copy=False, bias=None, **kwargs):
            tensors = tuple(tensors)
            if bias is None and tensors[0].shape[0] == peers * rows:
                return tensors
            return owned(tensors, peers, rows, copy=copy, bias=bias, **kwargs)
        fused.resize_rank_rows = resize_rank_rows
    elif what:
        raise SystemExit(f'unknown sabotage {what!r}')


def _varlen_attention(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None, max_seqlen_k=None,
                      causal=False, softmax_scale=None, **_):
    """Stand-in for a variable-length flash-attention call ([tokens, heads, dim] operands, sequences
    delimited by cu_seqlens): torch's math attention per sequence, FP32 inside, the operands' type out."""
    recording = STATE.recording      # the real function takes the sequence bounds on the device; this one reads them
    if recording is not None:
        recording.inside_launch = True
    try:
        bounds_q, bounds_k = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    finally:
        if recording is not None:
            recording.inside_launch = False
    pieces = []
    for (q0, q1), (k0, k1) in zip(zip(bounds_q, bounds_q[1:]), zip(bounds_k, bounds_k[1:])):
        out = torch.nn.functional.scaled_dot_product_attention(
            q[q0:q1].transpose(0, 1).float(), k[k0:k1].transpose(0, 1).float(), v[k0:k1].transpose(0, 1).float(),
            is_causal=causal, scale=softmax_scale)
        pieces.append(out.transpose(0, 1).to(q.dtype))
    return torch.cat(pieces)


def _stand_in_attention():
    """Make `from flash_attn.cute.interface import flash_attn_varlen_func` resolve to the function above
    (the attention kernel is a dependency of a test program, not of the package)."""
    for name in ('flash_attn', 'flash_attn.cute', 'flash_attn.cute.interface'):
        module = types.ModuleType(name)
        module.__path__ = []
        sys.modules[name] = module
    sys.modules['flash_attn.cute.interface'].flash_attn_varlen_func = _varlen_attention
    sys.modules['flash_attn'].cute = sys.modules['flash_attn.cute']
    sys.modules['flash_attn.cute'].interface = sys.modules['flash_attn.cute.interface']


def _stand_in_scaled_mm():
    """The reference's MXFP8 checks multiply with torch's block-scaled matmul, which has no CPU
    implementation: here it multiplies exactly the values that the E4M3 bytes and E8M0 scale bytes stand
    for (oracle/mxfp8_oracle.py). The quantizer those checks call is the package's own wrapper, which on
    the stage reaches the simulated library's byte-level quantizer."""
    from oracle import mxfp8_oracle

    def values(payload, scales):
        rows, k = payload.shape
        raw = payload.contiguous().view(torch.uint8).numpy()
        return torch.from_numpy(mxfp8_oracle.dequantize(raw, scales.contiguous().view(torch.uint8).numpy(), rows, k)
                                .reshape(rows, k))

    def scaled_mm(a, b, scale_a, recipe_a, scale_b, recipe_b, swizzle_a=None, swizzle_b=None, bias=None,
                  output_dtype=None, **_):
        product = values(a, scale_a) @ values(b.t(), scale_b).t()
        return product.to(output_dtype or torch.bfloat16)

    torch.nn.functional.scaled_mm = scaled_mm


def _spawn_ranks(ranks, port, flags, arguments, timeout):
    """One child per rank, each running this file again with its rank in the environment."""
    import subprocess
    children = []
    for rank in range(ranks):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(ranks), MASTER_ADDR='127.0.0.1',
                   MASTER_PORT=str(port))
        children.append(subprocess.Popen([sys.executable, os.path.abspath(__file__), *flags, *arguments], env=env,
                                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    worst = 0
    for rank, child in enumerate(children):
        try:
            output, _ = child.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            child.kill()
            output, _ = child.communicate()
            output += f'\n[rank {rank}: no end after {timeout} s]'
        sys.stdout.write(output if rank == 0 or child.returncode else '')
        worst = worst or child.returncode
    return worst


def main():
    arguments = sys.argv[1:]
    options = dict(ranks=1, port=29690, timeout=1500)
    flags = []
    while arguments and arguments[0].startswith('--'):   # the stage's own options come first
        flag = arguments.pop(0)
        if flag in ('--cpu-is-elsewhere', '--stand-in-attention', '--real-library'):
            flags.append(flag)
        elif flag[2:] in options:
            options[flag[2:]] = int(arguments.pop(0))
        else:
            raise SystemExit(f'unknown option {flag}\n{__doc__}')
    if not arguments:
        raise SystemExit(__doc__)
    if 'RANK' not in os.environ and options['ranks'] > 1:
        raise SystemExit(_spawn_ranks(options['ranks'], options['port'], flags, arguments, options['timeout']))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', str(options['port']))
    for name, value in (('RANK', '0'), ('LOCAL_RANK', '0'), ('WORLD_SIZE', '1')):
        os.environ.setdefault(name, value)
    threads = int(os.environ.get('FGA_STAGE_THREADS', 0)) or (os.cpu_count() or 2) // int(os.environ['WORLD_SIZE'])
    torch.set_num_threads(max(1, threads))
    install('--cpu-is-elsewhere' in flags, '--real-library' in flags)
    if '--stand-in-attention' in flags:
        _stand_in_attention()
    _stand_in_scaled_mm()
    if arguments[0] == '-m':                       # a module, as in `python -m pytest ...`
        sys.argv = arguments[1:]
        runpy.run_module(arguments[1], run_name='__main__', alter_sys=True)
        return
    sys.argv = arguments
    STATE.program = os.path.abspath(arguments[0])
    runpy.run_path(arguments[0], run_name='__main__')


if __name__ == '__main__':
    main()
