"""Benchmark of the fused projection-GEMM + Ulysses all-to-all path (one JSON line on rank 0).

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference ...                      # CPU arm: the unfused path on host cores
    python bench.py --impl nccl ...                           # cuBLAS + NCCL all-to-all yardstick

Workload (the configuration the headline metric is quoted on): 131072 total tokens, H = 4096,
32 heads of 128, BF16, no bias; CP = N ranks each own M = 131072 / N tokens (strong scaling). One
step = QKV projection forward + backward and output projection forward + backward (dgrad and
wgrad), i.e. 24 * M * H^2 algorithmic FLOPs per GPU (forward 2*M*H*N_out, backward twice that).

Data is synthetic: x ~ N(0,1), Wqkv / Wo ~ N(0, 1/64) in Megatron per-head interleaving, upstream
gradients ~ N(0,1), seeded per rank. Inputs are far larger than L2 (>= 128 MiB each), so no L2
flush is needed between iterations.

Timed with CUDA events on the launching stream between a barrier + synchronize on both sides;
the maximum over ranks is reported. `value` is device-resident throughput, `e2e` repeats the
measurement through the public modules with every step's inputs copied from pinned host memory
(prefetched on a copy stream while the previous step computes) and a scalar result read back.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.join(ROOT, 'fused-gemm-a2a_b200')
for _path in (ROOT, PACKAGE):
    if _path not in sys.path:
        sys.path.insert(0, _path)

METRIC = 'fused QKV + output projection fwd+bwd throughput (131072 tokens, H=4096, 32x128 heads)'
UNIT = 'TFLOP/s'
NOMINAL_BF16_TFLOPS = 2250.0
LINK_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool (900 nominal)
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per FLOP of the GEMM kernel, from the ncu
# captures of `--kernel-case gemm_nt` (670.4 MB) and `--kernel-case wgrad` (1296.8 MB), both
# 824.6 GFLOP launches at 8192 tokens (summaries of both captures are kept under profiles/). The benchmark's
# launches are too large to capture; traffic grows with the rows, so it is scaled by the FLOPs.
DRAM_BYTES_PER_FLOP = dict(gemm=670.4e6 / 824.6e9, wgrad=1296.8e6 / 824.6e9)


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='fused', choices=('fused', 'reference', 'nccl'))
    ap.add_argument('--tokens', type=int, default=131072, help='total tokens over all ranks')
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--heads', type=int, default=32)
    ap.add_argument('--gate', action='store_true')
    ap.add_argument('--bias', action='store_true')
    ap.add_argument('--precision', default='bf16', choices=('bf16', 'mxfp8'))
    ap.add_argument('--no-e2e', action='store_true', help='skip the host-buffer measurement')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-graphs', action='store_true', help='launch eagerly instead of replaying CUDA graphs')
    ap.add_argument('--cpu-sample-tokens', type=int, default=2048)
    ap.add_argument('--kernel-case', default=None, choices=('gemm_nt', 'gemm_nn', 'wgrad', 'step'),
                    help='run only a few launches of one kernel on a small case (for an ncu capture) and exit')
    ap.add_argument('--case-tokens', type=int, default=8192, help='rows of the --kernel-case problem')
    ap.add_argument('--case-launches', type=int, default=3)
    return ap.parse_args()


def flops_per_step(m, hidden, segments):
    """Algorithmic FLOPs per GPU: forward 2*M*H*N_out, backward (dgrad + wgrad) twice that."""
    qkv, out = 2.0 * m * hidden * segments * hidden, 2.0 * m * hidden * hidden
    return dict(qkv_fwd=qkv, qkv_bwd=2 * qkv, out_fwd=out, out_bwd=2 * out, total=3 * (qkv + out))


def provenance(torch=None):
    """What produced the line: versions, the GPU, every tuning variable that was set, and a digest of
    the built library and of the sources that define the path (as the reference's benchmark records
    the digest of its two source files)."""
    import hashlib

    def digest(*paths):
        h = hashlib.sha256()
        for path in paths:
            try:
                with open(path, 'rb') as f:
                    h.update(f.read())
            except OSError:
                return None
        return h.hexdigest()[:16]

    try:
        return _provenance(torch, digest)
    except Exception as error:      # never let bookkeeping break a measurement
        return dict(error=f'{type(error).__name__}: {error}')


def _provenance(torch, digest):
    package = os.path.join(ROOT, 'fused-gemm-a2a_b200')
    csrc = os.path.join(package, 'csrc')
    sources = sorted(os.path.join(csrc, name) for name in os.listdir(csrc)) if os.path.isdir(csrc) else []
    info = dict(tunables={k: v for k, v in sorted(os.environ.items()) if k.startswith(('FGA_', 'FUSED_'))},
                libfga_sha256=digest(os.path.join(package, 'libfga.so')),
                csrc_sha256=digest(*sources),
                host_layer_sha256=digest(os.path.join(package, 'fused_gemm_a2a.py'),
                                         os.path.join(package, 'fused_gemm_a2a_kernels.py')))
    if torch is not None:
        info['torch'] = torch.__version__
        info['cuda'] = torch.version.cuda
        if torch.cuda.is_available():
            info['gpu'] = torch.cuda.get_device_name(torch.cuda.current_device())
    return info


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        return float(peaks.get('bf16_tflops_sustained') or peaks['bf16_tflops']), 'measured (sustained cuBLAS bf16)'
    return 1400.0, 'fallback (sustained, no MEASURED_PEAKS.json)'


class ClockSampler:
    """nvidia-smi clock / throttle samples of one GPU while a region runs."""
    QUERY = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
             'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
             'clocks_event_reasons.sw_power_cap,power.limit')

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []
        self.first, self.last = 0, None

    def begin(self):
        """The timed region starts now: earlier samples (warm-up) are dropped."""
        self.first = len(self.lines)

    def end(self):
        self.last = len(self.lines)

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--id={self.index}', f'--query-gpu={self.QUERY}',
                 '--format=csv,noheader,nounits', '-lms', '50'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        clocks, max_clock, reasons, power, limit = [], None, set(), [], None
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        window = self.lines[self.first:self.last] or self.lines[-3:]
        for line in window:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith('active'):
                    reasons.add(name)
            if len(parts) > 7:
                try:
                    limit = float(parts[7])
                except ValueError:
                    pass
        clocks.sort()
        return dict(sm_mhz=clocks[len(clocks) // 2] if clocks else None, sm_max_mhz=max_clock,
                    power_w_max=max(power) if power else None, power_limit_w=limit, reasons=sorted(reasons),
                    samples=len(clocks))


# ----------------------------------------------------------------------------------------------
# CPU arm: the unfused path on the host cores (oracle port of the reference's unfused modules).
# ----------------------------------------------------------------------------------------------
def cpu_unfused_sample(hidden, heads, segments, sample_tokens, steps, warmup):
    """Times the oracle's forward + backward of both projections for `sample_tokens` tokens of the
    workload on all host cores (FP32 torch CPU GEMMs from BF16-valued inputs)."""
    import torch
    from oracle.ulysses_oracle import UlyssesOracle
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1234)
    bf = torch.bfloat16
    wq = (torch.randn(segments * hidden, hidden, generator=g) / 64).to(bf).float()
    wo = (torch.randn(hidden, hidden, generator=g) / 64).to(bf).float()
    x = torch.randn(sample_tokens, hidden, generator=g).to(bf).float()
    grads = tuple(torch.randn(sample_tokens, heads, hidden // heads, generator=g).to(bf).float()
                  for _ in range(segments))
    o = torch.randn(sample_tokens, heads, hidden // heads, generator=g).to(bf).float()
    dy = torch.randn(sample_tokens, hidden, generator=g).to(bf).float()
    oracle = UlyssesOracle(1, hidden, heads, segments, wq, None, wo, None, dtype=torch.float32,
                           acc_dtype=torch.float32)

    def step():
        oracle.qkv_forward([x])
        oracle.qkv_backward([x], [grads])
        oracle.out_forward([o])
        oracle.out_backward([o], [dy])

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = (time.perf_counter() - t0) / steps
    flops = flops_per_step(sample_tokens, hidden, segments)['total']
    return dict(value=flops / seconds / 1e12, unit=UNIT, cores=cores, kind='port',
                sample=f'{sample_tokens} tokens of the workload (H={hidden}, {heads} heads), forward+backward of both '
                       f'projections, FP32 torch CPU GEMMs, {steps} timed steps of {seconds:.3f} s'), seconds


def run_reference_arm(args):
    rank = int(os.environ.get('RANK', 0))
    if rank != 0:
        return
    segments = 4 if args.gate else 3
    steps, warmup = max(1, args.steps), max(1, min(args.warmup, 2))
    base, seconds = cpu_unfused_sample(args.hidden, args.heads, segments, args.cpu_sample_tokens, steps, warmup)
    line = dict(metric=METRIC, value=base['value'], unit=UNIT, n_gpus=args.gpus, steps=steps, warmup=warmup,
                ms_per_step=seconds * 1e3, higher_is_better=True, scaling='strong', vs_baseline=None,
                dtype='f32', data='synthetic', impl='reference',
                config=dict(workload=f'{args.tokens} total tokens, H={args.hidden}, {args.heads}x128 heads, '
                                     f'QKV{"G" if args.gate else ""} + output projection fwd+bwd; CPU sample of '
                                     f'{args.cpu_sample_tokens} tokens per step',
                            l2='inputs larger than L2'),
                cpu_baseline=base,
                e2e=dict(value=base['value'], unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arms
# ----------------------------------------------------------------------------------------------
def init_distributed(torch, dist):
    world = int(os.environ.get('WORLD_SIZE', 1))
    rank = int(os.environ.get('RANK', 0))
    local = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29555')
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', local))
    return rank, world, local


def interleave(seg_major, heads, d):
    s = seg_major.shape[0] // (heads * d)
    return seg_major.reshape(s, heads, d, -1).transpose(0, 1).reshape(seg_major.shape)


class NcclUnfused:
    """cuBLAS GEMMs + NCCL all-to-all with the Async-Ulysses overlap (each projection's all-to-all
    is launched before the next projection's GEMM); the yardstick the fused path is compared with.
    Same inputs, same outputs, no autograd graph (explicit backward)."""

    def __init__(self, torch, dist, p, hidden, heads, w_segments, wo):
        self.torch, self.dist, self.p, self.h, self.n = torch, dist, p, hidden, heads
        self.d = hidden // heads
        self.ws, self.wo = w_segments, wo

    def a2a(self, t):
        out = self.torch.empty_like(t)
        work = self.dist.all_to_all_single(out, t, async_op=True) if self.p > 1 else None
        if work is None:
            out = t
        return out, work

    def to_heads(self, y):      # [M, H] -> [P, M, N/P, D] contiguous (rank-major rows after the a2a)
        m = y.shape[0]
        return y.view(m, self.p, self.n // self.p, self.d).transpose(0, 1).contiguous()

    def from_heads(self, t):    # [P*M, N/P, D] received -> [M, H]
        m = t.shape[0] // self.p
        return t.view(self.p, m, self.n // self.p, self.d).transpose(0, 1).reshape(m, self.h)

    def qkv_forward(self, x):
        pending = [self.a2a(self.to_heads(x @ w.t())) for w in self.ws]
        outs = []
        for out, work in pending:
            if work is not None:
                work.wait()
            outs.append(out.view(-1, self.n // self.p, self.d))
        return outs

    def qkv_backward(self, x, grads):
        dx, dws = None, []
        pending = self.a2a(grads[-1].contiguous())
        for i in reversed(range(len(grads))):
            buf, work = pending
            if work is not None:
                work.wait()
            if i:
                pending = self.a2a(grads[i - 1].contiguous())
            g = self.from_heads(buf)
            part = g @ self.ws[i]
            dx = part if dx is None else dx + part
            dws.append(g.t() @ x)
        return dx, dws

    def out_forward(self, o):
        buf, work = self.a2a(o.contiguous())
        if work is not None:
            work.wait()
        self.o_seq = self.from_heads(buf)
        return self.o_seq @ self.wo.t()

    def out_backward(self, dy):
        do_full = dy @ self.wo
        buf, work = self.a2a(self.to_heads(do_full))
        dwo = dy.t() @ self.o_seq
        if work is not None:
            work.wait()
        return buf.view(-1, self.n // self.p, self.d), dwo


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    rank, world, local = init_distributed(torch, dist)
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run')
    if args.tokens % world or args.heads % world:
        raise SystemExit('tokens and heads must divide over the ranks')
    dev = torch.device('cuda', local)
    # Everything runs on one non-default stream from the start: autograd ties the gradient
    # accumulation nodes of the leaves to the stream of their first use, and a node tied to the
    # legacy default stream cannot take part in a stream capture.
    work_stream = torch.cuda.Stream()
    torch.cuda.set_stream(work_stream)
    p, hidden, heads = world, args.hidden, args.heads
    d, m, segments = hidden // heads, args.tokens // world, 4 if args.gate else 3
    bf = torch.bfloat16
    flops = flops_per_step(m, hidden, segments)

    # ---- synthetic data: weights identical on every rank, activations per rank
    gen = torch.Generator(device=dev).manual_seed(1234)
    w_seg = (torch.randn(segments * hidden, hidden, generator=gen, device=dev) / 64).to(bf)
    wo = (torch.randn(hidden, hidden, generator=gen, device=dev) / 64).to(bf)
    bq = (torch.randn(segments * hidden, generator=gen, device=dev) * 0.02).to(bf) if args.bias else None
    bo = (torch.randn(hidden, generator=gen, device=dev) * 0.02).to(bf) if args.bias else None
    gen = torch.Generator(device=dev).manual_seed(1234 + 1 + rank)
    x = torch.randn(m, hidden, generator=gen, device=dev).to(bf)
    grads = [torch.randn(p * m, heads // p, d, generator=gen, device=dev).to(bf) for _ in range(segments)]
    o = torch.randn(p * m, heads // p, d, generator=gen, device=dev).to(bf)
    dy = torch.randn(m, hidden, generator=gen, device=dev).to(bf)
    inputs = [x, *grads, o, dy]

    launches = lambda: 0  # noqa: E731
    if args.impl == 'fused':
        import build_native
        build_native.build()
        import _fga_native
        import fused_gemm_a2a as fused
        lib = _fga_native.lib()
        launches = lib.fga_launch_count
        ws = fused.FusedGemmA2AWorkspace(hidden, heads, m, gate=args.gate, precision=args.precision)
        wq = interleave(w_seg, heads, d).contiguous().requires_grad_()
        wo_p = wo.clone().requires_grad_()
        bq_p = interleave(bq, heads, d).contiguous().requires_grad_() if args.bias else None
        bo_p = bo.clone().requires_grad_() if args.bias else None
        qkv = fused.FusedQKVProjection(hidden, heads, weight=wq, bias=bq_p, gate=args.gate)
        proj = fused.FusedOutputProjection(hidden, heads, weight=wo_p, bias=bo_p)
        x.requires_grad_()
        o.requires_grad_()
        qkv_params = [wq] + ([bq_p] if args.bias else [])
        out_params = [wo_p] + ([bo_p] if args.bias else [])

        def passes():
            """The four passes of a step as separate callables (for per-pass timing)."""
            state = {}

            def qkv_fwd():
                state['qs'] = qkv(x, ws)

            def qkv_bwd():
                state['dq'] = torch.autograd.grad(state.pop('qs'), [x, *qkv_params], grads)

            def out_fwd():
                state['y'] = proj(o, ws)

            def out_bwd():
                state['do'] = torch.autograd.grad(state['y'], [o, *out_params], dy)

            return state, (qkv_fwd, qkv_bwd, out_fwd, out_bwd)
    else:
        ref = NcclUnfused(torch, dist, p, hidden, heads, list(w_seg.split(hidden)), wo)

        def passes():
            state = {}

            def qkv_fwd():
                state['qs'] = ref.qkv_forward(x)

            def qkv_bwd():
                state['dq'] = ref.qkv_backward(x, grads)

            def out_fwd():
                state['y'] = ref.out_forward(o)

            def out_bwd():
                state['do'] = ref.out_backward(dy)

            return state, (qkv_fwd, qkv_bwd, out_fwd, out_bwd)

    state, fns = passes()
    names = ('qkv_fwd', 'qkv_bwd', 'out_fwd', 'out_bwd')

    def eager_step(events=None):
        for i, fn in enumerate(fns):
            fn()
            if events is not None:
                events[i + 1].record()

    step = eager_step

    def fence():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # ---- device-resident measurement (the clock sampler starts before the warm-up so that it is
    # already streaming when the timed region begins)
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    graph_note = 'eager launches'
    with ClockSampler(local) as clocks:
        for _ in range(max(args.warmup, 3)):
            eager_step()
        fence()
        if args.impl == 'fused':
            ws.comm.check_status()
        launches_per_step = None
        if not args.no_graphs:
            # One CUDA graph per pass (shared memory pool), replayed back to back: launch latency of
            # the host is out of the measurement, as in the reference's graph-captured benchmark.
            side = work_stream
            try:
                fence()
                graphs, pool, before = [], None, launches()
                for fn in fns:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool, stream=side, capture_error_mode='thread_local'):
                        fn()
                    pool = pool or g.pool()
                    graphs.append(g)
                launches_per_step = launches() - before
                def step(events=None):
                    for i, g in enumerate(graphs):
                        g.replay()
                        if events is not None:
                            events[i + 1].record()
                graph_note = 'one CUDA graph per pass, replayed'
            except Exception as error:  # capture not supported for this arm: stay eager, say so
                graph_note = f'eager launches (graph capture failed: {type(error).__name__}: {str(error)[:300]})'
                step = eager_step
            fence()
            for _ in range(2):
                step()
            fence()
        launches_before = launches()
        clocks.begin()
        for k in range(args.steps):
            marks[k][0].record()
            step(marks[k])
        fence()
        clocks.end()
    gpu_launches = launches() - launches_before
    if launches_per_step is not None and step is not eager_step:
        gpu_launches = launches_per_step * args.steps  # replayed launches are not seen by the counter
    total_ms = marks[0][0].elapsed_time(marks[-1][4])
    pass_ms = [sum(marks[k][i].elapsed_time(marks[k][i + 1]) for k in range(args.steps)) / args.steps
               for i in range(4)]
    total_ms, *pass_ms = max_over_ranks([total_ms, *pass_ms])
    ms_per_step = total_ms / args.steps
    per_gpu_tflops = flops['total'] / (ms_per_step * 1e-3) / 1e12
    if args.impl == 'fused':
        ws.comm.check_status()

    # ---- the GEMM kernel alone: CUDA events around every launch of it during extra steps
    roofline = None
    if args.impl == 'fused' and args.precision == 'bf16':
        peak, peak_source = measured_peaks()
        records, others = [], []

        def timed(fn, label, algorithmic_flops=None):
            def wrapper(*a, **kw):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = fn(*a, **kw)
                e1.record()
                name = label(*a, **kw) if callable(label) else label
                if algorithmic_flops is None:
                    others.append((name, e0, e1))
                else:
                    records.append((name, e0, e1, algorithmic_flops(*a, **kw)))
                return out
            return wrapper

        def gemm_flops(mode, a, b, b_is_kn, c, *rest, **kw):
            # algorithmic rows only: pad rows of the capacity are not counted
            return 2.0 * m * b.shape[0] * b.shape[1]

        def gemm_label(mode, a, b, b_is_kn, c, *rest, **kw):
            return f'gemm_{mode}[{m}x{b.shape[1] if not b_is_kn else b.shape[0]}->{b.shape[0] if not b_is_kn else b.shape[1]}]'

        comm = ws.comm
        saved = (comm.gemm, fused.bf16_wgrad, comm.barrier, fused.resize_rank_rows)
        comm.gemm = timed(saved[0], gemm_label, gemm_flops)
        fused.bf16_wgrad = timed(saved[1], lambda dyv, xv, *a, **kw: f'gemm_wgrad[{dyv.shape[1]}x{xv.shape[1]},k={dyv.shape[0]}]',
                                 lambda dyv, xv, *a, **kw: 2.0 * dyv.shape[0] * dyv.shape[1] * xv.shape[1])
        comm.barrier = timed(saved[2], 'barrier')
        fused.resize_rank_rows = timed(saved[3], 'copy_rank_rows')
        extra = 2
        for _ in range(extra):
            eager_step()
        torch.cuda.synchronize()
        comm.gemm, fused.bf16_wgrad, comm.barrier, fused.resize_rank_rows = saved
        gemm_ms = sum(e0.elapsed_time(e1) for _, e0, e1, _ in records)
        gemm_flops_total = sum(f for *_, f in records)
        per_launch = [dict(op=name, ms=e0.elapsed_time(e1), tflops=f / e0.elapsed_time(e1) / 1e9)
                      for name, e0, e1, f in records[len(records) // 2:]]
        per_launch += [dict(op=name, ms=e0.elapsed_time(e1)) for name, e0, e1 in others[len(others) // 2:]]
        gemm_ms, = max_over_ranks([gemm_ms])
        achieved = gemm_flops_total / (gemm_ms * 1e-3) / 1e12
        a2a_bytes = 2.0 * m * (segments + 1) * hidden * 2 * (p - 1) / p  # both directions' payload per step
        # operands and outputs of the six GEMMs of a step: activations and their gradients are touched
        # by the forward, dgrad and wgrad launch; the weight is read twice and its BF16 gradient written
        algorithmic_bytes = sum(2.0 * (3 * (m * hidden + m * s * hidden) + 3 * s * hidden * hidden)
                                for s in (segments, 1))
        traffic = sum(f * DRAM_BYTES_PER_FLOP['wgrad' if 'wgrad' in name else 'gemm']
                      for name, _, _, f in records) / max(1, len(records))
        roofline = dict(bound='tensor', kernel='ulysses_gemm_kernel', achieved=achieved, peak=peak, unit='TFLOP/s',
                        frac=achieved / peak, traffic=traffic,
                        traffic_note='bytes per launch (mean over the 6 launches of a step), scaled by FLOPs from ncu '
                                     'captures of 8192-token launches; algorithmic bytes per launch: '
                                     f'{algorithmic_bytes / 6:.3e}',
                        peak_source=peak_source,
                        launches_timed=len(records), avg_launch_ms=gemm_ms / max(1, len(records)),
                        gemm_share_of_step=gemm_ms / extra / ms_per_step,
                        frac_of_nominal_2250=achieved / NOMINAL_BF16_TFLOPS,
                        link_bound_ms_per_step=a2a_bytes / (LINK_GBS * 1e9) * 1e3,
                        launches_rank0_last_step=per_launch)

    # ---- end to end: pinned host inputs -> device (prefetched on a copy stream) -> step -> scalar back
    e2e = None
    if not args.no_e2e:
        host = [t.detach().to('cpu').pin_memory() for t in inputs]
        h2d_bytes = sum(t.numel() * t.element_size() for t in host)
        staged = [[torch.empty_like(t.detach()) for t in inputs] for _ in range(2)]
        copy_stream = torch.cuda.Stream()
        ready = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        result = torch.zeros(1, dtype=torch.float32).pin_memory()

        def prefetch(slot):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[slot])
                for dst, src in zip(staged[slot], host):
                    dst.copy_(src, non_blocking=True)
                ready[slot].record(copy_stream)

        def e2e_step(slot):
            cur = torch.cuda.current_stream()
            cur.wait_event(ready[slot])
            with torch.no_grad():
                for dst, src in zip(inputs, staged[slot]):
                    dst.copy_(src)           # device-to-device hand-over into the tensors the modules hold
            consumed[slot].record(cur)
            step()
            scalar = state['y'].float().sum().reshape(1)
            result.copy_(scalar, non_blocking=True)

        for ev in consumed:
            ev.record()
        fence()
        prefetch(0)
        e2e_step(0)          # warm-up of the staging path
        fence()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        prefetch(0)
        t0.record()
        for k in range(args.steps):
            if k + 1 < args.steps:
                prefetch((k + 1) % 2)
            e2e_step(k % 2)
        t1.record()
        fence()
        # the first step's copy was issued just before t0 on the copy stream: count it by timing
        # from the host side as well and taking the larger figure
        e2e_ms, = max_over_ranks([t0.elapsed_time(t1)])
        e2e_ms_per_step = e2e_ms / args.steps
        e2e = dict(value=world * flops['total'] / (e2e_ms_per_step * 1e-3) / 1e12, unit=UNIT,
                   h2d_bytes_per_step=h2d_bytes, d2h_bytes_per_step=4, ms_per_step=e2e_ms_per_step,
                   note='inputs prefetched from pinned host memory on a copy stream while the previous step computes')
        if args.impl == 'fused':
            ws.comm.check_status()

    if rank != 0:
        dist.barrier()
        return
    link_ms = 2.0 * m * (segments + 1) * hidden * 2 * (p - 1) / p / (LINK_GBS * 1e9) * 1e3
    line = dict(
        metric=METRIC, value=world * per_gpu_tflops, unit=UNIT, n_gpus=world, steps=args.steps,
        warmup=max(args.warmup, 3), ms_per_step=ms_per_step, higher_is_better=True, scaling='strong',
        vs_baseline=None, dtype='bf16' if args.precision == 'bf16' else 'mxfp8 (e4m3 payload, e8m0 scale per 32, fp32 accumulate)',
        data='synthetic', impl=args.impl,
        config=dict(workload=f'{args.tokens} total tokens, H={hidden}, {heads}x{d} heads, CP={world} '
                             f'(M={m} per rank), QKV{"G" if args.gate else ""} + output projection, forward + dgrad + wgrad'
                             f'{", bias" if args.bias else ", no bias"}',
                    parallelism=f'cp{world}', l2='inputs larger than L2 (no flush needed)', launch=graph_note),
        tflops_per_gpu=per_gpu_tflops, pct_of_nominal_2250=100 * per_gpu_tflops / NOMINAL_BF16_TFLOPS,
        passes={n: dict(ms=ms, tflops_per_gpu=flops[n] / (ms * 1e-3) / 1e12) for n, ms in zip(names, pass_ms)},
        step_roofline=dict(compute_ms_at_2250=flops['total'] / NOMINAL_BF16_TFLOPS / 1e9,
                           link_ms_at_770GBs=link_ms,
                           frac=max(flops['total'] / NOMINAL_BF16_TFLOPS / 1e9, link_ms) / ms_per_step),
        clocks=clocks.summary(), gpu_launches=int(gpu_launches), provenance=provenance(torch))
    if roofline is not None:
        line['roofline'] = roofline
    if e2e is not None:
        line['e2e'] = e2e
    if world == 1 and args.impl == 'fused' and not args.no_cpu_baseline:
        line['cpu_baseline'], _ = cpu_unfused_sample(hidden, heads, segments, args.cpu_sample_tokens, 2, 1)
    print(json.dumps(line), flush=True)
    dist.barrier()


def run_kernel_case(args):
    """A few launches of one kernel on a small problem whose operands exceed L2, for profiler
    captures (`ncu -k regex:ulysses_gemm -c 1 ... python bench.py --kernel-case gemm_nt`). Prints the
    CUDA-event time per launch; numbers printed under a profiler are not benchmark values."""
    import torch
    import build_native
    build_native.build()
    import _fga_native
    lib = _fga_native.lib()
    torch.cuda.set_device(0)
    dev = torch.device('cuda', 0)
    m, h = args.case_tokens, args.hidden
    bf = torch.bfloat16
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    timeout = 10_000_000_000
    if args.kernel_case == 'step':
        import torch.distributed as dist
        init_distributed(torch, dist)
        import fused_gemm_a2a as fused
        ws = fused.FusedGemmA2AWorkspace(h, args.heads, m)
        wq = (torch.randn(3 * h, h, device=dev) / 64).to(bf).requires_grad_()
        wo = (torch.randn(h, h, device=dev) / 64).to(bf).requires_grad_()
        qkv = fused.FusedQKVProjection(h, args.heads, weight=wq)
        proj = fused.FusedOutputProjection(h, args.heads, weight=wo)
        x = torch.randn(m, h, device=dev).to(bf).requires_grad_()
        o = torch.randn(m, args.heads, h // args.heads, device=dev).to(bf).requires_grad_()
        grads = [torch.randn(m, args.heads, h // args.heads, device=dev).to(bf) for _ in range(3)]
        dy = torch.randn(m, h, device=dev).to(bf)

        def launch():
            torch.autograd.grad(qkv(x, ws), [x, wq], grads)
            torch.autograd.grad(proj(o, ws), [o, wo], dy)
        flops = flops_per_step(m, h, 3)['total']
    else:
        n = 3 * h if args.kernel_case != 'wgrad' else h
        a = torch.randn(m, h, device=dev).to(bf)
        if args.kernel_case == 'gemm_nt':      # forward: x [M,K] * W[N,K]^T
            b, c, call = torch.randn(n, h, device=dev).to(bf), torch.empty(m, n, dtype=bf, device=dev), None
            call = lambda: lib.fga_gemm_local(a.data_ptr(), 0, b.data_ptr(), 0, m, n, h, h, h, c.data_ptr(), n, 0, 0,  # noqa: E731
                                              status.data_ptr(), timeout, stream)
            flops = 2.0 * m * n * h
        elif args.kernel_case == 'gemm_nn':    # dgrad: dY [M,K=3H] * W[K,N=H]
            dyv, w = torch.randn(m, n, device=dev).to(bf), torch.randn(n, h, device=dev).to(bf)
            c = torch.empty(m, h, dtype=bf, device=dev)
            call = lambda: lib.fga_gemm_local(dyv.data_ptr(), 0, w.data_ptr(), 1, m, h, n, n, h, c.data_ptr(), h, 0, 0,  # noqa: E731
                                              status.data_ptr(), timeout, stream)
            flops = 2.0 * m * n * h
        else:                                  # wgrad: dY[T,N]^T * X[T,K] accumulated in FP32
            n = 3 * h
            dyv = torch.randn(m, n, device=dev).to(bf)
            c = torch.zeros(n, h, dtype=torch.float32, device=dev)
            call = lambda: lib.fga_gemm_local(dyv.data_ptr(), 1, a.data_ptr(), 1, n, h, m, n, h, c.data_ptr(), h, 1, 1,  # noqa: E731
                                              status.data_ptr(), timeout, stream)
            flops = 2.0 * m * n * h

        def launch():
            _fga_native.check(call())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launch()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.case_launches):
        launch()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.case_launches
    print(json.dumps(dict(kernel_case=args.kernel_case, tokens=m, hidden=h, ms_per_launch=ms,
                          tflops=flops / ms / 1e9, status=status.tolist())), flush=True)


def main():
    args = parse_args()
    if args.kernel_case:
        run_kernel_case(args)
    elif args.impl == 'reference':
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


def guarded_main():
    """Ranks of a fused multi-GPU run write into each other's buffers, and a rank that exits frees
    its own. So a rank that fails does not leave at once: its kernels finish, then it stays (buffers
    mapped) until the peers' bounded device waits (FGA_TIMEOUT_S, default 20 s) have run out and
    their sticky error status keeps later launches from writing here. Then it exits non-zero."""
    try:
        main()
    except SystemExit:
        raise
    except BaseException:
        import traceback
        traceback.print_exc()
        if int(os.environ.get('WORLD_SIZE', '1')) > 1:
            try:
                import torch
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
            except Exception:
                pass
            time.sleep(float(os.environ.get('FGA_TIMEOUT_S', '20')) + 2.0)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)


if __name__ == '__main__':
    guarded_main()
