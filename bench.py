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

Order of a run: warm-up, a parity check of one step's outputs and gradients against FP32 products
of the same BF16 inputs (sampled row blocks and weight-gradient tiles; a mismatch ends the run on
every rank before anything is timed), graph capture, the timed region, instrumented eager steps
for the per-kernel roofline, the end-to-end measurement. Timed with CUDA events on the launching
stream between a barrier + synchronize on both sides; the maximum over ranks is reported. The
timed region repeats the requested K steps until it is at least --min-seconds long, so that the
clock sampler sees it; `steps` in the line is the number actually timed. `value` is
device-resident throughput; `e2e` repeats the measurement through the public modules with every
step's inputs copied from pinned host memory and the step's results (y and every gradient the
caller receives) copied back to pinned host memory, all inside the timed region.
"""
import argparse
import importlib.util
import json
import math
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
NOMINAL_FP8_TFLOPS = 4500.0
# Peer-copy bandwidth per direction per GPU that the pool's operators measured on these machines
# (nominal NVLink 5: 900 GB/s); the denominator of every link bound below.
LINK_GBS = 770.0
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per FLOP of the GEMM kernel, from the ncu
# captures of `--kernel-case gemm_nt` (670.4 MB) and `--kernel-case wgrad` (1296.8 MB), both
# 824.6 GFLOP launches at 8192 tokens (summaries of both captures are kept under profiles/). The benchmark's
# launches are too large to capture; traffic grows with the rows, so it is scaled by the FLOPs.
DRAM_BYTES_PER_FLOP = dict(gemm=670.4e6 / 824.6e9, wgrad=1296.8e6 / 824.6e9)
# Parity gate in front of the timed region: (max error / largest reference magnitude, relative
# Frobenius error). BF16 as in the test-suite. MXFP8 is compared with the same FP32 products of the
# unquantized inputs, so its bound is the quantization noise itself: an E4M3 value (3 mantissa bits)
# carries a relative rounding error of about 2.6 % RMS, a product of two about 3.7 %, and a sum of
# independent terms keeps that ratio; 8 % leaves room for groups with outliers, whose small members
# lose more, while a wrong head or row mapping shows up as an error of order 100 %.
PARITY_TOLERANCE = dict(bf16=(1e-2, 2e-3), mxfp8=(2.5e-1, 8e-2))


def parity_tolerance(precision, bias, unfused=False):
    """The gate's bound for a run. With a bias the projections round to BF16 twice (GEMM result, then
    the bias add) while the gate's FP32 reference rounds never, which puts the relative Frobenius error
    of a correct BF16 result at about 2.3e-3 (sqrt(2) times a single rounding); the test-suite's oracle
    models that double rounding, the gate allows for it. The unfused comparison arm rounds more often
    still: its dX is the BF16 sum of three or four separately rounded BF16 products (one per
    projection), which measures 2.9e-3 to 3.2e-3 on correct results, so that arm gets twice the bound."""
    worst, frobenius = PARITY_TOLERANCE[precision]
    if unfused:
        return worst, frobenius * 2.0
    return (worst, frobenius * 1.5) if bias and precision == 'bf16' else (worst, frobenius)


def parse_args(argv=None):
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
    ap.add_argument('--min-seconds', type=float, default=2.0,
                    help='the timed region repeats the K steps until it lasts at least this long')
    ap.add_argument('--no-validate', action='store_true', help='skip the parity check in front of the timed region')
    ap.add_argument('--no-e2e', action='store_true', help='skip the host-buffer measurement')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-graphs', action='store_true', help='launch eagerly instead of replaying CUDA graphs')
    ap.add_argument('--cpu-sample-tokens', type=int, default=2048)
    ap.add_argument('--kernel-case', default=None, choices=('gemm_nt', 'gemm_nn', 'wgrad', 'gemm_nt_mx', 'step'),
                    help='run only a few launches of one kernel on a small case (for an ncu capture) and exit')
    ap.add_argument('--case-tokens', type=int, default=8192, help='rows of the --kernel-case problem')
    ap.add_argument('--case-launches', type=int, default=3)
    ap.add_argument('--device', default='cuda', choices=('cuda', 'cpu'),
                    help='cpu: run the harness itself (not the fused kernels) on CPU ranks under gloo; for tests only')
    return ap.parse_args(argv)


def flops_per_step(m, hidden, segments):
    """Algorithmic FLOPs per GPU: forward 2*M*H*N_out, backward (dgrad + wgrad) twice that."""
    qkv, out = 2.0 * m * hidden * segments * hidden, 2.0 * m * hidden * hidden
    return dict(qkv_fwd=qkv, qkv_bwd=2 * qkv, out_fwd=out, out_bwd=2 * out, total=3 * (qkv + out))


def link_bytes_per_step(m, hidden, segments, p):
    """BF16 payload that leaves a GPU per step: one all-to-all per projection per pass (QKV forward
    and backward, output forward and backward), (P-1)/P of it over NVLink."""
    return 2.0 * m * (segments + 1) * hidden * 2 * (p - 1) / p


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


def measured_peaks(precision='bf16'):
    """(peak TFLOP/s, where it comes from). BF16: the pool's measured sustained cuBLAS rate (the
    kernel is timed inside a long, power-capped step). MXFP8: no FP8 rate was measured on this pool,
    so twice the BF16 figure stands in for it (the tensor pipe's FP8 rate is twice its BF16 rate);
    the fraction of the nominal 4500 is reported beside it."""
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        bf16, source = float(peaks.get('bf16_tflops_sustained') or peaks['bf16_tflops']), 'measured (sustained cuBLAS bf16)'
    else:
        bf16, source = 1400.0, 'fallback (sustained, no MEASURED_PEAKS.json)'
    if precision == 'mxfp8':
        return 2.0 * bf16, f'derived: 2 x {source}; no FP8 peak was measured on this pool'
    return bf16, source


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


def timed_steps(requested, estimate_ms, min_seconds):
    """Steps of the timed region: the requested K, repeated a whole number of times until the region
    is expected to last `min_seconds` (a 50 ms clock sampler then has tens of samples inside it)."""
    requested = max(1, requested)
    if estimate_ms <= 0 or min_seconds <= 0:
        return requested
    repeats = max(1, math.ceil(min_seconds * 1e3 / (requested * estimate_ms)))
    return requested * min(repeats, 1000)


# ----------------------------------------------------------------------------------------------
# The reference's own unfused modules (benchmark/reference.py of the reference project), when the
# build step has placed an unmodified copy under oracle/_ref/ (see oracle/build_ref.py).
# ----------------------------------------------------------------------------------------------
def load_reference_modules():
    """The reference's benchmark/reference.py as a module, or None when oracle/_ref/ is absent."""
    path = os.path.join(ROOT, 'oracle', '_ref', 'benchmark', 'reference.py')
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location('fga_reference_unfused', path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


class ReferenceUnfused:
    """The reference's UlyssesQKVProjection / UlyssesOutputProjection (Async-Ulysses: cuBLAS or CPU
    GEMMs with an overlapped torch.distributed all-to-all per projection), unmodified, driven
    through autograd exactly as its own benchmark drives them."""

    kind = 'reference'

    def __init__(self, module, torch, hidden, heads, w_segments, wo, biases, bias_out, device, dtype, gate,
                 cp_group=None):
        self.torch = torch
        with_bias = biases is not None
        self.qkv = module.UlyssesQKVProjection(hidden, heads, bias=with_bias, cp_group=cp_group, device=device,
                                               dtype=dtype, gate=gate)
        self.out = module.UlyssesOutputProjection(hidden, heads, bias=with_bias, cp_group=cp_group, device=device,
                                                  dtype=dtype)
        with torch.no_grad():
            for index, (linear, weight) in enumerate(zip(self.qkv.projections, w_segments)):
                linear.weight.copy_(weight)
                if with_bias:
                    linear.bias.copy_(biases[index])
            self.out.o_proj.weight.copy_(wo)
            if with_bias:
                self.out.o_proj.bias.copy_(bias_out)
        self.qkv_params = [linear.weight for linear in self.qkv.projections]
        self.out_params = [self.out.o_proj.weight]

    def qkv_forward(self, x):
        return list(self.qkv(x))

    def qkv_backward(self, outs, x, grads):
        dx, *dws = self.torch.autograd.grad(outs, [x, *self.qkv_params], grads)
        return dx, dws                       # one weight gradient per segment, in segment order

    def out_forward(self, o):
        return self.out(o)

    def out_backward(self, y, o, dy):
        do, dwo = self.torch.autograd.grad(y, [o, *self.out_params], dy)
        return do, dwo


class NcclUnfused:
    """cuBLAS GEMMs + NCCL all-to-all with the Async-Ulysses overlap (each projection's all-to-all
    is launched before the next projection's GEMM); used as the yardstick only when the reference's
    own modules are not available. Same inputs, same outputs, no autograd graph (explicit backward)."""

    kind = 'port'

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
        return dx, dws              # weight gradients come back last segment first

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


# ----------------------------------------------------------------------------------------------
# CPU arm: the unfused path on the host cores.
# ----------------------------------------------------------------------------------------------
def cpu_unfused_sample(hidden, heads, segments, sample_tokens, steps, warmup):
    """Times forward + backward of both unfused projections for `sample_tokens` tokens of the
    workload on all host cores, FP32 torch CPU GEMMs from BF16-valued inputs. With the reference's
    modules available (oracle/_ref) it is the reference's own code under a one-rank gloo group
    (kind "reference"); otherwise the oracle's restatement of it (kind "port")."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1234)
    bf = torch.bfloat16
    d = hidden // heads
    w_seg = (torch.randn(segments * hidden, hidden, generator=g) / 64).to(bf).float()
    wo = (torch.randn(hidden, hidden, generator=g) / 64).to(bf).float()
    x = torch.randn(sample_tokens, hidden, generator=g).to(bf).float()
    grads = tuple(torch.randn(sample_tokens, heads, d, generator=g).to(bf).float() for _ in range(segments))
    o = torch.randn(sample_tokens, heads, d, generator=g).to(bf).float()
    dy = torch.randn(sample_tokens, hidden, generator=g).to(bf).float()
    module = load_reference_modules()
    if module is not None:
        import torch.distributed as dist
        # A one-rank gloo group of this process: its own default group when nothing is initialized yet,
        # else (the one-GPU benchmark's NCCL group is still alive) a gloo subgroup, because the
        # reference's all-to-all is issued even for a single rank and NCCL cannot move CPU tensors.
        own_group = not dist.is_initialized()
        if own_group:
            dist.init_process_group('gloo', store=dist.HashStore(), rank=0, world_size=1)
            group = None
        else:
            group = dist.new_group(ranks=[dist.get_rank()], backend='gloo')
        arm = ReferenceUnfused(module, torch, hidden, heads, list(w_seg.split(hidden)), wo, None, None, 'cpu',
                               torch.float32, segments == 4, cp_group=group)
        x.requires_grad_()
        o.requires_grad_()

        def step():
            arm.qkv_backward(arm.qkv_forward(x), x, list(grads))
            arm.out_backward(arm.out_forward(o), o, dy)
        kind, what = 'reference', "the reference's unfused modules (unmodified copy of its benchmark/reference.py) under gloo"
    else:
        from oracle.ulysses_oracle import UlyssesOracle, interleave_qkv_rows
        oracle = UlyssesOracle(1, hidden, heads, segments, interleave_qkv_rows(w_seg, heads, d), None, wo, None,
                               dtype=torch.float32, acc_dtype=torch.float32)
        own_group = False

        def step():
            oracle.qkv_forward([x])
            oracle.qkv_backward([x], [grads])
            oracle.out_forward([o])
            oracle.out_backward([o], [dy])
        kind, what = 'port', "the oracle's restatement of the reference's unfused modules"

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = (time.perf_counter() - t0) / steps
    if own_group:
        dist.destroy_process_group()
    flops = flops_per_step(sample_tokens, hidden, segments)['total']
    return dict(value=flops / seconds / 1e12, unit=UNIT, cores=cores, kind=kind,
                sample=f'{sample_tokens} tokens of the workload (H={hidden}, {heads} heads), forward+backward of both '
                       f'projections by {what}, FP32 torch CPU GEMMs, {steps} timed steps of {seconds:.3f} s'), seconds


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
# Parity gate: one step's results against FP32 products of the same inputs
# ----------------------------------------------------------------------------------------------
def sample_rows(torch, m, device, block=128):
    """The first and the last `block` local rows (all rows when there are few)."""
    if m <= 2 * block:
        return torch.arange(m, device=device)
    return torch.cat([torch.arange(block, device=device), torch.arange(m - block, m, device=device)])


def validate_step(torch, dist, rank, p, hidden, heads, inputs, weights, results, tolerance, tile=256):
    """Compare one step's results on this rank with FP32 products of the same inputs, as the
    reference's benchmark does before it times anything (full-token FP32 linear, then this rank's
    heads and rows), on samples that stay cheap at the benchmark's size: two row blocks of every
    row-wise result and two tiles per weight gradient, which sum over all local tokens.

    inputs:  x [M, H], grads: S x [P*M, H/P/D, D], o [P*M, H/P/D, D], dy [M, H]
    weights: w_seg [S*H, H] in segment-major row order [Q; K; V(; G)], wo [H, H], optional biases
    results: outs (S x [P*M, heads/P, D]), dx [M, H], dw_seg [S*H, H] segment-major, y [M, H],
             do [P*M, heads/P, D], dwo [H, H]
    Returns (report dict, list of failures); collective over the group (same calls on every rank)."""
    x, grads, o, dy = inputs['x'], inputs['grads'], inputs['o'], inputs['dy']
    w_seg, wo = weights['w_seg'].float(), weights['wo'].float()
    bq, bo = weights.get('bq'), weights.get('bo')
    segments, m, c = len(grads), x.shape[0], hidden // p
    idx = sample_rows(torch, m, x.device)
    n = idx.numel()
    max_tol, fro_tol = tolerance
    report, failures = {}, []

    def gather(t):
        t = t.contiguous()
        if p == 1:
            return [t]
        parts = [torch.empty_like(t) for _ in range(p)]
        dist.all_gather(parts, t)
        return parts

    def exchange(t):
        """Head side [P*M, c] -> sequence side [M, H]: the all-to-all of the unfused path."""
        t = t.reshape(p * m, c).contiguous()
        if p > 1:
            out = torch.empty_like(t)
            dist.all_to_all_single(out, t)
            t = out
        return t.view(p, m, c).transpose(0, 1).reshape(m, hidden)

    def check(name, actual, expected):
        actual, expected = actual.detach().float(), expected.float()
        if actual.shape != expected.shape:
            failures.append(f'{name}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}')
            return
        scale = expected.abs().max().clamp_min(1e-6)
        worst = ((actual - expected).abs().max() / scale).item()
        fro = (torch.linalg.norm(actual - expected) / torch.linalg.norm(expected).clamp_min(1e-6)).item()
        report[name] = dict(max_rel=worst, frobenius=fro)
        if not (worst <= max_tol and fro <= fro_tol):     # also catches NaN
            failures.append(f'{name}: max error {worst:.3g} of scale, Frobenius {fro:.3g}')

    def sampled_sequence_side(t):
        """Rows `idx` of this rank's sequence-side matrix, assembled from every rank's head-side t."""
        mine = gather(t.reshape(p, m, c)[:, idx])          # [dst][src, n, c]
        return torch.cat([part[rank] for part in mine], dim=1)   # [n, H]

    # ---- QKV forward: out[s][src*M + i, heads of this rank] = x_src[i] . W_s[heads of this rank]
    xs = gather(x[idx])
    for s in range(segments):
        rows = w_seg[s * hidden + rank * c:s * hidden + (rank + 1) * c]
        expected = torch.stack([xr.float() @ rows.t() for xr in xs])          # [src, n, c]
        if bq is not None:
            expected = expected + bq[s * hidden + rank * c:s * hidden + (rank + 1) * c].float()
        actual = results['outs'][s].reshape(p, m, c)[:, idx]
        check(f'qkv_fwd segment {s}', actual, expected)
    # ---- QKV backward: dx = sum_s dY_s W_s ; dW_s = dY_s^T x over all local tokens
    dx = torch.zeros(n, hidden, dtype=torch.float32, device=x.device)
    for s in range(segments):
        dx += sampled_sequence_side(grads[s]).float() @ w_seg[s * hidden:(s + 1) * hidden]
    check('qkv_bwd dx', results['dx'][idx], dx)
    corners = [(0, 0), (hidden - tile, hidden - tile)]
    x32 = x.detach().float()
    for s in range(segments):
        dy_s = exchange(grads[s]).float()
        for r0, c0 in corners:
            expected = dy_s[:, r0:r0 + tile].t() @ x32[:, c0:c0 + tile]
            check(f'qkv_bwd dW segment {s} tile {r0},{c0}',
                  results['dw_seg'][s * hidden + r0:s * hidden + r0 + tile, c0:c0 + tile], expected)
        del dy_s
    # ---- output forward: y = O_seq Wo^T
    y = sampled_sequence_side(o.detach()).float() @ wo.t()
    if bo is not None:
        y = y + bo.float()
    check('out_fwd y', results['y'][idx], y)
    # ---- output backward: dO[src*M + i, heads of this rank] = dy_src[i] . Wo[:, columns of this rank]
    dys = gather(dy[idx])
    expected = torch.stack([dr.float() @ wo[:, rank * c:(rank + 1) * c] for dr in dys])
    check('out_bwd dO', results['do'].reshape(p, m, c)[:, idx], expected)
    o_seq, dy32 = exchange(o.detach()).float(), dy.float()
    for r0, c0 in corners:
        check(f'out_bwd dW tile {r0},{c0}', results['dwo'][r0:r0 + tile, c0:c0 + tile],
              dy32[:, r0:r0 + tile].t() @ o_seq[:, c0:c0 + tile])
    return report, failures


# ----------------------------------------------------------------------------------------------
# GPU arms
# ----------------------------------------------------------------------------------------------
class CudaApi:
    """The CUDA runtime objects the measurement uses, behind one object so that the control flow of a
    run (warm-up, parity gate, timed region, end-to-end leg, the JSON line) can be exercised on CPU
    ranks by the tests with HostApi in its place."""

    name, backend = 'cuda', 'nccl'

    def __init__(self, torch, local):
        self.torch, self.local = torch, local
        torch.cuda.set_device(local)
        self.device = torch.device('cuda', local)
        self.Stream, self.CUDAGraph = torch.cuda.Stream, torch.cuda.CUDAGraph
        self.set_stream, self.current_stream, self.stream = torch.cuda.set_stream, torch.cuda.current_stream, torch.cuda.stream
        self.synchronize, self.graph = torch.cuda.synchronize, torch.cuda.graph

    def Event(self, enable_timing=False):
        return self.torch.cuda.Event(enable_timing=enable_timing)

    def generator(self, seed):
        return self.torch.Generator(device=self.device).manual_seed(seed)

    @staticmethod
    def pin(tensor):
        return tensor.pin_memory()

    def init_process_group(self, dist, rank, world):
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=self.device)


class HostApi:
    """CPU stand-in for CudaApi (tests only; `--device cpu`, no fused arm): work is done when the call
    returns, so an event is a timestamp, a stream does nothing, and graph capture is refused (the
    run then takes its eager path). Numbers printed with it are not measurements of anything."""

    name, backend = 'cpu', 'gloo'

    class _Event:
        def __init__(self):
            self.t = None

        def record(self, *_):
            self.t = time.perf_counter()

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

        def synchronize(self):
            return None

        @staticmethod
        def query():
            return True

    class _Stream:
        def wait_event(self, *_):
            return None

        def wait_stream(self, *_):
            return None

        def synchronize(self):
            return None

    def __init__(self, torch, local):
        import contextlib
        self.torch, self.local, self.device = torch, local, torch.device('cpu')
        self._stream, self._null = self._Stream(), contextlib.nullcontext

    def Event(self, enable_timing=False):
        return self._Event()

    def Stream(self):
        return self._Stream()

    def CUDAGraph(self):
        raise RuntimeError('no graph capture on the host')

    def graph(self, *a, **kw):
        raise RuntimeError('no graph capture on the host')

    def set_stream(self, *_):
        return None

    def current_stream(self):
        return self._stream

    def stream(self, *_):
        return self._null()

    def synchronize(self):
        return None

    def generator(self, seed):
        return self.torch.Generator().manual_seed(seed)

    @staticmethod
    def pin(tensor):
        return tensor

    def init_process_group(self, dist, rank, world):
        dist.init_process_group('gloo', rank=rank, world_size=world)


def init_distributed(torch, dist, device='cuda'):
    world = int(os.environ.get('WORLD_SIZE', 1))
    rank = int(os.environ.get('RANK', 0))
    local = int(os.environ.get('LOCAL_RANK', 0))
    api = (HostApi if device == 'cpu' else CudaApi)(torch, local)
    if not dist.is_initialized():
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29555')
        api.init_process_group(dist, rank, world)
    return rank, world, local, api


def interleave(seg_major, heads, d):
    s = seg_major.shape[0] // (heads * d)
    return seg_major.reshape(s, heads, d, -1).transpose(0, 1).reshape(seg_major.shape)


def deinterleave(per_head, heads, d):
    s = per_head.shape[0] // (heads * d)
    return per_head.reshape(heads, s, d, -1).transpose(0, 1).reshape(per_head.shape)


class FusedArm:
    """This repository's path behind the harness: the public modules over libfga.so, with the weights
    in the per-head interleaved row order the modules take. passes = the four passes of a step, each
    reading and writing the shared `state`; results() = the step's results in the arm-independent form
    validate_step() takes (weight gradients back in segment-major row order)."""

    note = 'this repository: libfga.so through the public modules'

    def __init__(self, torch, fused, hidden, heads, m, data, parameters, gate=False, precision='bf16'):
        self.torch, self.heads, self.d = torch, heads, hidden // heads
        self.x, self.grads, self.o, self.dy = data['x'], data['grads'], data['o'], data['dy']
        self.ws = fused.FusedGemmA2AWorkspace(hidden, heads, m, gate=gate, precision=precision)
        wq = interleave(parameters['w_seg'], heads, self.d).contiguous().requires_grad_()
        wo = parameters['wo'].clone().requires_grad_()
        with_bias = parameters.get('bq') is not None
        bq = interleave(parameters['bq'], heads, self.d).contiguous().requires_grad_() if with_bias else None
        bo = parameters['bo'].clone().requires_grad_() if with_bias else None
        self.qkv = fused.FusedQKVProjection(hidden, heads, weight=wq, bias=bq, gate=gate)
        self.proj = fused.FusedOutputProjection(hidden, heads, weight=wo, bias=bo)
        self.x.requires_grad_()
        self.o.requires_grad_()
        self.qkv_params = [wq] + ([bq] if with_bias else [])
        self.out_params = [wo] + ([bo] if with_bias else [])
        self.passes = (self.qkv_fwd, self.qkv_bwd, self.out_fwd, self.out_bwd)

    def qkv_fwd(self, state):
        state['qs'] = self.qkv(self.x, self.ws)

    def qkv_bwd(self, state):
        state['dq'] = self.torch.autograd.grad(state['qs'], [self.x, *self.qkv_params], self.grads)

    def out_fwd(self, state):
        state['y'] = self.proj(self.o, self.ws)

    def out_bwd(self, state):
        state['do'] = self.torch.autograd.grad(state['y'], [self.o, *self.out_params], self.dy)

    def results(self, state):
        return dict(outs=list(state['qs']), dx=state['dq'][0], dw_seg=deinterleave(state['dq'][1], self.heads, self.d),
                    y=state['y'], do=state['do'][0], dwo=state['do'][1])


class UnfusedArm:
    """The comparison arm behind the same harness: the reference's own Async-Ulysses modules when the
    build step has staged them (`module`), else the restatement in this file (no bias support)."""

    def __init__(self, torch, dist, module, p, hidden, heads, data, parameters, device, dtype, gate):
        self.torch = torch
        self.x, self.grads, self.o, self.dy = data['x'], data['grads'], data['o'], data['dy']
        w_segments, wo = list(parameters['w_seg'].split(hidden)), parameters['wo']
        self.staged = module is not None
        if self.staged:
            with_bias = parameters.get('bq') is not None
            seg_biases = list(parameters['bq'].split(hidden)) if with_bias else None
            self.ref = ReferenceUnfused(module, torch, hidden, heads, w_segments, wo, seg_biases, parameters.get('bo'),
                                        device, dtype, gate)
            self.x.requires_grad_()
            self.o.requires_grad_()
            self.note = ("the reference's Async-Ulysses modules (unmodified copy of its benchmark/reference.py): "
                         'cuBLAS + NCCL')
        else:
            self.ref = NcclUnfused(torch, dist, p, hidden, heads, w_segments, wo)
            self.note = 'cuBLAS + NCCL all-to-all with the Async-Ulysses overlap, restated in bench.py (oracle/_ref absent)'
        self.passes = (self.qkv_fwd, self.qkv_bwd, self.out_fwd, self.out_bwd)

    def qkv_fwd(self, state):
        state['qs'] = self.ref.qkv_forward(self.x)

    def qkv_bwd(self, state):
        state['dq'] = (self.ref.qkv_backward(state['qs'], self.x, self.grads) if self.staged
                       else self.ref.qkv_backward(self.x, self.grads))

    def out_fwd(self, state):
        state['y'] = self.ref.out_forward(self.o)

    def out_bwd(self, state):
        state['do'] = (self.ref.out_backward(state['y'], self.o, self.dy) if self.staged
                       else self.ref.out_backward(self.dy))

    def results(self, state):
        # the restated arm returns its weight gradients last segment first
        dws = list(state['dq'][1]) if self.staged else list(reversed(state['dq'][1]))
        return dict(outs=list(state['qs']), dx=state['dq'][0], dw_seg=self.torch.cat(dws), y=state['y'],
                    do=state['do'][0], dwo=state['do'][1])


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    rank, world, local, api = init_distributed(torch, dist, args.device)
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run')
    if args.tokens % world or args.heads % world:
        raise SystemExit('tokens and heads must divide over the ranks')
    if args.device == 'cpu' and args.impl == 'fused':
        raise SystemExit('--device cpu exercises the harness with the unfused arm only; the fused path has no CPU fallback')
    torch.backends.cuda.matmul.allow_tf32 = False      # the parity gate multiplies in true FP32
    dev = api.device
    # Everything runs on one non-default stream from the start: autograd ties the gradient
    # accumulation nodes of the leaves to the stream of their first use, and a node tied to the
    # legacy default stream cannot take part in a stream capture.
    work_stream = api.Stream()
    api.set_stream(work_stream)
    p, hidden, heads = world, args.hidden, args.heads
    d, m, segments = hidden // heads, args.tokens // world, 4 if args.gate else 3
    bf = torch.bfloat16 if args.device == 'cuda' else torch.float32
    flops = flops_per_step(m, hidden, segments)

    # ---- synthetic data: weights identical on every rank, activations per rank
    gen = api.generator(1234)
    w_seg = (torch.randn(segments * hidden, hidden, generator=gen, device=dev) / 64).to(bf)
    wo = (torch.randn(hidden, hidden, generator=gen, device=dev) / 64).to(bf)
    bq = (torch.randn(segments * hidden, generator=gen, device=dev) * 0.02).to(bf) if args.bias else None
    bo = (torch.randn(hidden, generator=gen, device=dev) * 0.02).to(bf) if args.bias else None
    gen = api.generator(1234 + 1 + rank)
    x = torch.randn(m, hidden, generator=gen, device=dev).to(bf)
    grads = [torch.randn(p * m, heads // p, d, generator=gen, device=dev).to(bf) for _ in range(segments)]
    o = torch.randn(p * m, heads // p, d, generator=gen, device=dev).to(bf)
    dy = torch.randn(m, hidden, generator=gen, device=dev).to(bf)
    inputs = [x, *grads, o, dy]

    launches = lambda: 0  # noqa: E731
    state = {}
    fused = ws = None
    data = dict(x=x, grads=grads, o=o, dy=dy)
    parameters = dict(w_seg=w_seg, wo=wo, bq=bq, bo=bo)
    if args.impl == 'fused':
        import build_native
        build_native.build()
        import _fga_native
        import fused_gemm_a2a as fused
        fused.install_exit_guards()
        launches = _fga_native.lib().fga_launch_count
        arm = FusedArm(torch, fused, hidden, heads, m, data, parameters, gate=args.gate, precision=args.precision)
        ws = arm.ws
    else:
        module = load_reference_modules()
        if module is None and args.bias:
            raise SystemExit('--impl nccl --bias needs the staged reference modules (oracle/_ref): the restated arm has no bias')
        arm = UnfusedArm(torch, dist, module, p, hidden, heads, data, parameters, dev, bf, args.gate)
    arm_note = arm.note
    qkv_fwd, qkv_bwd, out_fwd, out_bwd = (lambda fn=fn: fn(state) for fn in arm.passes)

    def results():
        return arm.results(state)

    fns = (qkv_fwd, qkv_bwd, out_fwd, out_bwd)
    names = ('qkv_fwd', 'qkv_bwd', 'out_fwd', 'out_bwd')

    def eager_step(events=None):
        for i, fn in enumerate(fns):
            fn()
            if events is not None:
                events[i + 1].record()

    step = eager_step

    def fence():
        api.synchronize()
        dist.barrier()
        api.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def device_status():
        if ws is not None:
            ws.comm.check_status()

    # ---- warm-up, parity gate, graph capture, timed region (the clock sampler starts before the
    # warm-up so that it is already streaming when the timed region begins)
    warmup = max(args.warmup, 3)
    graph_note = 'eager launches'
    parity = None
    with ClockSampler(local) as clocks:
        for _ in range(warmup):
            eager_step()
        fence()
        device_status()
        if not args.no_validate:
            # Nothing is timed before one step's results have been checked; a mismatch on any rank
            # ends the run on every rank (nobody leaves alone).
            tolerance = parity_tolerance(args.precision if args.impl == 'fused' else 'bf16', args.bias,
                                         unfused=args.impl != 'fused')
            report, failures = validate_step(
                torch, dist, rank, p, hidden, heads, dict(x=x.detach(), grads=grads, o=o.detach(), dy=dy),
                dict(w_seg=w_seg, wo=wo, bq=bq, bo=bo), results(), tolerance)
            failed, = max_over_ranks([float(len(failures))])
            if failed:
                raise RuntimeError(f'parity check failed before timing (rank {rank}: {failures})')
            parity = dict(passed=True, checked=sorted(report), sampled_rows_per_rank=int(min(m, 256)),
                          reference='FP32 products of the same BF16 inputs (full-token linear, this rank\'s heads and rows)',
                          tolerance=dict(max_error_over_scale=tolerance[0], relative_frobenius=tolerance[1]),
                          worst_max_error_over_scale=max(v['max_rel'] for v in report.values()),
                          worst_relative_frobenius=max(v['frobenius'] for v in report.values()))
            fence()
        launches_per_step = None
        if not args.no_graphs:
            # One CUDA graph per pass (shared memory pool), replayed back to back: launch latency of
            # the host is out of the measurement, as in the reference's graph-captured benchmark.
            try:
                fence()
                graphs, pool, before = [], None, launches()
                for fn in fns:
                    g = api.CUDAGraph()
                    with api.graph(g, pool=pool, stream=work_stream, capture_error_mode='thread_local'):
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
        # Two more warm steps in the final launch mode, timed, to size the region.
        probe = [api.Event(enable_timing=True) for _ in range(2)]
        step()
        probe[0].record()
        for _ in range(2):
            step()
        probe[1].record()
        fence()
        estimate_ms, = max_over_ranks([probe[0].elapsed_time(probe[1]) / 2])
        steps = timed_steps(args.steps, estimate_ms, args.min_seconds)
        marks = [[api.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
        fence()
        launches_before = launches()
        clocks.begin()
        for k in range(steps):
            marks[k][0].record()
            step(marks[k])
        # ---- the GEMM kernel alone, in the same power state: instrumented eager steps are queued
        # right behind the timed region, with no fence and no idle gap in between
        instrumented = None
        if args.impl == 'fused':
            instrumented = queue_instrumented_steps(api, fused, ws, eager_step, m, extra=10)
        marks[-1][4].synchronize()
        clocks.end()
        fence()
    gpu_launches = launches() - launches_before
    if instrumented is not None:
        gpu_launches -= instrumented['launches']
    if launches_per_step is not None and step is not eager_step:
        gpu_launches = launches_per_step * steps  # replayed launches are not seen by the counter
    total_ms = marks[0][0].elapsed_time(marks[-1][4])
    pass_ms = [sum(marks[k][i].elapsed_time(marks[k][i + 1]) for k in range(steps)) / steps for i in range(4)]
    total_ms, *pass_ms = max_over_ranks([total_ms, *pass_ms])
    ms_per_step = total_ms / steps
    per_gpu_tflops = flops['total'] / (ms_per_step * 1e-3) / 1e12
    device_status()

    roofline = None
    if instrumented is not None:
        roofline = kernel_roofline(args, instrumented, max_over_ranks, m, hidden, segments, p, ms_per_step, flops)

    e2e = None
    if not args.no_e2e:
        e2e = end_to_end(torch, api, args, inputs, state, step, fence, max_over_ranks, world, flops)
        device_status()

    if rank == 0:
        link_ms = link_bytes_per_step(m, hidden, segments, p) / (LINK_GBS * 1e9) * 1e3
        nominal = NOMINAL_BF16_TFLOPS if args.precision == 'bf16' else NOMINAL_FP8_TFLOPS
        compute_ms = flops['total'] / nominal / 1e9
        line = dict(
            metric=METRIC, value=world * per_gpu_tflops, unit=UNIT, n_gpus=world, steps=steps, steps_requested=args.steps,
            warmup=warmup, ms_per_step=ms_per_step, higher_is_better=True, scaling='strong',
            vs_baseline=None,
            dtype='bf16' if args.precision == 'bf16' else 'mxfp8 (e4m3 payload, e8m0 scale per 32, fp32 accumulate)',
            data='synthetic', impl=args.impl,
            config=dict(workload=f'{args.tokens} total tokens, H={hidden}, {heads}x{d} heads, CP={world} '
                                 f'(M={m} per rank), QKV{"G" if args.gate else ""} + output projection, forward + dgrad + wgrad'
                                 f'{", bias" if args.bias else ", no bias"}',
                        parallelism=f'cp{world}', l2='inputs larger than L2 (no flush needed)', launch=graph_note,
                        arm=arm_note,
                        timed_region=f'{steps} steps = {steps // max(1, args.steps)} x the requested {args.steps}, so that the '
                                     f'region lasts at least {args.min_seconds} s'),
            tflops_per_gpu=per_gpu_tflops, pct_of_nominal=100 * per_gpu_tflops / nominal, nominal_tflops=nominal,
            passes={n: dict(ms=ms, tflops_per_gpu=flops[n] / (ms * 1e-3) / 1e12) for n, ms in zip(names, pass_ms)},
            step_roofline=dict(compute_ms_at_nominal=compute_ms, link_ms_at_770GBs=link_ms,
                               frac=max(compute_ms, link_ms) / ms_per_step),
            parity_check=parity if parity is not None else dict(passed=None, note='skipped (--no-validate)'),
            clocks=clocks.summary(), gpu_launches=int(gpu_launches), provenance=provenance(torch))
        if roofline is not None:
            line['roofline'] = roofline
        if e2e is not None:
            line['e2e'] = e2e
        if world == 1 and args.impl == 'fused' and not args.no_cpu_baseline:
            try:
                line['cpu_baseline'], _ = cpu_unfused_sample(hidden, heads, segments, args.cpu_sample_tokens, 2, 1)
            except Exception as error:     # the device measurements above must not be lost to the host-side leg
                line['cpu_baseline'] = dict(value=None, unit=UNIT, unavailable=f'{type(error).__name__}: {str(error)[:300]}')
        print(json.dumps(line), flush=True)
    # ---- leave together: every rank drains its device and gives its symmetric buffers back
    fence()
    if fused is not None:
        fused.release_all()
    dist.barrier()
    dist.destroy_process_group()


def queue_instrumented_steps(api, fused, ws, eager_step, m, extra):
    """Queue `extra` eager steps with CUDA events around every libfga launch of the host layer.
    Returns the recorded events; durations are read after the device has been synchronized."""
    import _fga_native
    records, others = [], []

    def timed(fn, label, algorithmic_flops=None):
        def wrapper(*a, **kw):
            e0, e1 = api.Event(enable_timing=True), api.Event(enable_timing=True)
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

    def gemm_flops(mode, a, b, b_is_kn, c, aux, counters, num_in, n_segment, num_segments, *rest, **kw):
        # algorithmic rows only: pad rows of the capacity are not counted
        width = n_segment * num_segments if mode == 'push' else c.shape[1]
        return 2.0 * m * a.shape[1] * width

    def gemm_label(mode, a, b, b_is_kn, c, aux, counters, num_in, n_segment, num_segments, *rest, **kw):
        width = n_segment * num_segments if mode == 'push' else c.shape[1]
        return f'gemm_{mode}{"_mx" if kw.get("scales") else ""}[{m}x{a.shape[1]}->{width}]'

    comm = ws.comm
    saved = (comm.gemm, fused.bf16_wgrad, fused.mxfp8_wgrad, fused.mxfp8_quantize, comm.barrier, fused.resize_rank_rows,
             fused.reduce_bias_grad)
    comm.gemm = timed(saved[0], gemm_label, gemm_flops)
    fused.bf16_wgrad = timed(saved[1], lambda dyv, xv, *a, **kw: f'gemm_wgrad[{dyv.shape[1]}x{xv.shape[1]},k={dyv.shape[0]}]',
                             lambda dyv, xv, *a, **kw: 2.0 * dyv.shape[0] * dyv.shape[1] * xv.shape[1])
    fused.mxfp8_wgrad = timed(saved[2], lambda dyv, xv, *a, **kw: f'wgrad_mx incl. 2 quantizer passes[{dyv.shape[1]}x{xv.shape[1]},k={dyv.shape[0]}]',
                              lambda dyv, xv, *a, **kw: 2.0 * dyv.shape[0] * dyv.shape[1] * xv.shape[1])
    fused.mxfp8_quantize = timed(saved[3], 'mx_quantize')
    comm.barrier = timed(saved[4], 'barrier')
    fused.resize_rank_rows = timed(saved[5], 'copy_rank_rows')
    fused.reduce_bias_grad = timed(saved[6], 'bias_grad')
    before = _fga_native.lib().fga_launch_count()
    try:
        for _ in range(extra):
            eager_step()
    finally:
        (comm.gemm, fused.bf16_wgrad, fused.mxfp8_wgrad, fused.mxfp8_quantize, comm.barrier, fused.resize_rank_rows,
         fused.reduce_bias_grad) = saved
    return dict(records=records, others=others, extra=extra, launches=_fga_native.lib().fga_launch_count() - before)


def kernel_roofline(args, instrumented, max_over_ranks, m, hidden, segments, p, ms_per_step, flops):
    """The roofline object of the GEMM kernel from the instrumented steps (the first two of them
    are dropped: they overlap the tail of the graph replays on the host side)."""
    peak, peak_source = measured_peaks(args.precision)
    extra = instrumented['extra']
    per_step_gemm = len(instrumented['records']) // extra
    per_step_other = len(instrumented['others']) // extra
    records = instrumented['records'][2 * per_step_gemm:]
    others = instrumented['others'][2 * per_step_other:]
    counted = extra - 2
    gemm_ms = sum(e0.elapsed_time(e1) for _, e0, e1, _ in records)
    other_ms = sum(e0.elapsed_time(e1) for _, e0, e1 in others)
    gemm_flops_total = sum(f for *_, f in records)
    per_launch = [dict(op=name, ms=e0.elapsed_time(e1), tflops=f / e0.elapsed_time(e1) / 1e9)
                  for name, e0, e1, f in records[-per_step_gemm:]]
    per_launch += [dict(op=name, ms=e0.elapsed_time(e1)) for name, e0, e1 in others[-per_step_other:]]
    gemm_ms, other_ms = max_over_ranks([gemm_ms, other_ms])
    achieved = gemm_flops_total / (gemm_ms * 1e-3) / 1e12
    # operands and outputs of the six GEMMs of a step: activations and their gradients are touched
    # by the forward, dgrad and wgrad launch; the weight is read twice and its BF16 gradient written
    algorithmic_bytes = sum(2.0 * (3 * (m * hidden + m * s * hidden) + 3 * s * hidden * hidden)
                            for s in (segments, 1)) / 6
    traffic = None
    if args.precision == 'bf16':
        traffic = sum(f * DRAM_BYTES_PER_FLOP['wgrad' if 'wgrad' in name else 'gemm']
                      for name, _, _, f in records) / max(1, len(records))
    # The same rate seen from the timed region: the step's time minus what the non-GEMM launches
    # (barriers, row copies, quantizer and bias passes) took in the instrumented steps.
    implied_ms = ms_per_step - other_ms / counted
    nominal = NOMINAL_BF16_TFLOPS if args.precision == 'bf16' else NOMINAL_FP8_TFLOPS
    return dict(bound='tensor', kernel='ulysses_gemm_kernel' + ('<mx>' if args.precision == 'mxfp8' else ''),
                achieved=achieved, peak=peak, unit='TFLOP/s', frac=achieved / peak, traffic=traffic,
                traffic_source=None if traffic is None else
                'scaled: DRAM bytes per launch (mean over the 6 launches of a step) from ncu captures of 8192-token '
                'launches of the same kernel, scaled by each launch\'s FLOPs; not captured at this size',
                algorithmic_bytes_per_launch=algorithmic_bytes,
                peak_source=peak_source, frac_of_nominal=achieved / nominal, nominal_tflops=nominal,
                launches_timed=len(records), avg_launch_ms=gemm_ms / max(1, len(records)),
                timed_in=f'{counted} eager steps queued directly behind the timed region (same power state)',
                gemm_ms_per_step=gemm_ms / counted, other_launches_ms_per_step=other_ms / counted,
                gemm_share_of_step=(gemm_ms / counted) / ms_per_step,
                gemm_tflops_implied_by_timed_step=flops['total'] / (implied_ms * 1e-3) / 1e12 if implied_ms > 0 else None,
                link_bound_ms_per_step=link_bytes_per_step(m, hidden, segments, p) / (LINK_GBS * 1e9) * 1e3,
                launches_rank0_last_step=per_launch)


def end_to_end(torch, api, args, inputs, state, step, fence, max_over_ranks, world, flops):
    """The same K steps through the public modules with host buffers: inside the timed region every
    step's inputs travel from pinned host memory to the device (copy stream, double-buffered, so
    step k+1's copy overlaps step k's compute) and every step's results - y and every gradient the
    caller receives (dx, dW_qkv, dO, dW_o) - travel back to pinned host memory (second copy stream,
    double-buffered device staging). The first copy is issued after the start event."""
    def step_results():
        return [state['y'], state['dq'][0], *_tensors(state['dq'][1]), state['do'][0], *_tensors(state['do'][1])]

    def _tensors(value):
        return list(value) if isinstance(value, (list, tuple)) else [value]

    step()                                   # results of the final launch mode exist: size the buffers
    api.synchronize()
    shapes = [t.detach() for t in step_results()]
    h2d_bytes = sum(t.numel() * t.element_size() for t in inputs)
    d2h_bytes = sum(t.numel() * t.element_size() for t in shapes)
    # Pinned host buffers (inputs once, results twice) and device staging (both twice). A host that cannot
    # pin that much must not cost the run its line: every rank reports, and if any could not, all skip the leg.
    problem = ''
    try:
        host_in = [api.pin(t.detach().to('cpu')) for t in inputs]
        staged_in = [[torch.empty_like(t.detach()) for t in inputs] for _ in range(2)]
        staged_out = [[torch.empty_like(t) for t in shapes] for _ in range(2)]
        host_out = [[api.pin(torch.empty(t.shape, dtype=t.dtype)) for t in shapes] for _ in range(2)]
    except (RuntimeError, MemoryError) as error:
        problem = f'{type(error).__name__}: {str(error)[:200]}'
        host_in = staged_in = staged_out = host_out = None
    failed, = max_over_ranks([1.0 if problem else 0.0])
    if failed:
        return dict(value=None, unit=UNIT, h2d_bytes_per_step=h2d_bytes, d2h_bytes_per_step=d2h_bytes,
                    unavailable='the staging buffers of the end-to-end leg could not be allocated on every rank'
                                + (f' ({problem})' if problem else ''))
    h2d_stream, d2h_stream = api.Stream(), api.Stream()
    ready = [api.Event() for _ in range(2)]          # inputs of the slot are on the device
    consumed = [api.Event() for _ in range(2)]       # the step has taken them over
    produced = [api.Event() for _ in range(2)]       # results of the slot are staged
    drained = [api.Event() for _ in range(2)]        # and have reached the host

    def prefetch(slot):
        with api.stream(h2d_stream):
            h2d_stream.wait_event(consumed[slot])
            for dst, src in zip(staged_in[slot], host_in):
                dst.copy_(src, non_blocking=True)
            ready[slot].record(h2d_stream)

    def e2e_step(slot):
        cur = api.current_stream()
        cur.wait_event(ready[slot])
        with torch.no_grad():
            for dst, src in zip(inputs, staged_in[slot]):
                dst.copy_(src)               # device-to-device hand-over into the tensors the modules hold
        consumed[slot].record(cur)
        step()
        cur.wait_event(drained[slot])        # the staging buffers of this slot are free again
        with torch.no_grad():
            for dst, src in zip(staged_out[slot], step_results()):
                dst.copy_(src.detach())
        produced[slot].record(cur)
        with api.stream(d2h_stream):
            d2h_stream.wait_event(produced[slot])
            for dst, src in zip(host_out[slot], staged_out[slot]):
                dst.copy_(src, non_blocking=True)
            drained[slot].record(d2h_stream)

    for ev in (*consumed, *drained):
        ev.record()
    fence()
    prefetch(0)
    e2e_step(0)          # warm-up of the staging path
    fence()
    t0, t1 = api.Event(enable_timing=True), api.Event(enable_timing=True)
    t0.record()
    h2d_stream.wait_event(t0)                # the first copy starts inside the timed region
    prefetch(0)
    for k in range(args.steps):
        if k + 1 < args.steps:
            prefetch((k + 1) % 2)
        e2e_step(k % 2)
    api.current_stream().wait_stream(d2h_stream)     # the last results are on the host
    t1.record()
    fence()
    e2e_ms, = max_over_ranks([t0.elapsed_time(t1)])
    e2e_ms_per_step = e2e_ms / args.steps
    checksum = float(host_out[(args.steps - 1) % 2][0].float().sum())    # read on the host: the copy really happened
    return dict(value=world * flops['total'] / (e2e_ms_per_step * 1e-3) / 1e12, unit=UNIT,
                h2d_bytes_per_step=h2d_bytes, d2h_bytes_per_step=d2h_bytes, ms_per_step=e2e_ms_per_step,
                steps=args.steps, y_checksum_on_host=checksum,
                note='per step: inputs (x, upstream gradients, o, dy) from pinned host memory, results (y, dx, dW_qkv, dO, '
                     'dW_o) back to pinned host memory; copies run on two copy streams and overlap the neighbouring '
                     'steps\' compute; at one GPU the step is bound by the host link, not by the kernels')


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
        ws = fused.FusedGemmA2AWorkspace(h, args.heads, m, precision=args.precision)
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
        elif args.kernel_case == 'gemm_nt_mx':  # the same product with MXFP8 operands (quantized once, outside)
            from fused_gemm_a2a_kernels import mxfp8_quantize
            b, c = torch.randn(n, h, device=dev).to(bf), torch.empty(m, n, dtype=bf, device=dev)
            aq, sa = mxfp8_quantize(a)
            bq, sb = mxfp8_quantize(b)
            call = lambda: lib.fga_gemm_local_mx(aq.data_ptr(), sa.data_ptr(), aq.shape[0], bq.data_ptr(), sb.data_ptr(),  # noqa: E731
                                                 bq.shape[0], m, n, aq.shape[1], c.data_ptr(), n, 0, 0,
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
    """Ranks of a fused multi-GPU run write into each other's buffers. A rank that fails does not
    leave at once: its queued kernels finish and, where its buffers would disappear with the
    process (cudaMalloc + IPC backing), it keeps them mapped until the peers' bounded device waits
    have run out and their sticky error status keeps later launches from writing here
    (fused_gemm_a2a.hold_buffers_after_failure). Then it exits non-zero."""
    try:
        main()
    except SystemExit:
        raise
    except BaseException:
        import traceback
        traceback.print_exc()
        try:
            held = sys.modules.get('fused_gemm_a2a')
            if held is not None:
                held.hold_buffers_after_failure()
            else:
                torch = sys.modules.get('torch')
                if torch is not None and torch.cuda.is_available():
                    torch.cuda.synchronize()
        except Exception:
            pass
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)


if __name__ == '__main__':
    guarded_main()
