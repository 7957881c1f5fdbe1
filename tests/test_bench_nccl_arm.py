"""The comparison arm of bench.py (`--impl nccl`: cuBLAS GEMMs + an all-to-all per projection) must
compute the same projections as the fused path it is timed against. Here it runs on two and four
CPU ranks under gloo in FP32 and is compared with the oracle: same outputs, same gradients, same
head-side layouts. The benchmark's own parity gate (validate_step) is exercised on the same data:
it must accept correct results and name the tensor that is wrong."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def worker(rank, world, port, queue):
    for path in (ROOT, os.path.join(ROOT, 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import bench
    from oracle.ulysses_oracle import UlyssesOracle, interleave_qkv_rows
    hidden, heads, tokens, segments = 256, 4, 5, 3
    d = hidden // heads
    g = torch.Generator().manual_seed(7)
    w_seg = torch.randn(segments * hidden, hidden, generator=g) / hidden ** 0.5      # segment-major [Q; K; V]
    wo = torch.randn(hidden, hidden, generator=g) / hidden ** 0.5
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(tokens, hidden, generator=g)
    grads = [torch.randn(world * tokens, heads // world, d, generator=g) for _ in range(segments)]
    o = torch.randn(world * tokens, heads // world, d, generator=g)
    dy = torch.randn(tokens, hidden, generator=g)
    arm = bench.NcclUnfused(torch, dist, world, hidden, heads, list(w_seg.split(hidden)), wo)
    outs = arm.qkv_forward(x)
    dx, dws = arm.qkv_backward(x, grads)
    y = arm.out_forward(o)
    do, dwo = arm.out_backward(dy)

    def everyone(value):
        box = [None] * world
        dist.all_gather_object(box, value)
        return box

    oracle = UlyssesOracle(world, hidden, heads, segments, interleave_qkv_rows(w_seg, heads, d), None, wo, None,
                           dtype=torch.float32)
    xs, all_grads, all_o, dys = everyone(x), everyone(tuple(grads)), everyone(o), everyone(dy)
    problems = []

    def same(actual, expected, what):
        if actual.shape != expected.shape or not torch.allclose(actual, expected, rtol=1e-4, atol=1e-4):
            problems.append(what)

    for name, got, want in zip('qkv', outs, oracle.qkv_forward(xs)[rank]):
        same(got, want, name)
    rdx, rdw, _ = oracle.qkv_backward(xs, all_grads)[rank]
    same(dx, rdx, 'dx')
    # the arm keeps one weight per segment (dws comes back last segment first); the oracle's is interleaved per head
    per_segment = torch.cat(list(reversed(dws)))
    same(interleave_qkv_rows(per_segment, heads, d), rdw, 'dW_qkv')
    same(y, oracle.out_forward(all_o)[rank], 'y')
    rdos, rparams = oracle.out_backward(all_o, dys)
    same(do, rdos[rank], 'dO')
    same(dwo, rparams[rank][0], 'dW_o')
    # The parity gate bench.py runs in front of its timed region accepts these results ...
    inputs = dict(x=x, grads=grads, o=o, dy=dy)
    weights = dict(w_seg=w_seg, wo=wo, bq=None, bo=None)
    results = dict(outs=outs, dx=dx, dw_seg=per_segment, y=y, do=do, dwo=dwo)
    report, failures = bench.validate_step(torch, dist, rank, world, hidden, heads, inputs, weights, results,
                                           (1e-4, 1e-4), tile=128)
    problems += [f'gate rejected correct results: {f}' for f in failures]
    if len(report) != segments + 1 + 2 * segments + 1 + 1 + 2:
        problems.append(f'gate checked {sorted(report)}')
    # ... and names exactly the tensor that is wrong (a QKV weight gradient whose segments are swapped,
    # an output that belongs to another rank's heads)
    swapped = torch.cat([per_segment[hidden:2 * hidden], per_segment[:hidden], per_segment[2 * hidden:]])
    _, failures = bench.validate_step(torch, dist, rank, world, hidden, heads, inputs, weights,
                                      dict(results, dw_seg=swapped), (1e-4, 1e-4), tile=128)
    if not failures or not all('qkv_bwd dW segment' in f and 'segment 2' not in f for f in failures):
        problems.append(f'swapped weight-gradient segments: {failures}')
    _, failures = bench.validate_step(torch, dist, rank, world, hidden, heads, inputs, weights,
                                      dict(results, y=y.roll(1, 0)), (1e-4, 1e-4), tile=128)
    if [f.split(':')[0] for f in failures] != ['out_fwd y']:
        problems.append(f'shifted y: {failures}')
    # The reference's own unfused modules (staged copy), when present, through the same adapter the
    # benchmark times: same results, and the gate accepts them.
    module = bench.load_reference_modules()
    if module is not None:
        ref = bench.ReferenceUnfused(module, torch, hidden, heads, list(w_seg.split(hidden)), wo, None, None, 'cpu',
                                     torch.float32, False)
        xr, orr = x.clone().requires_grad_(), o.clone().requires_grad_()
        r_outs = ref.qkv_forward(xr)
        r_dx, r_dws = ref.qkv_backward(r_outs, xr, grads)
        r_y = ref.out_forward(orr)
        r_do, r_dwo = ref.out_backward(r_y, orr, dy)
        r_results = dict(outs=r_outs, dx=r_dx, dw_seg=torch.cat(list(r_dws)), y=r_y, do=r_do, dwo=r_dwo)
        _, failures = bench.validate_step(torch, dist, rank, world, hidden, heads, inputs, weights, r_results,
                                          (1e-4, 1e-4), tile=128)
        problems += [f'reference modules: {f}' for f in failures]
        for name in ('dx', 'dw_seg', 'y', 'do', 'dwo'):
            same(r_results[name], results[name], f'reference modules vs restated arm: {name}')
    queue.put((rank, problems))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 4])
def test_comparison_arm_computes_the_same_projections(world):
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, 29720 + world, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, problems in results:
        assert problems == [], f'rank {rank}: {problems}'


def fused_arm_worker(rank, world, port, queue, gate, bias):
    """bench.FusedArm (the adapter between the public modules and the harness) over the simulated
    library: its results, in the form the parity gate takes, must pass the gate at the BF16 bound."""
    here = os.path.dirname(os.path.abspath(__file__))
    for path in (here, ROOT, os.path.join(ROOT, 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.set_num_threads(2)
    import abi_simulator
    import bench
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    problems = []
    try:
        hidden, heads, m, bf = 512, 4, 300, torch.bfloat16
        segments, d = (4 if gate else 3), 128
        g = torch.Generator().manual_seed(1234)
        parameters = dict(w_seg=(torch.randn(segments * hidden, hidden, generator=g) / 64).to(bf),
                          wo=(torch.randn(hidden, hidden, generator=g) / 64).to(bf),
                          bq=(torch.randn(segments * hidden, generator=g) * 0.02).to(bf) if bias else None,
                          bo=(torch.randn(hidden, generator=g) * 0.02).to(bf) if bias else None)
        g = torch.Generator().manual_seed(1235 + rank)
        data = dict(x=torch.randn(m, hidden, generator=g).to(bf),
                    grads=[torch.randn(world * m, heads // world, d, generator=g).to(bf) for _ in range(segments)],
                    o=torch.randn(world * m, heads // world, d, generator=g).to(bf),
                    dy=torch.randn(m, hidden, generator=g).to(bf))
        arm = bench.FusedArm(torch, fused, hidden, heads, m, data, parameters, gate=gate)
        state = {}
        for one_pass in arm.passes:
            one_pass(state)
        report, failures = bench.validate_step(
            torch, dist, rank, world, hidden, heads,
            dict(x=data['x'].detach(), grads=data['grads'], o=data['o'].detach(), dy=data['dy']), parameters,
            arm.results(state), bench.parity_tolerance('bf16', bias))
        problems += failures
        if len(report) != segments + 1 + 2 * segments + 1 + 1 + 2:
            problems.append(f'gate checked {sorted(report)}')
        # the gate is sensitive to the adapter's row order: without the de-interleave it must object
        wrong = dict(arm.results(state), dw_seg=state['dq'][1])
        _, failures = bench.validate_step(
            torch, dist, rank, world, hidden, heads,
            dict(x=data['x'].detach(), grads=data['grads'], o=data['o'].detach(), dy=data['dy']), parameters,
            wrong, bench.parity_tolerance('bf16', bias))
        if not any('qkv_bwd dW' in f for f in failures):
            problems.append('interleaved weight-gradient rows passed as segment-major')
    finally:
        undo()
    queue.put((rank, problems))
    dist.destroy_process_group()


@pytest.mark.parametrize('gate,bias', [(False, False), (True, True)])
def test_fused_arm_adapter_passes_the_parity_gate_on_simulated_ranks(gate, bias):
    world = 2
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=fused_arm_worker, args=(r, world, 29735 + gate, queue, gate, bias)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, problems in results:
        assert problems == [], f'rank {rank}: {problems}'
