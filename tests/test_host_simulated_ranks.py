"""The host layer end to end on CPU ranks (gloo, world size 1, 2 and 4) against the oracle.

libfga.so is replaced by tests/abi_simulator.py: shared-memory "symmetric" buffers, gloo barriers,
torch GEMMs, all following the contract of include/fga.h. Everything above the C ABI is the real
package: workspace construction and handle exchange, slab carving, peer tables, the autograd
functions with their bias, padding, ownership and main_grad handling. Checked per rank: the public
outputs and gradients against the oracle (same tolerance as the GPU tests: max error 1e-2 of the
scale, Frobenius 2e-3), the transport buffers bit for bit including zeroed pad rows, the arrival
counters, and that outputs own their storage.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
BF = torch.bfloat16

CASES = (dict(gate=False, bias=False, bias_in_gemm=False, main_grad=False, precision='bf16'),
         dict(gate=True, bias=True, bias_in_gemm=False, main_grad=False, precision='bf16'),
         dict(gate=False, bias=True, bias_in_gemm=True, main_grad=True, precision='bf16'),
         dict(gate=False, bias=False, bias_in_gemm=False, main_grad=False, precision='mxfp8'),
         dict(gate=True, bias=True, bias_in_gemm=False, main_grad=True, precision='mxfp8'),
         dict(gate=False, bias=True, bias_in_gemm=True, main_grad=False, precision='mxfp8'))


def close(actual, expected, what):
    actual, expected = actual.detach().float(), expected.detach().float()
    assert actual.shape == expected.shape, f'{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}'
    scale = expected.abs().max().clamp_min(1e-6)
    assert (actual - expected).abs().max() <= 1e-2 * scale, f'{what}: max error'
    assert torch.linalg.norm(actual - expected) <= 2e-3 * torch.linalg.norm(expected) + 1e-6, f'{what}: Frobenius'


def same(actual, expected, what):
    """Bit-for-bit equality, with the place of the first difference in the message."""
    assert actual.shape == expected.shape, f'{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}'
    if not torch.equal(actual, expected):
        where = (actual != expected).nonzero()
        raise AssertionError(f'{what}: {len(where)} elements differ, first at {where[0].tolist()} '
                             f'({actual[tuple(where[0])].item()} vs {expected[tuple(where[0])].item()}), '
                             f'last at {where[-1].tolist()}')


def landed(buffer, expected, tokens, capacity, what):
    """A head-side buffer [P*capacity, width] after a push: GEMM results (FP32 sums in another
    order than the oracle's, so BF16 values may differ in the last bit) in the logical rows of every
    source rank, and exactly the oracle's pad rows (zeros, or the bias when the GEMM adds it)."""
    close(buffer, expected, what)
    pad = torch.ones(buffer.shape[0], dtype=torch.bool)
    for source in range(buffer.shape[0] // capacity):
        pad[source * capacity:source * capacity + tokens] = False
    same(buffer[pad], expected[pad], what + ' pad rows')


def everyone(value):
    box = [None] * dist.get_world_size()
    dist.all_gather_object(box, value)
    return box


def run_rank(hidden, heads, capacity_tokens, token_counts, cases=None):
    import abi_simulator
    import fused_gemm_a2a as fused
    import numpy as np
    from oracle import mxfp8_oracle, ulysses_oracle
    from oracle.ulysses_oracle import UlyssesOracle
    p, rank = dist.get_world_size(), dist.get_rank()
    plain_mm = ulysses_oracle._mm

    def mx_mm(a, b, acc_dtype):
        """The oracle's GEMM with both operands quantized to MXFP8 along the reduction axis."""
        return abi_simulator.mx_product(a.to(BF), b.t().to(BF)).to(acc_dtype)

    d = hidden // heads
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    completed = False
    try:
        for case in (CASES if cases is None else cases):
            quantized = case['precision'] == 'mxfp8'
            if quantized and p > 2 and case['gate']:
                continue      # the numpy MXFP8 oracle is slow and every rank evaluates it for all ranks
            ulysses_oracle._mm = mx_mm if quantized else plain_mm      # every GEMM of the oracle follows the precision
            segments = 4 if case['gate'] else 3
            g = torch.Generator().manual_seed(4321)            # parameters: the same on every rank
            wq = (torch.randn(segments * hidden, hidden, generator=g) / 32).to(BF)
            wo = (torch.randn(hidden, hidden, generator=g) / 32).to(BF)
            bq = torch.randn(segments * hidden, generator=g).mul(0.5).to(BF) if case['bias'] else None
            bo = torch.randn(hidden, generator=g).mul(0.5).to(BF) if case['bias'] else None
            params = dict(wq=wq.clone().requires_grad_(), wo=wo.clone().requires_grad_(),
                          bq=None if bq is None else bq.clone().requires_grad_(),
                          bo=None if bo is None else bo.clone().requires_grad_())
            start = {}
            if case['main_grad']:
                for name, param in params.items():
                    if param is not None:
                        start[name] = torch.randn(param.shape, generator=g)
                        param.main_grad = start[name].clone()
            ws = fused.FusedGemmA2AWorkspace(hidden, heads, capacity_tokens, gate=case['gate'],
                                             precision=case['precision'])
            qkv = fused.FusedQKVProjection(hidden, heads, weight=params['wq'], bias=params['bq'], gate=case['gate'],
                                           bias_in_gemm=case['bias_in_gemm'])
            proj = fused.FusedOutputProjection(hidden, heads, weight=params['wo'], bias=params['bo'])
            oracle = UlyssesOracle(p, hidden, heads, segments, wq, bq, wo, bo, bias_in_gemm=case['bias_in_gemm'])
            accumulated = {name: torch.zeros_like(t) for name, t in start.items()}
            # the numpy MXFP8 oracle is the slow side: one rank alone runs every length, several ranks one
            for tokens in (token_counts[1:2] if quantized and p > 1 else token_counts):
                g = torch.Generator().manual_seed(1000 * tokens + rank)
                x = torch.randn(tokens, hidden, generator=g).to(BF).requires_grad_()
                grads = [torch.randn(p * tokens, heads // p, d, generator=g).to(BF) for _ in range(segments)]
                o = torch.randn(p * tokens, heads // p, d, generator=g).to(BF).requires_grad_()
                dy = torch.randn(tokens, hidden, generator=g).to(BF)
                outs = qkv(x, ws)
                view = ws._view(tokens, segments)
                cap = view.capacity
                xs = everyone(x.detach())
                # head-side buffers right after the push: every rank's tile landed where the oracle puts it
                for seg, want in enumerate(oracle.qkv_heads_buffers(xs, cap)[rank]):
                    landed(view.heads[seg], want, tokens, cap, f'head buffer {seg}')
                got = torch.autograd.grad(outs, [x, params['wq']] + ([params['bq']] if case['bias'] else []), grads)
                all_grads = everyone(tuple(grads))
                same(view.recv, oracle.qkv_recv_buffer(all_grads, rank, cap), 'QKV dgrad transport')
                arrivals = p * segments * fused._Comm.push_split(view.recv, segments, p)
                assert view.counters.tolist() == [arrivals + (16 if quantized else 0)] * (cap // 128)
                if quantized:     # the receive-side quantizer's copy is the standalone quantizer's output
                    payload, scales = mxfp8_oracle.quantize(abi_simulator.bf16_bits(view.recv), k_multiple=128)
                    assert np.array_equal(view.mx_recv.view(torch.uint8).numpy(), payload[:cap])
                    assert np.array_equal(view.mx_scale.numpy(), scales[:view.mx_scale.numel()])
                for name, t, want in zip('qkvg', outs, oracle.qkv_forward(xs)[rank]):
                    close(t, want, f'{name} tokens={tokens}')
                    assert t.shape == (p * tokens, heads // p, d)
                    assert t.untyped_storage().data_ptr() not in {h.untyped_storage().data_ptr() for h in view.heads}
                rdx, rdw, rdb = oracle.qkv_backward(xs, all_grads)[rank]
                close(got[0], rdx, 'dx')
                y = proj(o, ws)
                all_o = everyone(o.detach())
                out_view = ws._view(tokens, 1)
                same(out_view.recv, oracle.out_recv_buffer(all_o, rank, cap), 'output transport')
                close(y, oracle.out_forward(all_o)[rank], 'y')
                got_out = torch.autograd.grad(y, [o, params['wo']] + ([params['bo']] if case['bias'] else []), dy)
                dys = everyone(dy)
                landed(out_view.heads[0], oracle.out_dhead_buffers(dys, cap)[rank], tokens, cap, 'dO head buffer')
                rdos, rparams = oracle.out_backward(all_o, dys)
                close(got_out[0], rdos[rank], 'dO')
                if case['main_grad']:
                    accumulated['wq'] += rdw
                    accumulated['wo'] += rparams[rank][0]
                    accumulated['bq'] += rdb
                    accumulated['bo'] += rparams[rank][1]
                    assert params['wq'].grad_added_to_main_grad and params['wo'].grad_added_to_main_grad
                    assert got[1].shape == wq.shape and got_out[1].shape == wo.shape     # placeholders
                else:
                    close(got[1], rdw, 'dW_qkv')
                    close(got_out[1], rparams[rank][0], 'dW_o')
                    if case['bias']:
                        close(got[2], rdb, 'dbias_qkv')
                        close(got_out[2], rparams[rank][1], 'dbias_o')
            for name, total in accumulated.items():
                close(params[name].main_grad - start[name], total, f'main_grad of {name}')
        completed = True
        return sim.launches
    finally:
        ulysses_oracle._mm = plain_mm
        undo(meet=completed)     # after a failure the peers are not at the same point: do not wait for them


def worker(rank, world, port, queue, geometry=None):
    for path in (HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.set_num_threads(2)
    try:
        if geometry is None:
            launches = run_rank(hidden=512, heads=4, capacity_tokens=300, token_counts=(300, 129, 1))
        else:
            hidden, heads, cases = geometry
            launches = run_rank(hidden=hidden, heads=heads, capacity_tokens=300, token_counts=(129,),
                                cases=[CASES[index] for index in cases])
        queue.put((rank, 'ok', launches))
    except BaseException as error:   # report and leave at once; the parent stops the peers
        import traceback
        queue.put((rank, 'fail', f'{type(error).__name__}: {error}\n{traceback.format_exc()[-2500:]}'))
        queue.close()
        queue.join_thread()
        os._exit(1)
    dist.destroy_process_group()


@pytest.mark.parametrize('world', [1, 2, 4])
def test_modules_on_simulated_ranks_match_the_oracle(world):
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, 29660 + world, queue)) for r in range(world)]
    for proc in procs:
        proc.start()
    results = []
    try:
        for _ in range(world):
            results.append(queue.get(timeout=600))
            assert results[-1][1] == 'ok', f'rank {results[-1][0]}: {results[-1][2]}'
    finally:
        for proc in procs:
            proc.join(timeout=5 if results and results[-1][1] != 'ok' else 120)
            if proc.is_alive():
                proc.terminate()
    for rank, verdict, detail in sorted(results):
        # at least 3 BF16 cases x 3 token counts x (6 barriers + 4 GEMMs + 2 weight gradients + 2 row copies)
        # plus the MXFP8 cases
        assert detail > 3 * 3 * 14


@pytest.mark.parametrize('hidden,heads,cases', [(768, 6, (1, 2)), (1280, 10, (0, 3))])
def test_three_and_five_heads_per_rank_on_two_simulated_ranks(hidden, heads, cases):
    """The heads-per-rank counts of the benchmark configurations with 24 and 40 heads at CP = 8
    (three and five): an odd number of 128-wide head units per rank, so push tiles and pusher chunks
    do not pair up evenly. BF16 with gate and bias (early and late) for three, BF16 and MXFP8 for five."""
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, 2, 29664 + heads, queue, (hidden, heads, cases))) for r in range(2)]
    for proc in procs:
        proc.start()
    results = []
    try:
        for _ in range(2):
            results.append(queue.get(timeout=600))
            assert results[-1][1] == 'ok', f'rank {results[-1][0]}: {results[-1][2]}'
    finally:
        for proc in procs:
            proc.join(timeout=5 if results and results[-1][1] != 'ok' else 120)
            if proc.is_alive():
                proc.terminate()


def mismatch_worker(rank, world, port, queue):
    for path in (HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import abi_simulator
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    verdict = 'no error'
    try:
        fused.CHECK_TOKENS = True
        ws = fused.FusedGemmA2AWorkspace(512, 4, 300)
        qkv = fused.FusedQKVProjection(512, 4, weight=torch.zeros(1536, 512, dtype=BF))
        proj = fused.FusedOutputProjection(512, 4, weight=torch.zeros(512, 512, dtype=BF))
        before = sim.launches
        for module, tensor in ((qkv, torch.zeros(129 + rank, 512, dtype=BF)),
                               (proj, torch.zeros(world * (129 + rank), 4 // world, 128, dtype=BF))):
            try:
                module(tensor, ws)
            except ValueError as error:
                verdict = str(error)
            else:
                verdict = 'no error'
                break
        if sim.launches != before:
            verdict = 'kernels were launched'
        qkv(torch.zeros(200, 512, dtype=BF), ws)          # equal counts pass, and the ranks are still in step
    finally:
        fused.CHECK_TOKENS = False
        undo()
    queue.put((rank, verdict))
    dist.destroy_process_group()


def test_unequal_token_counts_are_caught_on_the_host_when_asked():
    """FGA_CHECK_TOKENS: two ranks calling with 129 and 130 tokens both get the same ValueError from
    either projection before anything is launched, and go on together afterwards."""
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=mismatch_worker, args=(r, 2, 29669, queue)) for r in range(2)]
    for proc in procs:
        proc.start()
    results = sorted(queue.get(timeout=300) for _ in range(2))
    for proc in procs:
        proc.join(timeout=60)
    for rank, verdict in results:
        assert 'same number of local tokens' in verdict and '129 to 130' in verdict, (rank, verdict)


def vmm_worker(rank, world, port, queue):
    for path in (HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.set_num_threads(2)
    import fused_gemm_a2a as fused
    open_before = len(os.listdir('/proc/self/fd'))
    fused.SYMM_BACKEND = 'vmm'
    try:
        launches = run_rank(hidden=512, heads=4, capacity_tokens=300, token_counts=(129,), cases=CASES[1:3])
        leaked = len(os.listdir('/proc/self/fd')) - open_before
        queue.put((rank, 'ok' if launches > 0 else 'nothing ran', leaked))
    except BaseException as error:
        import traceback
        queue.put((rank, f'{type(error).__name__}: {error}\n{traceback.format_exc()[-2000:]}', 0))
        queue.close()
        queue.join_thread()
        os._exit(1)
    finally:
        fused.SYMM_BACKEND = 'ipc'
    dist.destroy_process_group()


def test_descriptor_backed_buffers_carry_the_same_protocol(world=2):
    """FGA_SYMM=vmm on CPU ranks: every allocation's file descriptor really travels to the peers over
    Unix-domain sockets, each side maps it, and the projections match the oracle through those
    mappings. No descriptor is left open afterwards (each rank closes its own and the received ones)."""
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=vmm_worker, args=(r, world, 29675 + world, queue)) for r in range(world)]
    for proc in procs:
        proc.start()
    results = []
    try:
        for _ in range(world):
            results.append(queue.get(timeout=600))
            assert results[-1][1] == 'ok', f'rank {results[-1][0]}: {results[-1][1]}'
    finally:
        for proc in procs:
            proc.join(timeout=5 if results and results[-1][1] != 'ok' else 120)
            if proc.is_alive():
                proc.terminate()
    for rank, _, leaked in results:
        assert leaked <= 0, f'rank {rank} left {leaked} descriptors open'


def release_worker(rank, world, port, queue, backend):
    for path in (HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import abi_simulator
    import fused_gemm_a2a as fused
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    fused.SYMM_BACKEND = backend
    try:
        ws = fused.FusedGemmA2AWorkspace(512, 4, 300)
        comm = ws.comm
        allocations = list(comm._allocations)
        comm.release()
        again = fused.FusedGemmA2AWorkspace(512, 4, 300)          # a fresh runtime, fresh buffers
        report = dict(allocations=len(allocations), released=list(sim.released),
                      expected=[(kind, local, seen, mapped) for kind, local, seen, mapped in allocations],
                      fresh=again.comm is not comm and len(again.comm._allocations) == len(allocations),
                      emptied=not comm._allocations and not comm.projection_buffers)
        queue.put((rank, report))
    finally:
        fused.SYMM_BACKEND = 'ipc'
        undo()
    dist.destroy_process_group()


@pytest.mark.parametrize('backend', ['ipc', 'vmm'])
def test_release_unmaps_every_peer_and_frees_every_buffer_once(backend):
    world = 2
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=release_worker, args=(r, world, 29730 + len(backend), queue, backend)) for r in range(world)]
    for proc in procs:
        proc.start()
    results = sorted(queue.get(timeout=300) for _ in range(world))
    for proc in procs:
        proc.join(timeout=60)
        assert proc.exitcode == 0
    for rank, report in results:
        assert report['allocations'] == 3 and report['fresh'] and report['emptied']      # flags + two buffer sets
        wanted = []
        for kind, local, seen, mapped in report['expected']:
            assert kind == backend
            for owner, address in enumerate(seen):
                if owner != rank:
                    wanted.append(('release', address, mapped) if backend == 'vmm' else ('close', address))
            wanted.append(('release', local, mapped) if backend == 'vmm' else ('free', local))
        assert report['released'] == wanted


def pipeline_worker(rank, world, port, queue):
    """Four ranks = two pipeline stages of CP 2 (reference tests/pipeline_setup_driver.py:26-77 with
    --prepare): every stage creates its workspace on its own CP subgroup first; then stage 0 posts
    the receive of the token that stage 1 sends back only after its own receive has completed."""
    for path in (HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    import datetime
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    torch.set_num_threads(1)
    import abi_simulator
    import fused_gemm_a2a as fused
    from oracle.ulysses_oracle import UlyssesOracle
    stage_size = world // 2
    cp_groups = [dist.new_group(list(range(stage_size))), dist.new_group(list(range(stage_size, world)))]
    pp_forward = [dist.new_group([i, i + stage_size]) for i in range(stage_size)]
    pp_return = [dist.new_group([i, i + stage_size]) for i in range(stage_size)]
    stage = rank // stage_size
    cp = cp_groups[stage]
    recv_group = pp_return[rank % stage_size] if stage == 0 else pp_forward[rank % stage_size]
    send_group = pp_forward[rank % stage_size] if stage == 0 else pp_return[rank % stage_size]
    peer = (rank + stage_size) % world
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    problems = []
    try:
        hidden, heads, tokens = 256 * stage_size, 2 * stage_size, 100
        g = torch.Generator().manual_seed(9 + stage)
        weight = (torch.randn(4 * hidden, hidden, generator=g) / hidden ** 0.5).to(BF)
        qkv = fused.FusedQKVProjection(hidden, heads, gate=True, weight=weight)
        workspace = fused.FusedGemmA2AWorkspace(hidden, heads, 128, cp_group=cp, gate=True)      # --prepare
        if workspace.comm.p != stage_size or workspace.comm.rank != rank % stage_size:
            problems.append(f'runtime of the subgroup has p={workspace.comm.p} rank={workspace.comm.rank}')
        signal, received = torch.tensor([rank + 1.0]), torch.zeros(1)
        pending = dist.irecv(received, src=peer, group=recv_group)
        if stage == 1:
            pending.wait()
        again = fused.FusedGemmA2AWorkspace(hidden, heads, 128, cp_group=cp, gate=True)          # no communication
        if again.comm is not workspace.comm or again._buffers[4] is not workspace._buffers[4]:
            problems.append('a second handle of the same geometry built new buffers')
        dist.isend(signal, dst=peer, group=send_group).wait()
        if stage == 0:
            pending.wait()
        if received.item() != peer + 1.0:
            problems.append(f'pipeline token {received.item()}')
        # and the projection runs on the subgroup: this stage's two ranks against a two-rank oracle
        x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(100 + rank)).to(BF)
        outs = qkv(x, workspace)
        xs = [None] * stage_size
        dist.all_gather_object(xs, x, group=cp)
        oracle = UlyssesOracle(stage_size, hidden, heads, 4, weight)
        for name, got, want in zip('qkvg', outs, oracle.qkv_forward(xs)[rank % stage_size]):
            try:
                close(got, want, name)
            except AssertionError as error:
                problems.append(str(error))
        queue.put((rank, problems))
    finally:
        undo()
    dist.destroy_process_group()


def test_workspaces_on_cp_subgroups_before_posted_pipeline_receives():
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=pipeline_worker, args=(r, 4, 29683, queue)) for r in range(4)]
    for proc in procs:
        proc.start()
    try:
        results = sorted(queue.get(timeout=300) for _ in range(4))
    finally:
        for proc in procs:
            proc.join(timeout=120)
            if proc.is_alive():
                proc.terminate()
    for rank, problems in results:
        assert problems == [], f'rank {rank}: {problems}'


def grouped_query_worker(rank, world, port, queue, heads, kv_heads, gate, bias, bias_in_gemm, precision='bf16'):
    """The public modules with fewer key/value heads than query heads, on simulated ranks, against the
    grouped-query oracle (itself pinned by the reference's unfused modules with num_kv_heads <
    num_heads): outputs of different widths per kind, transport buffers bit for bit, dX, parameter
    gradients in the grouped row order, and the output projection of the same workspace."""
    for path in (HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), 'fused-gemm-a2a_b200')):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.set_num_threads(2)
    import abi_simulator
    import fused_gemm_a2a as fused
    from oracle import mxfp8_oracle, ulysses_oracle
    from oracle.ulysses_oracle import GroupedQueryOracle
    quantized = precision == 'mxfp8'
    if quantized:       # every GEMM of the oracle with both operands quantized along the reduction axis
        ulysses_oracle._mm = lambda a, b, acc_dtype: abi_simulator.mx_product(a.to(BF), b.t().to(BF)).to(acc_dtype)
    p, d = world, 128
    hidden = heads * d
    r = heads // kv_heads
    rows = (heads * (2 if gate else 1) + 2 * kv_heads) * d
    kinds = 4 if gate else 3
    sim, undo = abi_simulator.install(fused, abi_simulator.unique_tag())
    problems = []
    completed = False
    try:
        g = torch.Generator().manual_seed(77)
        wq = (torch.randn(rows, hidden, generator=g) / 32).to(BF)
        wo = (torch.randn(hidden, hidden, generator=g) / 32).to(BF)
        bq = torch.randn(rows, generator=g).mul(0.5).to(BF) if bias else None
        wq_p, wo_p = wq.clone().requires_grad_(), wo.clone().requires_grad_()
        bq_p = bq.clone().requires_grad_() if bias else None
        ws = fused.FusedGemmA2AWorkspace(hidden, heads, 300, gate=gate, num_kv_heads=kv_heads, precision=precision)
        qkv = fused.FusedQKVProjection(hidden, heads, kv_heads, weight=wq_p, bias=bq_p, gate=gate,
                                       bias_in_gemm=bias_in_gemm)
        proj = fused.FusedOutputProjection(hidden, heads, weight=wo_p)
        oracle = GroupedQueryOracle(p, hidden, heads, kv_heads, gate, weight_qkv=wq, bias_qkv=bq, weight_out=wo,
                                    bias_in_gemm=bias_in_gemm)
        widths = [heads // p if kind in (0, 3) else kv_heads // p for kind in range(kinds)]
        for tokens in ((129,) if quantized else (129, 300)):      # the numpy MXFP8 oracle is the slow side
            g = torch.Generator().manual_seed(1000 * tokens + rank)
            x = torch.randn(tokens, hidden, generator=g).to(BF).requires_grad_()
            grads = [torch.randn(p * tokens, width, d, generator=g).to(BF) for width in widths]
            o = torch.randn(p * tokens, heads // p, d, generator=g).to(BF).requires_grad_()
            dy = torch.randn(tokens, hidden, generator=g).to(BF)
            outs = qkv(x, ws)
            view = ws._view(tokens, kinds)
            xs = everyone(x.detach())
            for kind, want in enumerate(oracle.qkv_heads_buffers(xs, view.capacity)[rank]):
                landed(view.heads[kind], want, tokens, view.capacity, f'head buffer {kind} tokens={tokens}')
            for name, got, want in zip('qkvg', outs, oracle.qkv_forward(xs)[rank]):
                assert got.shape == want.shape, f'{name}: {tuple(got.shape)} vs {tuple(want.shape)}'
                close(got, want, f'{name} tokens={tokens}')
                assert got.data_ptr() not in {t.data_ptr() for t in view.heads}
            got = torch.autograd.grad(outs, [x, wq_p] + ([bq_p] if bias else []), grads)
            all_grads = everyone(tuple(grads))
            same(view.recv, oracle.qkv_recv_buffer(all_grads, rank, view.capacity), f'dY transport tokens={tokens}')
            arrivals = p * kinds * fused.push_split(kinds * hidden, p, kinds)
            assert view.counters.tolist() == [arrivals + (16 if quantized else 0)] * (view.capacity // 128)
            if quantized:     # the receive-side quantizer's copy is the standalone quantizer's output
                payload, scales = mxfp8_oracle.quantize(abi_simulator.bf16_bits(view.recv), k_multiple=128)
                assert torch.equal(view.mx_recv.view(torch.uint8), torch.from_numpy(payload[:view.capacity]))
                assert torch.equal(view.mx_scale, torch.from_numpy(scales[:view.mx_scale.numel()]))
            rdx, rdw, rdb = oracle.qkv_backward(xs, all_grads)[rank]
            close(got[0], rdx, 'dx')
            close(got[1], rdw, 'dW_qkv (grouped row order)')
            if bias:
                close(got[2], rdb, 'dbias_qkv')
            y = proj(o, ws)
            close(y, oracle.out_forward(everyone(o.detach()))[rank], 'y')
            do, dwo = torch.autograd.grad(y, [o, wo_p], dy)
            rdos, rparams = oracle.out_backward(everyone(o.detach()), everyone(dy))
            close(do, rdos[rank], 'dO')
            close(dwo, rparams[rank][0], 'dW_o')
        completed = True
    except AssertionError as error:
        problems.append(str(error))
    finally:
        undo(meet=completed)
    queue.put((rank, problems))
    if completed:
        dist.destroy_process_group()
    else:
        os._exit(1)


@pytest.mark.parametrize('world,heads,kv_heads,gate,bias,bias_in_gemm,precision', [
    (1, 4, 2, False, False, False, 'bf16'), (2, 8, 2, True, True, False, 'bf16'), (2, 4, 2, False, True, True, 'bf16'),
    (2, 6, 2, False, False, False, 'bf16'), (2, 4, 2, True, True, False, 'mxfp8')])
def test_grouped_query_modules_on_simulated_ranks(world, heads, kv_heads, gate, bias, bias_in_gemm, precision):
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    port = 29640 + heads + world + (20 if precision == 'mxfp8' else 0)
    procs = [ctx.Process(target=grouped_query_worker,
                         args=(r, world, port, queue, heads, kv_heads, gate, bias, bias_in_gemm, precision))
             for r in range(world)]
    for proc in procs:
        proc.start()
    results = []
    try:
        for _ in range(world):
            results.append(queue.get(timeout=600))
    finally:
        for proc in procs:
            proc.join(timeout=30)
            if proc.is_alive():
                proc.terminate()
    for rank, problems in sorted(results):
        assert problems == [], f'rank {rank}: {problems}'
