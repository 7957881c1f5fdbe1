"""Multi-GPU parity driver (one process per GPU, launched by torch.distributed.run).

Every rank runs the public modules on its own GPU; inputs of all ranks are gathered so that each
rank can evaluate the CPU oracle for the whole CP group and compare its own outputs, gradients and
the raw transport buffers. Exits non-zero on any mismatch or device-side timeout.

Ranks leave together. A rank that exits frees the buffers its peers write into, and a peer that
went on to its next launch would then store into unmapped memory. So a failed comparison is
recorded, not raised; after every case the ranks agree (one all-reduce) whether anybody failed and,
if so, all stop at that point with nothing in flight. An unexpected exception keeps the process,
and with it its buffers, alive until the peers' bounded waits have run out.
"""
import contextlib
import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
for path in (ROOT, os.path.join(ROOT, 'fused-gemm-a2a_b200')):
    if path not in sys.path:
        sys.path.insert(0, path)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import fused_gemm_a2a  # noqa: E402
from fused_gemm_a2a import FusedGemmA2AWorkspace, FusedOutputProjection, FusedQKVProjection  # noqa: E402
from oracle.ulysses_oracle import UlyssesOracle  # noqa: E402

BF = torch.bfloat16


def close(actual, expected, what):
    actual, expected = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert actual.shape == expected.shape, f'{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}'
    scale = expected.abs().max().clamp_min(1e-6)
    assert (actual - expected).abs().max() <= 1e-2 * scale, f'{what}: max error'
    assert torch.linalg.norm(actual - expected) <= 2e-3 * torch.linalg.norm(expected) + 1e-6, f'{what}: Frobenius'


class Agreement:
    """Soft assertions with a collective verdict."""

    def __init__(self, dev):
        self.dev, self.failures = dev, []

    @contextlib.contextmanager
    def checks(self, label):
        try:
            yield
        except AssertionError as error:
            self.failures.append(f'{label}: {error}')

    def settle(self, label):
        """All ranks learn whether any rank failed; if so, all of them stop here."""
        flag = torch.tensor([len(self.failures)], dtype=torch.int32, device=self.dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if flag.item() == 0:
            return
        for failure in self.failures:
            print(f'[rank {dist.get_rank()}] FAIL {failure}', flush=True)
        fused_gemm_a2a.release_all()       # collective: drain, meet, unmap the peers, free
        dist.destroy_process_group()
        sys.exit(1)


def gather(t):
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, t.contiguous())
    return [p.cpu() for p in parts]


def main():
    local = int(os.environ['LOCAL_RANK'])
    # FGA_DRIVER_SIMULATED=1 (the CPU test-suite): the same checks on gloo ranks with tests/abi_simulator.py
    # in place of libfga.so, so that the driver itself - its geometries, gathers and expected values -
    # has run before it meets a GPU. The CUDA-graph section needs a GPU and is skipped there.
    simulated = os.environ.get('FGA_DRIVER_SIMULATED') == '1'
    if simulated:
        sys.path.insert(0, os.path.join(ROOT, 'tests'))
        import abi_simulator
        dev = torch.device('cpu')
        dist.init_process_group('gloo')
        torch.set_num_threads(2)
        _, leave_simulation = abi_simulator.install(fused_gemm_a2a, abi_simulator.unique_tag())
        device_sync = lambda: None      # noqa: E731
    else:
        torch.cuda.set_device(local)
        dev = torch.device('cuda', local)
        dist.init_process_group('nccl', device_id=dev)
        device_sync = torch.cuda.synchronize
    fused_gemm_a2a.install_exit_guards()   # SIGTERM from the launcher: finish queued GPU work first
    rank, p = dist.get_rank(), dist.get_world_size()
    checks = 0
    verdict = Agreement(dev)
    every_length = (129, 1) if simulated else (300, 129, 1, 512, 255)
    configurations = [(1024, 8, False, False, False, every_length), (1024, 8, True, True, False, every_length),
                      (1024, 8, False, True, True, every_length),
                      # the benchmark configurations' geometries (at CP = 8: 4 and 3 heads per rank), one length each
                      (4096, 32, False, False, False, (129,)), (3072, 24, True, True, True, (77,))]
    for hidden, heads, gate, with_bias, bias_in_gemm, lengths in configurations:
        d = hidden // heads
        segments = 4 if gate else 3
        g = torch.Generator().manual_seed(4321)  # replicated parameters
        wq = (torch.randn(segments * hidden, hidden, generator=g) / 32).to(BF)
        wo = (torch.randn(hidden, hidden, generator=g) / 32).to(BF)
        bq = torch.randn(segments * hidden, generator=g).mul(0.5).to(BF) if with_bias else None
        bo = torch.randn(hidden, generator=g).mul(0.5).to(BF) if with_bias else None
        ws = FusedGemmA2AWorkspace(hidden, heads, 600, gate=gate)
        wq_d, wo_d = wq.to(dev).requires_grad_(), wo.to(dev).requires_grad_()
        bq_d = bq.to(dev).requires_grad_() if with_bias else None
        bo_d = bo.to(dev).requires_grad_() if with_bias else None
        qkv = FusedQKVProjection(hidden, heads, weight=wq_d, bias=bq_d, gate=gate, bias_in_gemm=bias_in_gemm)
        proj = FusedOutputProjection(hidden, heads, weight=wo_d, bias=bo_d)
        oracle = UlyssesOracle(p, hidden, heads, segments, wq, bq, wo, bo, bias_in_gemm=bias_in_gemm)
        for tokens in lengths:
            g = torch.Generator().manual_seed(1000 * tokens + rank)
            x = torch.randn(tokens, hidden, generator=g).to(BF).to(dev).requires_grad_()
            grads = [torch.randn(p * tokens, heads // p, d, generator=g).to(BF).to(dev) for _ in range(segments)]
            o = torch.randn(p * tokens, heads // p, d, generator=g).to(BF).to(dev).requires_grad_()
            dy = torch.randn(tokens, hidden, generator=g).to(BF).to(dev)
            outs = qkv(x, ws)
            dx, dwq, *dbq = torch.autograd.grad(outs, [x, wq_d] + ([bq_d] if with_bias else []), grads)
            y = proj(o, ws)
            do, dwo, *dbo = torch.autograd.grad(y, [o, wo_d] + ([bo_d] if with_bias else []), dy)
            device_sync()
            all_grads = list(zip(*[gather(t) for t in grads]))       # [rank][segment]
            all_o = gather(o.detach())
            xs, dys = gather(x.detach()), gather(dy)
            label = f'hidden={hidden} gate={gate} bias={with_bias} bias_in_gemm={bias_in_gemm} tokens={tokens}'
            with verdict.checks(label):
                assert ws.comm.status.tolist()[0] == 0, f'device status {ws.comm.status.tolist()}'
                # exact transport: the QKV receive buffer still holds this rank's dY, the output
                # receive buffer this rank's sequence-side O, pad rows zero
                cap = ws._view(tokens, segments).capacity
                want_dy = oracle.qkv_recv_buffer(all_grads, rank, cap)
                assert torch.equal(ws._view(tokens, segments).recv.cpu(), want_dy), 'QKV dgrad transport'
                assert torch.equal(ws._view(tokens, 1).recv.cpu(),
                                   oracle.out_recv_buffer(all_o, rank, cap)), 'output transport'
                want_outs = oracle.qkv_forward(xs)[rank]
                for name, got, want in zip('qkvg', outs, want_outs):
                    close(got, want, f'{name} tokens={tokens}')
                rdx, rdw, rdb = oracle.qkv_backward(xs, all_grads)[rank]
                close(dx, rdx, 'dx')
                close(dwq, rdw, 'dW_qkv')
                close(y, oracle.out_forward(all_o)[rank], 'y')
                rdos, rparams = oracle.out_backward(all_o, dys)
                close(do, rdos[rank], 'dO')
                close(dwo, rparams[rank][0], 'dW_o')
                if with_bias:
                    close(dbq[0], rdb, 'dbias_qkv')
                    close(dbo[0], rparams[rank][1], 'dbias_o')
            verdict.settle(label)
            checks += 1
        if rank == 0:
            print(f'PASS hidden={hidden} heads={heads} gate={gate} bias={with_bias} bias_in_gemm={bias_in_gemm}',
                  flush=True)

    # MXFP8: only BF16 crosses the links; expected values quantize every GEMM's operands along its
    # reduction axis on the CPU (E4M3 + E8M0/32) and multiply the exact dequantized values
    import numpy as np
    from oracle import mxfp8_oracle as mx

    def bits(t):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    def mm(a, b):
        return torch.from_numpy(mx.mx_matmul(bits(a), bits(b))).to(BF)

    # (hidden 5120 with 40 heads is the MXFP8 benchmark configuration: 5 heads per rank at CP = 8)
    # (simulated: 10 heads keep five heads per rank on two ranks; the float64 numpy products are the slow side)
    mx_geometries = ((1024, 8, (129,)), (1280, 10, (129,))) if simulated else ((1024, 8, (300, 129)), (5120, 40, (129,)))
    for hidden, heads, lengths in mx_geometries:
        d, hpr = hidden // heads, heads // p
        g = torch.Generator().manual_seed(99)
        wq = (torch.randn(3 * hidden, hidden, generator=g) / 32).to(BF)
        wo = (torch.randn(hidden, hidden, generator=g) / 32).to(BF)
        ws = FusedGemmA2AWorkspace(hidden, heads, 600, precision='mxfp8')
        wq_d, wo_d = wq.to(dev).requires_grad_(), wo.to(dev).requires_grad_()
        qkv = FusedQKVProjection(hidden, heads, weight=wq_d)
        proj = FusedOutputProjection(hidden, heads, weight=wo_d)
        for tokens in lengths:
            g = torch.Generator().manual_seed(555 * tokens + rank)
            x = torch.randn(tokens, hidden, generator=g).to(BF).to(dev).requires_grad_()
            grads = [torch.randn(p * tokens, hpr, d, generator=g).to(BF).to(dev) for _ in range(3)]
            o = torch.randn(p * tokens, hpr, d, generator=g).to(BF).to(dev).requires_grad_()
            dy = torch.randn(tokens, hidden, generator=g).to(BF).to(dev)
            outs = qkv(x, ws)
            dx, dwq = torch.autograd.grad(outs, [x, wq_d], grads)
            y = proj(o, ws)
            do, dwo = torch.autograd.grad(y, [o, wo_d], dy)
            device_sync()
            xs, dys, all_o = gather(x.detach()), gather(dy), gather(o.detach())
            all_grads = list(zip(*[gather(t) for t in grads]))
            label = f'mxfp8 hidden={hidden} tokens={tokens}'
            with verdict.checks(label):
                assert ws.comm.status.tolist()[0] == 0, f'device status {ws.comm.status.tolist()}'
                plain = UlyssesOracle(p, hidden, heads, 3)
                # rows quantize independently: all ranks' tokens go through one product per weight
                projected = mm(torch.cat(xs), wq).view(p * tokens, heads, 3, d)
                for seg in range(3):
                    close(outs[seg], projected[:, rank * hpr:(rank + 1) * hpr, seg], f'mxfp8 segment {seg}')
                dyq = plain.qkv_recv_buffer(all_grads, rank)
                close(dx, mm(dyq, wq.t()), 'mxfp8 dx')
                close(dwq, mm(dyq.t(), xs[rank].t()), 'mxfp8 dW_qkv')
                o_seq = plain.out_recv_buffer(all_o, rank)
                close(y, mm(o_seq, wo), 'mxfp8 y')
                full_do = mm(torch.cat(dys), wo.t())[:, rank * hpr * d:(rank + 1) * hpr * d]
                close(do, full_do.reshape(p * tokens, hpr, d), 'mxfp8 dO')
                close(dwo, mm(dys[rank].t(), o_seq.t()), 'mxfp8 dW_o')
            verdict.settle(label)
    if rank == 0:
        print('PASS mxfp8', flush=True)

    if simulated:
        if rank == 0:
            print(f'PASS simulated; {checks} eager configurations checked on {p} CPU ranks', flush=True)
        leave_simulation()
        dist.destroy_process_group()
        return

    # CUDA graph: one captured step replayed with changed inputs
    hidden, heads, tokens, segments = 1024, 8, 333, 3
    d = hidden // heads
    ws = FusedGemmA2AWorkspace(hidden, heads, 600)
    sx = torch.zeros(tokens, hidden, dtype=BF, device=dev).requires_grad_()
    so = torch.zeros(p * tokens, heads // p, d, dtype=BF, device=dev).requires_grad_()
    sg = [torch.zeros(p * tokens, heads // p, d, dtype=BF, device=dev) for _ in range(3)]
    sdy = torch.zeros(tokens, hidden, dtype=BF, device=dev)
    g = torch.Generator().manual_seed(4321)
    wq = (torch.randn(3 * hidden, hidden, generator=g) / 32).to(BF)
    wo = (torch.randn(hidden, hidden, generator=g) / 32).to(BF)
    wq_d, wo_d = wq.to(dev).requires_grad_(), wo.to(dev).requires_grad_()
    qkv = FusedQKVProjection(hidden, heads, weight=wq_d)
    proj = FusedOutputProjection(hidden, heads, weight=wo_d)
    oracle = UlyssesOracle(p, hidden, heads, 3, wq, None, wo, None)

    def step():
        qs = qkv(sx, ws)
        dx, dw = torch.autograd.grad(qs, [sx, wq_d], sg)
        y = proj(so, ws)
        do, dwo = torch.autograd.grad(y, [so, wo_d], sdy)
        return (*qs, dx, dw, y, do, dwo)

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        step()
    stream.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        outputs = step()
    torch.cuda.current_stream().wait_stream(stream)
    dist.barrier()
    for replay in range(3):
        g = torch.Generator().manual_seed(77 * replay + rank)
        with torch.no_grad():
            sx.copy_(torch.randn(sx.shape, generator=g).to(BF))
            so.copy_(torch.randn(so.shape, generator=g).to(BF))
            sdy.copy_(torch.randn(sdy.shape, generator=g).to(BF))
            for t in sg:
                t.copy_(torch.randn(t.shape, generator=g).to(BF))
        torch.cuda.synchronize()
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        xs, all_o, dys = gather(sx.detach()), gather(so.detach()), gather(sdy)
        all_grads = list(zip(*[gather(t) for t in sg]))
        with verdict.checks(f'graph replay {replay}'):
            assert ws.comm.status.tolist()[0] == 0, f'device status {ws.comm.status.tolist()}'
            q, k, v, dx, dw, y, do, dwo = outputs
            for got, want in zip((q, k, v), oracle.qkv_forward(xs)[rank]):
                close(got, want, f'replay {replay} qkv')
            rdx, rdw, _ = oracle.qkv_backward(xs, all_grads)[rank]
            close(dx, rdx, 'replay dx')
            close(dw, rdw, 'replay dW_qkv')
            close(y, oracle.out_forward(all_o)[rank], 'replay y')
            rdos, rparams = oracle.out_backward(all_o, dys)
            close(do, rdos[rank], 'replay dO')
            close(dwo, rparams[rank][0], 'replay dW_o')
        verdict.settle(f'graph replay {replay}')
    if rank == 0:
        print(f'PASS cuda graph replay; {checks} eager configurations checked on {p} GPUs', flush=True)
    fused_gemm_a2a.release_all()           # collective: drain, meet, unmap the peers, free
    dist.destroy_process_group()


if __name__ == '__main__':
    try:
        main()
    except SystemExit:
        raise
    except BaseException:
        # Not a comparison failure: this rank cannot tell where its peers are. Its kernels finish,
        # then it keeps its buffers mapped until the peers' bounded waits (FGA_TIMEOUT_S) have
        # expired and their sticky error status has stopped further launches from writing here.
        traceback.print_exc()
        try:
            import fused_gemm_a2a
            fused_gemm_a2a.hold_buffers_after_failure()   # drain, then wait out the peers' device time limit
        except Exception:
            pass
        os._exit(1)
