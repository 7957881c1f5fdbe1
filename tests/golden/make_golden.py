"""Generate golden vectors from the reference's own unfused Ulysses modules under gloo.

Run in a container that has the reference tree (it cannot travel to the GPU box):

    python tests/golden/make_golden.py --reference <checkout of the reference project>

Spawns CPU ranks (gloo, 127.0.0.1), imports benchmark/reference.py from the reference tree, runs
UlyssesQKVProjection and UlyssesOutputProjection forward + backward and writes

  tests/golden/ulysses_small_p2.npz   every input and output of a small geometry (P=2, M=5,
                                      H=32, 4 heads of 8, QKVG with bias), float32
  tests/golden/ulysses_small_p4.npz   the same for P=4, M=3, H=64, 8 heads of 8, QKV without bias
  tests/golden/ulysses_c1_p2.npz      the CPU configuration of the benchmark (P=2, per-rank M=512,
                                      H=1024, 8 heads, fp32, seed 0, no bias): inputs are
                                      regenerated from the seed, so only strided samples and
                                      float64 checksums of every output are stored

  tests/golden/ulysses_gqa_p2.npz     grouped-query attention (P=2, M=5, H=64, 8 query heads and
                                      2 key/value heads of 8, QKVG with bias): the reference's
                                      unfused modules with num_kv_heads < num_heads
  tests/golden/ulysses_gqa_r2_p2.npz  the same with 4 key/value heads, QKV without bias

The stored weights are segment-major [Q; K; V(; G)] exactly as the reference modules hold them; the
tests interleave them per head (or per key/value group) before handing them to the oracle.
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def c1_inputs(rank, p, m, hidden, heads, dtype=torch.float32):
    """Seeded inputs of the CPU benchmark configuration (also used by the tests and bench.py):
    weights from seed 0 on every rank, activations from seed 1 + rank."""
    d = hidden // heads
    g = torch.Generator().manual_seed(0)
    w = [torch.randn(hidden, hidden, generator=g, dtype=dtype) / hidden ** 0.5 for _ in range(3)]
    wo = torch.randn(hidden, hidden, generator=g, dtype=dtype) / hidden ** 0.5
    g = torch.Generator().manual_seed(1 + rank)
    x = torch.randn(m, hidden, generator=g, dtype=dtype)
    grads = [torch.randn(p * m, heads // p, d, generator=g, dtype=dtype) for _ in range(3)]
    o = torch.randn(p * m, heads // p, d, generator=g, dtype=dtype)
    dy = torch.randn(m, hidden, generator=g, dtype=dtype)
    return w, wo, x, grads, o, dy


def small_inputs(rank, p, m, hidden, heads, gate, bias, seed):
    d = hidden // heads
    s = 4 if gate else 3
    g = torch.Generator().manual_seed(seed)
    w = [torch.randn(hidden, hidden, generator=g) / hidden ** 0.5 for _ in range(s)]
    b = [torch.randn(hidden, generator=g) for _ in range(s)] if bias else None
    wo = torch.randn(hidden, hidden, generator=g) / hidden ** 0.5
    bo = torch.randn(hidden, generator=g) if bias else None
    g = torch.Generator().manual_seed(seed + 1 + rank)
    x = torch.randn(m, hidden, generator=g)
    grads = [torch.randn(p * m, heads // p, d, generator=g) for _ in range(s)]
    o = torch.randn(p * m, heads // p, d, generator=g)
    dy = torch.randn(m, hidden, generator=g)
    return w, b, wo, bo, x, grads, o, dy


def gqa_inputs(rank, p, m, hidden, heads, kv_heads, gate, bias, seed):
    """Like small_inputs with fewer key/value heads: K and V weights are [kv_heads*d, hidden]."""
    d = hidden // heads
    widths = [hidden, kv_heads * d, kv_heads * d] + ([hidden] if gate else [])
    g = torch.Generator().manual_seed(seed)
    w = [torch.randn(width, hidden, generator=g) / hidden ** 0.5 for width in widths]
    b = [torch.randn(width, generator=g) for width in widths] if bias else None
    wo = torch.randn(hidden, hidden, generator=g) / hidden ** 0.5
    bo = torch.randn(hidden, generator=g) if bias else None
    g = torch.Generator().manual_seed(seed + 1 + rank)
    x = torch.randn(m, hidden, generator=g)
    grads = [torch.randn(p * m, width // d // p, d, generator=g) for width in widths]
    o = torch.randn(p * m, heads // p, d, generator=g)
    dy = torch.randn(m, hidden, generator=g)
    return w, b, wo, bo, x, grads, o, dy


def run_reference(ref, hidden, heads, gate, w, b, wo, bo, x, grads, o, dy, kv_heads=None):
    """One forward + backward through the reference modules; returns a dict of float32 arrays."""
    qkv = ref.UlyssesQKVProjection(hidden, heads, kv_heads, bias=b is not None, gate=gate, dtype=x.dtype)
    out = ref.UlyssesOutputProjection(hidden, heads, bias=bo is not None, dtype=x.dtype)
    with torch.no_grad():
        for proj, weight in zip(qkv.projections, w):
            proj.weight.copy_(weight)
        if b is not None:
            for proj, bias in zip(qkv.projections, b):
                proj.bias.copy_(bias)
            out.o_proj.bias.copy_(bo)
        out.o_proj.weight.copy_(wo)
    xr = x.clone().requires_grad_()
    outs = qkv(xr)
    torch.autograd.backward(list(outs), grads)
    orr = o.clone().requires_grad_()
    y = out(orr)
    y.backward(dy)
    res = {f'out{i}': t.detach() for i, t in enumerate(outs)}
    res.update(dx=xr.grad, y=y.detach(), do=orr.grad,
               dw=torch.cat([p.weight.grad for p in qkv.projections]), dwo=out.o_proj.weight.grad)
    if b is not None:
        res.update(db=torch.cat([p.bias.grad for p in qkv.projections]), dbo=out.o_proj.bias.grad)
    return {k: v.float().numpy() for k, v in res.items()}


def sample(a, count=64):
    flat = np.ascontiguousarray(a).reshape(-1)
    idx = np.linspace(0, flat.size - 1, count).astype(np.int64)
    return flat[idx]


def worker(rank, world, reference_root, port, queue):
    sys.path.insert(0, reference_root)
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
    from benchmark import reference as ref
    results = {}
    if world == 2:
        w, b, wo, bo, x, grads, o, dy = small_inputs(rank, 2, 5, 32, 4, True, True, seed=100)
        res = run_reference(ref, 32, 4, True, w, b, wo, bo, x, grads, o, dy)
        res.update(x=x.numpy(), o=o.numpy(), dy=dy.numpy(),
                   **{f'g{i}': t.numpy() for i, t in enumerate(grads)})
        if rank == 0:
            res.update(w=torch.cat(w).numpy(), b=torch.cat(b).numpy(), wo=wo.numpy(), bo=bo.numpy())
        results['small_p2'] = res
        for name, kv_heads, gate, bias, seed in (('gqa_p2', 2, True, True, 300), ('gqa_r2_p2', 4, False, False, 400)):
            w, b, wo, bo, x, grads, o, dy = gqa_inputs(rank, 2, 5, 64, 8, kv_heads, gate, bias, seed)
            res = run_reference(ref, 64, 8, gate, w, b, wo, bo, x, grads, o, dy, kv_heads=kv_heads)
            res.update(x=x.numpy(), o=o.numpy(), dy=dy.numpy(), **{f'g{i}': t.numpy() for i, t in enumerate(grads)})
            if rank == 0:
                res.update(w=torch.cat(w).numpy(), wo=wo.numpy())
                if bias:
                    res.update(b=torch.cat(b).numpy(), bo=bo.numpy())
            results[name] = res
        w, wo, x, grads, o, dy = c1_inputs(rank, 2, 512, 1024, 8)
        res = run_reference(ref, 1024, 8, False, w, None, wo, None, x, grads, o, dy)
        results['c1_p2'] = {k + '_sample': sample(v) for k, v in res.items()} | {
            k + '_sum': np.float64(v.astype(np.float64).sum()) for k, v in res.items()} | {
            k + '_abs': np.float64(np.abs(v.astype(np.float64)).sum()) for k, v in res.items()}
    else:
        w, b, wo, bo, x, grads, o, dy = small_inputs(rank, 4, 3, 64, 8, False, False, seed=200)
        res = run_reference(ref, 64, 8, False, w, None, wo, None, x, grads, o, dy)
        res.update(x=x.numpy(), o=o.numpy(), dy=dy.numpy(),
                   **{f'g{i}': t.numpy() for i, t in enumerate(grads)})
        if rank == 0:
            res.update(w=torch.cat(w).numpy(), wo=wo.numpy())
        results['small_p4'] = res
    queue.put((rank, results))
    dist.barrier()
    dist.destroy_process_group()


def collect(world, reference_root, port):
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, reference_root, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(queue.get() for _ in range(world))
    for p in procs:
        p.join()
    return got


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument('--reference', default=os.environ.get(
        'FGA_REFERENCE_ROOT', os.path.join(os.path.expanduser('~'), 'reference')),
        help='checkout of the reference project (default: $FGA_REFERENCE_ROOT, else ~/reference)')
    args = ap.parse_args()
    for world, port in ((2, 29611), (4, 29612)):
        per_rank = collect(world, args.reference, port)
        for name in per_rank[0]:
            flat = {}
            for rank in range(world):
                for key, value in per_rank[rank][name].items():
                    shared = key in ('w', 'b', 'wo', 'bo')
                    flat[key if shared else f'r{rank}_{key}'] = value
            path = os.path.join(HERE, f'ulysses_{name}.npz')
            np.savez_compressed(path, **flat)
            print(path, os.path.getsize(path), 'bytes')


if __name__ == '__main__':
    main()
