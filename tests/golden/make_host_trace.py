"""Writes tests/golden/host_call_trace_p1.json and host_call_trace_p2_rank{0,1}.json: the C-ABI call
sequence of the host layer for the scenario in tests/host_trace.py, recorded on the CPU (gloo).
Run it only after a deliberate change of the launch plan, and review the diff it produces.

    python tests/golden/make_host_trace.py
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for path in (ROOT, os.path.join(ROOT, 'fused-gemm-a2a_b200'), os.path.join(ROOT, 'tests')):
    if path not in sys.path:
        sys.path.insert(0, path)

import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

P2_CONFIGS = (1, 3)


def worker(rank, world, port, configs, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import host_trace
    calls = host_trace.trace(configs)
    name = 'host_call_trace_p1.json' if world == 1 else f'host_call_trace_p{world}_rank{rank}.json'
    with open(os.path.join(out_dir, name), 'w') as f:
        f.write(host_trace.dump(calls))
    dist.barrier()
    dist.destroy_process_group()


def record(world, configs, out_dir, port):
    ctx = mp.get_context('spawn')
    procs = [ctx.Process(target=worker, args=(r, world, port, configs, out_dir)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        if p.exitcode != 0:
            raise SystemExit(f'trace worker failed with exit code {p.exitcode}')


if __name__ == '__main__':
    record(1, (0, 1, 2, 3, 4), HERE, 29631)
    record(2, P2_CONFIGS, HERE, 29632)
