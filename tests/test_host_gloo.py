"""Host-side multi-rank plumbing on CPU: two gloo ranks exchange memory handles and derive peer
address tables exactly as the GPU path does, with the device allocator replaced by a fake."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, queue):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import fused_gemm_a2a as fused
    layout = [('head0', (world * 256, 128), torch.bfloat16), ('recv', (256, 384), torch.bfloat16),
              ('counters', (2,), torch.int32)]
    offsets, total = fused.slab_offsets(layout)
    local = 0x10000000 * (rank + 1)
    handle = bytes([rank]) * 64
    opened = []

    def open_peer(raw):
        opened.append(raw[0])
        return 0x20000000 * (raw[0] + 1) + rank  # distinct mapping per (owner, opener)

    addresses = fused.exchange_handles(dist.group.WORLD, rank, world, handle, local, open_peer)
    queue.put((rank, offsets, total, addresses, sorted(opened)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 3])
def test_handle_exchange_and_slab_layout(world):
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29650 + world, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, offsets, total, addresses, opened in results:
        assert [o for o, _ in offsets] == [0, world * 256 * 128 * 2, world * 256 * 128 * 2 + 256 * 384 * 2]
        assert all(o % 1024 == 0 for o, _ in offsets) and total % 1024 == 0
        assert total >= offsets[-1][0] + 8
        assert opened == [r for r in range(world) if r != rank]
        assert addresses[rank] == 0x10000000 * (rank + 1)
        for peer in range(world):
            if peer != rank:
                assert addresses[peer] == 0x20000000 * (peer + 1) + rank


def test_malformed_exchange_is_rejected(monkeypatch):
    import fused_gemm_a2a as fused

    def fake_gather(out, obj, group=None):
        out[0], out[1] = (0, b'x' * 64), (0, b'y' * 64)   # rank 1 reports the wrong sender

    monkeypatch.setattr(fused.dist, 'all_gather_object', fake_gather)
    with pytest.raises(RuntimeError, match='malformed'):
        fused.exchange_handles(None, 0, 2, b'x' * 64, 1, lambda raw: 2)


def _descriptor_worker(rank, world, port, queue):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import fused_gemm_a2a as fused
    mine = os.memfd_create(f'rank{rank}')
    os.write(mine, f'memory of rank {rank}'.encode())
    received = fused.exchange_descriptors(dist.group.WORLD, rank, world, mine)
    contents = [os.pread(fd, len('memory of rank 0'), 0).decode() for fd in received]
    distinct = len(set(received)) == world and received[rank] == mine
    dist.barrier()
    # writes through a received descriptor reach the owner's memory file
    for owner, fd in enumerate(received):
        os.pwrite(fd, f'{rank}'.encode(), 32 + rank)
    dist.barrier()
    marks = os.pread(mine, world, 32).decode()
    for owner, fd in enumerate(received):
        if owner != rank:
            os.close(fd)
    os.close(mine)
    queue.put((rank, contents, distinct, marks))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 3])
def test_descriptors_travel_to_every_peer(world):
    """The exchange used for VMM-backed symmetric memory, with memory files standing in for CUDA
    shareable handles: every rank ends up with a working descriptor of every peer's file."""
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    procs = [ctx.Process(target=_descriptor_worker, args=(r, world, 29690 + world, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, contents, distinct, marks in results:
        assert contents == [f'memory of rank {owner}' for owner in range(world)]
        assert distinct
        assert marks == ''.join(str(r) for r in range(world))
