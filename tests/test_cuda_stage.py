"""The CPU stage's emulation of CUDA-graph capture and replay (tests/cuda_stage.py), checked on its
own: the staged runs of the reference's programs mean something only if a replay really recomputes,
keeps the host decisions of the capture, and refuses what a real capture refuses."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import abi_simulator  # noqa: E402
import cuda_stage  # noqa: E402


def test_replay_recomputes_forward_and_backward_from_the_same_memory():
    g = torch.Generator().manual_seed(0)
    a = torch.randn(5, 7, generator=g, requires_grad=True)
    b = torch.randn(7, 3, generator=g, requires_grad=True)
    upstream = torch.randn(5, 3, generator=g)

    def step():
        y = (a @ b).relu()
        return (y, *torch.autograd.grad(y, (a, b), upstream))

    graph = cuda_stage.Graph()
    with cuda_stage.capture(graph):
        captured = step()
    for _ in range(2):
        with torch.no_grad():
            a.normal_()
            b.normal_()
            upstream.normal_()
        stale = [t.clone() for t in captured]
        graph.replay()
        for got, want, before in zip(captured, step(), stale):
            assert torch.equal(got, want)
            assert not torch.equal(got, before)


def test_host_decisions_are_frozen_at_capture():
    x = torch.ones(4)
    out = torch.zeros(4)
    mode = {'double': True}

    def step():
        out.copy_(x * 2 if mode['double'] else x * 3)

    graph = cuda_stage.Graph()
    with cuda_stage.capture(graph):
        step()
    mode['double'] = False              # a replay runs no Python of the program: it still doubles
    x.fill_(5)
    graph.replay()
    assert out.tolist() == [10.0] * 4


def test_what_a_real_capture_refuses_is_refused():
    x = torch.ones(3)
    with cuda_stage.OnHost():
        graph = cuda_stage.Graph()
        for forbidden in (lambda: x.sum().item(), lambda: x.tolist(), lambda: bool(x[0] > 0),
                          lambda: cuda_stage.CUDA_STAND_INS['synchronize'](), lambda: cuda_stage.Stream().synchronize(),
                          lambda: cuda_stage.Event().query()):
            with pytest.raises(RuntimeError, match='while a stream is capturing'):
                with cuda_stage.capture(graph):
                    forbidden()
        assert x.sum().item() == 3.0      # and allowed again outside
        with pytest.raises(RuntimeError, match='captured nothing'):
            cuda_stage.Graph().replay()


def test_simulated_launches_are_nodes_that_run_again_with_the_same_arguments():
    calls = []
    source = torch.arange(6.0)
    target = torch.zeros(6)

    @abi_simulator._as_launch
    def launch(address_of_source, address_of_target, count):
        # host code standing for a kernel: free to read memory, use numpy, meet other ranks
        calls.append(count)
        target.copy_(torch.from_numpy(source.numpy() * 2))
        return 0

    fresh_outputs = []
    launch.__wrapped__.after_replay = lambda old, new: fresh_outputs.append((old, new))   # on the function itself
    with cuda_stage.OnHost():
        graph = cuda_stage.Graph()
        with cuda_stage.capture(graph):
            assert launch(source.data_ptr(), target.data_ptr(), 6) == 0
            after = target + 1            # an ATen node behind the launch
        assert abi_simulator.launch_hook is None and calls == [6]
        kinds = [node[0] for node in graph.recording.nodes]
        assert kinds[0] == 'launch' and 'op' in kinds[1:]
        source.mul_(10)
        graph.replay()
    assert calls == [6, 6] and len(fresh_outputs) == 1
    assert torch.equal(target, source * 2) and torch.equal(after, source * 2 + 1)
