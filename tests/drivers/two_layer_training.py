"""Two transformer layers, two micro-batches, attention between the fused projections.

The layout of the reference's tests/attention_training_driver.py with torch's scaled-dot-product
attention in place of FlashAttention-4 (not installed here): both micro-batches finish their
forward before either backward, the layers share one workspace, nothing is cloned by the caller.
That is the lifetime check: outputs of a projection must survive every later use of the shared
buffers, and what backward needs must still be intact after four more forwards.

Expected values: FP32 torch on the gathered inputs with the same BF16 rounding points (linear
outputs, attention output, residual sum). Tolerance, as in the reference driver: every element
within 0.02 * (peak + |expected|) and relative RMS error <= 0.02; weight gradients are summed over
the CP group first.

Importable (run(...) on an initialised process group) and runnable under torch.distributed.run,
where the ranks agree on the verdict before anybody leaves.
"""
import os
import sys
import time
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
for path in (ROOT, os.path.join(ROOT, 'fused-gemm-a2a_b200')):
    if path not in sys.path:
        sys.path.insert(0, path)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402

LABELS = ('mb0/y', 'mb1/y', 'mb0/dx', 'mb1/dx', 'layer0/dw_qkv', 'layer0/dw_o', 'layer1/dw_qkv', 'layer1/dw_o')


def run(dev, hidden=1024, heads=8, total_tokens=512, replays=2):
    """Returns (failures, errors): failed labels of this rank and the error figures of every check.
    Collective over the default process group; never raises on a numerical mismatch."""
    from fused_gemm_a2a import FusedGemmA2AWorkspace, FusedOutputProjection, FusedQKVProjection
    cp, rank = dist.get_world_size(), dist.get_rank()
    assert total_tokens % cp == 0 and heads % cp == 0
    head_dim = hidden // heads
    local = total_tokens // cp
    rows = slice(rank * local, (rank + 1) * local)
    bf = torch.bfloat16
    gen = torch.Generator(device='cpu').manual_seed(1234)   # parameters: identical on every rank

    def weight(n_rows):
        return torch.nn.Parameter((torch.randn(n_rows, hidden, generator=gen) * hidden ** -0.5).to(bf).to(dev))

    layers = [(FusedQKVProjection(hidden, heads, weight=weight(3 * hidden)),
               FusedOutputProjection(hidden, heads, weight=weight(hidden))) for _ in range(2)]
    workspace = FusedGemmA2AWorkspace(hidden, heads, local)
    parameters = tuple(module.weight for layer in layers for module in layer)
    reference_weights = [w.detach().float().requires_grad_() for w in parameters]
    gen = torch.Generator(device='cpu').manual_seed(5678 + rank)
    xs = [torch.randn(local, hidden, generator=gen).to(bf).to(dev).requires_grad_() for _ in range(2)]
    dys = [torch.randn(local, hidden, generator=gen).to(bf).to(dev) for _ in range(2)]

    def attention(q, k, v):      # [P*M, N/P, D] each: all tokens, this rank's heads
        o = F.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1))
        return o.transpose(0, 1).contiguous()

    def fused_step():
        ys = []
        for x in xs:
            for qkv, proj in layers:
                q, k, v = qkv(x, workspace)
                for tensor, buffer in zip((q, k, v), workspace._view(local, 3).heads):
                    assert tensor.untyped_storage().data_ptr() != buffer.untyped_storage().data_ptr()
                x = x + proj(attention(q, k, v), workspace)
            ys.append(x)
        gradients = torch.autograd.grad(ys, (*xs, *parameters), dys)
        return (*ys, *gradients)

    def gather(t):
        parts = [torch.empty_like(t) for _ in range(cp)]
        dist.all_gather(parts, t.detach().contiguous())
        return torch.cat(parts)

    def reference_step():
        inputs = [gather(x).requires_grad_() for x in xs]
        gradients = [gather(dy) for dy in dys]
        ys = []
        for x in inputs:
            for wqkv, wo in zip(reference_weights[::2], reference_weights[1::2]):
                packed = F.linear(x.float(), wqkv).to(bf)
                q, k, v = packed.view(total_tokens, heads, 3, head_dim).unbind(2)
                scores = torch.einsum('thd,shd->hts', q.float(), k.float()) * head_dim ** -0.5
                o = torch.einsum('hts,shd->thd', scores.softmax(-1), v.float()).to(bf)
                x = x + F.linear(o.flatten(1).float(), wo).to(bf)
            ys.append(x)
        grads = torch.autograd.grad(ys, (*inputs, *reference_weights), gradients)
        return (*(y[rows] for y in ys), *(g[rows] for g in grads[:2]), *grads[2:])

    failures, errors = [], {}

    def check(actuals, expected, label):
        for i, (actual, ref, name) in enumerate(zip(actuals, expected, LABELS)):
            if i >= 4:                       # weight gradients are partial sums over the CP group
                actual = actual.float().clone()
                dist.all_reduce(actual)
            actual, ref = actual.float(), ref.float()
            delta = (actual - ref).abs()
            peak = ref.abs().max().clamp_min(1e-12)
            rms = delta.square().mean().sqrt() / ref.square().mean().sqrt().clamp_min(1e-12)
            good = torch.isfinite(actual).all() & (delta <= 0.02 * (peak + ref.abs())).all() & (rms <= 0.02)
            errors[f'{label}/{name}'] = dict(max_error_over_peak=(delta.max() / peak).item(), relative_rms=rms.item())
            if not good.item():
                failures.append(f'{label}/{name}: {errors[f"{label}/{name}"]}')

    previous_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        expected = reference_step()
        check(fused_step(), expected, 'eager')
        # Saved-tensor hooks (activation offloading and the like) hand backward plain tensors in
        # place of Parameters; main_grad and the other metadata must still come from the module's
        # own Parameter (reference fused_gemm_a2a.py:348-351, tests/mxfp8_driver.py:136-138).
        with torch.autograd.graph.saved_tensors_hooks(lambda t: t.detach(), lambda t: t):
            check(fused_step(), expected, 'hooks')
        torch.cuda.synchronize()
        if workspace.comm.status.tolist()[0]:
            failures.append(f'device status {workspace.comm.status.tolist()}')
        anybody_failed = torch.tensor([len(failures)], dtype=torch.int32, device=dev)
        dist.all_reduce(anybody_failed, op=dist.ReduceOp.MAX)   # every rank takes the same branch
        if replays and anybody_failed.item() == 0:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                fused_step()
            stream.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                captured = fused_step()
            torch.cuda.current_stream().wait_stream(stream)
            for replay in range(replays):
                with torch.no_grad():
                    for t in (*xs, *dys):
                        t.normal_()
                torch.cuda.synchronize()
                dist.barrier()
                graph.replay()
                torch.cuda.synchronize()
                check(captured, reference_step(), f'graph{replay}')
                if workspace.comm.status.tolist()[0]:
                    failures.append(f'device status {workspace.comm.status.tolist()}')
    finally:
        torch.backends.cuda.matmul.allow_tf32 = previous_tf32
    return failures, errors


def main():
    local = int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    dist.init_process_group('nccl', device_id=dev)
    failures, errors = run(dev)
    # Ranks leave together: a rank that exits frees buffers its peers may still store into.
    flag = torch.tensor([len(failures)], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    for failure in failures:
        print(f'[rank {dist.get_rank()}] FAIL {failure}', flush=True)
    if dist.get_rank() == 0 and flag.item() == 0:
        worst = max(e['relative_rms'] for e in errors.values())
        print(f'PASS two layers x two micro-batches on {dist.get_world_size()} GPUs; worst relative RMS {worst:.2e}',
              flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if flag.item() else 0)


if __name__ == '__main__':
    try:
        main()
    except SystemExit:
        raise
    except BaseException:
        # Unexpected: keep this rank's buffers mapped until the peers' bounded waits have run out.
        traceback.print_exc()
        try:
            torch.cuda.synchronize()
        except Exception:
            pass
        time.sleep(float(os.environ.get('FGA_TIMEOUT_S', '10')) + 2.0)
        os._exit(1)
