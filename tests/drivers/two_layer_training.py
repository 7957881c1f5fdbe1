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
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
for path in (ROOT, os.path.join(ROOT, 'fused-gemm-a2a_b200')):
    if path not in sys.path:
        sys.path.insert(0, path)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402

TENSORS = ('mb0/y', 'mb1/y', 'mb0/dx', 'mb1/dx', 'layer0/dw_qkv', 'layer0/dw_o', 'layer1/dw_qkv', 'layer1/dw_o')
FIRST_WEIGHT_GRAD = 4          # from here on the tensors are partial sums over the CP group
ELEMENT_TOLERANCE = 0.02       # |actual - expected| <= 0.02 * (peak + |expected|)
RMS_TOLERANCE = 0.02           # relative RMS error


def deviation(actual, expected):
    """(max error over peak, relative RMS error, within tolerance) of one tensor."""
    actual, expected = actual.float(), expected.float()
    error = (actual - expected).abs()
    peak = expected.abs().max().clamp_min(1e-12)
    rms = (error.square().mean() / expected.square().mean().clamp_min(1e-24)).sqrt()
    within = bool(torch.isfinite(actual).all()) and bool((error <= ELEMENT_TOLERANCE * (peak + expected.abs())).all())
    return (error.max() / peak).item(), rms.item(), within and rms.item() <= RMS_TOLERANCE


class DenseReference:
    """The same two layers in FP32 on the gathered tokens of all ranks, rounding to BF16 where the
    fused path does: after each projection, after attention, after the residual sum."""

    def __init__(self, parameters, heads, head_dim):
        self.weights = [w.detach().float().requires_grad_() for w in parameters]
        self.heads, self.head_dim = heads, head_dim

    def layer(self, x, w_qkv, w_out):
        bf = torch.bfloat16
        tokens = x.shape[0]
        per_head = F.linear(x.float(), w_qkv).to(bf).view(tokens, self.heads, 3, self.head_dim)   # rows [q_h; k_h; v_h]
        q, k, v = (per_head[:, :, i].float() for i in range(3))
        probabilities = (torch.einsum('thd,shd->hts', q, k) * self.head_dim ** -0.5).softmax(-1)
        attended = torch.einsum('hts,shd->thd', probabilities, v).to(bf)
        return x + F.linear(attended.flatten(1).float(), w_out).to(bf)

    def step(self, inputs, output_grads, rows):
        """Expected (y per micro-batch, dx per micro-batch, dW per parameter); activations cut down
        to this rank's rows, weight gradients complete."""
        inputs = [x.requires_grad_() for x in inputs]
        outputs = []
        for x in inputs:
            for w_qkv, w_out in zip(self.weights[0::2], self.weights[1::2]):
                x = self.layer(x, w_qkv, w_out)
            outputs.append(x)
        grads = torch.autograd.grad(outputs, (*inputs, *self.weights), output_grads)
        n = len(inputs)
        return [y[rows] for y in outputs] + [g[rows] for g in grads[:n]] + list(grads[n:])


def run(dev, hidden=1024, heads=8, total_tokens=512, replays=2):
    """Returns (failures, errors): failed labels of this rank and the error figures of every check.
    Collective over the default process group; never raises on a numerical mismatch."""
    from fused_gemm_a2a import FusedGemmA2AWorkspace, FusedOutputProjection, FusedQKVProjection
    cp, rank = dist.get_world_size(), dist.get_rank()
    assert total_tokens % cp == 0 and heads % cp == 0
    head_dim, local = hidden // heads, total_tokens // cp
    my_rows = slice(rank * local, (rank + 1) * local)
    bf = torch.bfloat16

    shared = torch.Generator(device='cpu').manual_seed(1234)      # parameters: identical on every rank
    private = torch.Generator(device='cpu').manual_seed(5678 + rank)

    def parameter(out_rows):
        values = torch.randn(out_rows, hidden, generator=shared) * hidden ** -0.5
        return torch.nn.Parameter(values.to(bf).to(dev))

    def activation(requires_grad):
        return torch.randn(local, hidden, generator=private).to(bf).to(dev).requires_grad_(requires_grad)

    layers = [(FusedQKVProjection(hidden, heads, weight=parameter(3 * hidden)),
               FusedOutputProjection(hidden, heads, weight=parameter(hidden))) for _ in range(2)]
    workspace = FusedGemmA2AWorkspace(hidden, heads, local)      # one workspace for both layers
    parameters = [module.weight for layer in layers for module in layer]
    reference = DenseReference(parameters, heads, head_dim)
    xs = [activation(True) for _ in range(2)]
    dys = [activation(False) for _ in range(2)]

    def attend(q, k, v):         # [P*M, N/P, D] each: every token, this rank's heads
        by_head = [t.transpose(0, 1) for t in (q, k, v)]
        return F.scaled_dot_product_attention(*by_head).transpose(0, 1).contiguous()

    def fused_step():
        """Both micro-batches go forward through both layers before anything goes backward."""
        outputs = []
        for x in xs:
            for qkv, proj in layers:
                q, k, v = qkv(x, workspace)
                shared_buffers = {buffer.untyped_storage().data_ptr() for buffer in workspace._view(local, 3).heads}
                assert not shared_buffers & {t.untyped_storage().data_ptr() for t in (q, k, v)}   # outputs are owned
                x = x + proj(attend(q, k, v), workspace)
            outputs.append(x)
        return [*outputs, *torch.autograd.grad(outputs, (*xs, *parameters), dys)]

    def all_ranks(t):
        parts = [torch.empty_like(t) for _ in range(cp)]
        dist.all_gather(parts, t.detach().contiguous())
        return torch.cat(parts)

    def expected_step():
        return reference.step([all_ranks(x) for x in xs], [all_ranks(dy) for dy in dys], my_rows)

    failures, errors = [], {}

    def check(stage, actual, expected):
        for index, (name, got, want) in enumerate(zip(TENSORS, actual, expected)):
            if index >= FIRST_WEIGHT_GRAD:
                got = got.float().clone()
                dist.all_reduce(got)
            peak_error, rms, ok = deviation(got, want)
            errors[f'{stage}/{name}'] = dict(max_error_over_peak=peak_error, relative_rms=rms)
            if not ok:
                failures.append(f'{stage}/{name}: {errors[f"{stage}/{name}"]}')

    def device_errors():
        if dev.type == 'cuda':
            torch.cuda.synchronize()
        status = workspace.comm.status.tolist()
        if status[0]:
            failures.append(f'device status {status}')

    previous_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        expected = expected_step()
        check('eager', fused_step(), expected)
        # Saved-tensor hooks (activation offloading and the like) hand backward plain tensors in
        # place of Parameters; main_grad and the other metadata must still come from the module's
        # own Parameter (reference fused_gemm_a2a.py:348-351, tests/mxfp8_driver.py:136-138).
        with torch.autograd.graph.saved_tensors_hooks(lambda t: t.detach(), lambda t: t):
            check('hooks', fused_step(), expected)
        device_errors()
        anybody_failed = torch.tensor([len(failures)], dtype=torch.int32, device=dev)
        dist.all_reduce(anybody_failed, op=dist.ReduceOp.MAX)   # every rank takes the same branch
        if replays and anybody_failed.item() == 0:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fused_step()                 # warm-up on the capture stream
            side.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                captured = fused_step()
            torch.cuda.current_stream().wait_stream(side)
            for replay in range(replays):
                with torch.no_grad():
                    for t in (*xs, *dys):
                        t.normal_()          # new inputs in place: the graph reads the same storage
                torch.cuda.synchronize()
                dist.barrier()
                graph.replay()
                torch.cuda.synchronize()
                check(f'graph{replay}', captured, expected_step())
                device_errors()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = previous_tf32
    return failures, errors


def main():
    local = int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    dist.init_process_group('nccl', device_id=dev)
    import fused_gemm_a2a
    fused_gemm_a2a.install_exit_guards()   # SIGTERM from the launcher: finish queued GPU work first
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
    fused_gemm_a2a.release_all()           # collective: drain, meet, unmap the peers, free
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
            import fused_gemm_a2a
            fused_gemm_a2a.hold_buffers_after_failure()   # drain, then wait out the peers' device time limit
        except Exception:
            pass
        os._exit(1)
