"""Generate golden vectors of the auxiliary kernels from the reference's own Triton kernels.

The reference's row-copy and bias-gradient kernels (fused_gemm_a2a_kernels.py:1053-1142) are Triton
programs; Triton's interpreter (TRITON_INTERPRET=1) executes them on CPU tensors, so their outputs
can be recorded without a GPU. The public wrappers (`resize_rank_rows`, `reduce_bias_grad`,
fused_gemm_a2a_kernels.py:1086-1192) insist on CUDA tensors, so this script launches the kernels
directly with the grids and block sizes those wrappers compute (restated in `launch_*` below, each
citing the wrapper lines it follows).

Run in a container that has the reference tree:

    python tests/golden/make_golden_aux.py --reference <checkout of the reference project>

Writes tests/golden/aux_kernels.npz: for every case its inputs (BF16 as raw uint16 bit patterns, so
nothing is lost in the file), its parameters and the kernels' outputs.
"""
import argparse
import os
import sys

os.environ['TRITON_INTERPRET'] = '1'   # before triton is imported

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
BF = torch.bfloat16


def bits(t):
    """BF16 tensor -> uint16 numpy array of its bit patterns; other dtypes -> numpy as they are."""
    t = t.detach().contiguous()
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == BF else t.numpy()


def launch_bias_grad(k, dy, out, accumulate):
    """reduce_bias_grad, fused_gemm_a2a_kernels.py:1095-1103, without its CUDA check."""
    import triton
    rows, width = dy.shape
    block_m, block_n = min(256, triton.next_power_of_2(rows)), min(64, triton.next_power_of_2(width))
    parts = triton.cdiv(rows, block_m)
    partial = out if parts == 1 else torch.empty((parts, width), dtype=torch.float32)
    k._bias_grad_partial[(triton.cdiv(width, block_n), parts)](
        dy, partial, rows, width, block_m, block_n, parts == 1, accumulate, num_warps=4)
    if parts > 1:
        k._bias_grad_finish[(triton.cdiv(width, block_n),)](
            partial, out, width, parts, min(128, triton.next_power_of_2(parts)), block_n, accumulate, num_warps=4)
    return out


def launch_resize(k, tensors, peers, rows, bias=None, head_dim=128, head_offset=0):
    """resize_rank_rows, fused_gemm_a2a_kernels.py:1176-1191, without its CUDA check."""
    import triton
    first = tensors[0]
    input_rows, width = first.shape[0] // peers, first.shape[1]
    outputs = tuple(torch.full((peers * rows, width), float('nan'), dtype=t.dtype) for t in tensors)
    if bias is None:
        k._copy_rank_rows[(triton.cdiv(rows * width, 4096), peers, len(tensors))](
            tensors, outputs, input_rows, rows, width, 4096, num_warps=4)
    else:
        columns = min(512, triton.next_power_of_2(width))
        tile_rows = 2048 // columns
        grid = (triton.cdiv(rows, tile_rows) * triton.cdiv(width, columns), peers, len(tensors))
        k._copy_biased_rank_rows[grid](tensors, outputs, input_rows, rows, bias, width,
                                       tile_rows, columns, head_dim, head_offset, num_warps=4)
    return outputs


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument('--reference', default=os.environ.get(
        'FGA_REFERENCE_ROOT', os.path.join(os.path.expanduser('~'), 'reference')))
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import fused_gemm_a2a_kernels as k

    g = torch.Generator().manual_seed(77)
    out = {}

    # ---- bias gradient: one part (written directly), several parts (partials + finish), both output
    # types, with and without accumulation into a previous value. A BF16 result is narrowed by the
    # interpreter without rounding (see the biased copies below), so it may sit one BF16 step below a
    # correctly rounded one.
    cases = (('bias_one_part_bf16', 200, 40, BF, False), ('bias_one_part_f32_acc', 256, 96, torch.float32, True),
             ('bias_parts_bf16_acc', 1000, 96, BF, True), ('bias_parts_f32', 1537, 66, torch.float32, False),
             ('bias_many_parts_f32_acc', 33000, 8, torch.float32, True))
    for name, rows, width, dtype, accumulate in cases:
        if rows > 30000:
            # More than 128 partial rows (the finishing kernel loops). Quarter-integers: every FP32 sum is
            # exact, so this case is bit-exact whatever the order of the additions.
            dy = torch.randint(-8, 9, (rows, width), generator=g).float().div(4).to(BF)
        else:
            dy = torch.randn(rows, width, generator=g).mul(3).to(BF)
        previous = torch.randn(width, generator=g).to(dtype)
        result = launch_bias_grad(k, dy, previous.clone(), accumulate)
        out.update({f'{name}.dy': bits(dy), f'{name}.previous': bits(previous), f'{name}.out': bits(result),
                    f'{name}.accumulate': np.int64(accumulate)})

    # ---- row copies without bias: grow (zero rows added), shrink (tail rows dropped), same size.
    for name, peers, in_rows, rows, width, count in (('copy_grow', 3, 5, 8, 40, 2), ('copy_shrink', 2, 9, 4, 24, 3),
                                                     ('copy_same', 4, 6, 6, 16, 1)):
        tensors = tuple(torch.randn(peers * in_rows, width, generator=g).to(BF) for _ in range(count))
        results = launch_resize(k, tensors, peers, rows)
        out.update({f'{name}.peers': np.int64(peers), f'{name}.rows': np.int64(rows)})
        for i, (t, r) in enumerate(zip(tensors, results)):
            out.update({f'{name}.in{i}': bits(t), f'{name}.out{i}': bits(r)})

    # ---- row copies with the interleaved per-head bias, added in FP32 and rounded once. The
    # interpreter narrows FP32 to BF16 by dropping the low 16 bits, where the compiled kernel rounds to
    # nearest even (the reference's own check, tests/row_copy_driver.py:40-57, demands equality with
    # torch's BF16 sum). The first three cases therefore use quarter-integers, whose sums are exact in
    # BF16 under either rule: they pin which bias element meets which column, bit for bit. The last
    # case has random values and differs from a correctly rounded result by at most one BF16 step.
    for name, peers, in_rows, rows, heads, head_dim, count, head_offset in (
            ('biased_grow', 2, 5, 8, 2, 128, 3, 2), ('biased_shrink', 3, 7, 4, 3, 16, 4, 0),
            ('biased_same', 2, 6, 6, 1, 64, 3, 5), ('biased_random', 2, 5, 8, 2, 128, 4, 1)):
        width = heads * head_dim
        shape, bias_len = (peers * in_rows, width), (head_offset * head_dim + width) * count + 32
        if name == 'biased_random':
            tensors = tuple(torch.randn(shape, generator=g).to(BF) for _ in range(count))
            bias = torch.randn(bias_len, generator=g).to(BF)
        else:
            tensors = tuple(torch.randint(-16, 17, shape, generator=g).float().div(4).to(BF) for _ in range(count))
            bias = torch.randint(-16, 17, (bias_len,), generator=g).float().div(4).to(BF)
        results = launch_resize(k, tensors, peers, rows, bias=bias, head_dim=head_dim, head_offset=head_offset)
        out.update({f'{name}.peers': np.int64(peers), f'{name}.rows': np.int64(rows), f'{name}.bias': bits(bias),
                    f'{name}.head_dim': np.int64(head_dim), f'{name}.head_offset': np.int64(head_offset)})
        for i, (t, r) in enumerate(zip(tensors, results)):
            out.update({f'{name}.in{i}': bits(t), f'{name}.out{i}': bits(r)})

    path = os.path.join(HERE, 'aux_kernels.npz')
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), 'bytes,', len(out), 'arrays')


if __name__ == '__main__':
    main()
