"""Argument validation of the C ABI, without a GPU: every launcher checks its geometry on the host
before it touches CUDA, returns FGA_INVALID_ARGUMENT (-1) and leaves a message for fga_last_error().
The pointer arguments used here are never dereferenced (the calls are rejected first); the cases
cover the constraints that include/fga.h states and the message fragments the Python layer and the
reference's tests rely on."""
import ctypes

import pytest

import _fga_native

P = 0x1000            # any non-null "pointer": validation fails before it could be used
TABLES = (ctypes.c_void_p * 4)(P, P, P, P)
NS = 1_000_000_000


def push(m=300, k=512, a_rows=512, segments=3, n_segment=512, head_rows=512, rank=0, p=1, tables=TABLES, bias=None):
    return ('fga_gemm_push', (P, m, k, a_rows, P, 0, bias, segments, n_segment, tables, head_rows, rank, p, P, NS, None))


def recv_mx(c=P, roles=3):
    return ('fga_gemm_recv_mx', (P, P, P, 512, 1536, P, P, 512, 1536, 512, c, P, P, P, TABLES, 3, 300, 2, 0, 1, roles,
                                 None, None, P, NS, None))


def recv(recv_rows=512, k=1536, n=512, num_in=3, src_rows=300, split=2, rank=0, p=1, roles=3, srcs=TABLES):
    return ('fga_gemm_recv', (P, recv_rows, k, P, 1, n, P, P, P, P, srcs, num_in, src_rows, split, rank, p, roles,
                              None, None, P, NS, None))


def local(m=256, n=256, k=256, lda=256, ldb=256, ldc=256, out_f32=0, accumulate=0, c=P):
    return ('fga_gemm_local', (P, 0, P, 0, m, n, k, lda, ldb, c, ldc, out_f32, accumulate, P, NS, None))


CASES = [
    (push(segments=2), 'three/four'),
    (push(p=33), 'bad rank'),
    (push(rank=1, p=1), 'bad rank'),
    (push(k=100), 'multiple of 8'),
    (push(a_rows=300), 'tile multiple'),
    (push(a_rows=1024, head_rows=512), 'tile multiple'),
    (push(n_segment=384, p=2), r'CP \* tile N'),
    (push(n_segment=0), r'CP \* tile N'),
    (push(bias=P + 2), 'bias must be 16-byte aligned'),
    (('fga_gemm_push_mx', (P, P, 512, 512, 512, P, P, 1536, P + 8, 3, 512, TABLES, 512, 0, 1, P, NS, None)),
     'bias must be 16-byte aligned'),
    (recv_mx(c=P + 4), 'output must be 16-byte aligned'),
    (recv_mx(roles=0), 'roles'),
    (('fga_gemm_push_gqa', (P, 300, 512, 512, P, None, 6, 4, 0, TABLES, 512, 0, 4, P, NS, None)), 'split evenly over CP'),
    (('fga_gemm_push_gqa', (P, 300, 512, 512, P, None, 8, 0, 0, TABLES, 512, 0, 4, P, NS, None)), 'split evenly over CP'),
    (('fga_gemm_push_gqa', (P, 300, 512, 300, P, None, 8, 4, 0, TABLES, 512, 0, 4, P, NS, None)), 'tile multiple'),
    (('fga_gemm_push_gqa', (P, 300, 512, 512, P, P + 6, 8, 4, 1, TABLES, 512, 0, 4, P, NS, None)), 'bias must be 16-byte'),
    (('fga_gemm_recv_gqa', (P, 512, P, 512, P, P, P, P, TABLES, 6, 2, 0, 300, 2, 0, 4, 3, None, P, NS, None)),
     'split evenly over CP'),
    (('fga_gemm_recv_gqa', (P, 512, P, 512, P, P, P, P, TABLES, 8, 2, 0, 600, 2, 0, 4, 3, None, P, NS, None)),
     'Receive source rows'),
    (('fga_gemm_recv_gqa', (P, 512, P, 512, P + 8, P, P, P, TABLES, 8, 2, 1, 300, 2, 0, 4, 3, None, P, NS, None)),
     'output must be 16-byte aligned'),
    # push_gqa_mx: aq, sfa, a_rows_padded, kp, a_rows, bq, sfb, b_rows_padded, bias, kv_heads, q_per_kv, gate, tables, ...
    (('fga_gemm_push_gqa_mx', (P, P, 512, 512, 512, P, P, 4096, None, 6, 4, 0, TABLES, 512, 0, 4, P, NS, None)),
     'split evenly over CP'),
    (('fga_gemm_push_gqa_mx', (P, P, 512, 100, 512, P, P, 4096, None, 8, 2, 0, TABLES, 512, 0, 4, P, NS, None)),
     'multiple of 128'),
    (('fga_gemm_push_gqa_mx', (P, P, 512, 512, 300, P, P, 4096, None, 8, 2, 0, TABLES, 512, 0, 4, P, NS, None)),
     'tile multiple'),
    (('fga_gemm_push_gqa_mx', (P, P, 512, 512, 512, P, P, 1024, None, 8, 2, 0, TABLES, 512, 0, 4, P, NS, None)),
     'weight rows must be padded'),
    # recv_gqa_mx: recv, mx_recv, mx_scale, recv_rows, bq, sfb, b_rows_padded, b_kp, n, c, peer_recv, peer_counters,
    #              counters, srcs, kv_heads, q_per_kv, gate, src_rows, split, rank, p, roles, progress, status, ...
    (('fga_gemm_recv_gqa_mx', (P, P, P, 512, P, P, 512, 4096, 512, P, P, P, P, TABLES, 6, 2, 0, 300, 2, 0, 4, 3, None,
                               P, NS, None)), 'split evenly over CP'),
    (('fga_gemm_recv_gqa_mx', (P, P, P, 512, P, P, 512, 1024, 512, P, P, P, P, TABLES, 8, 2, 0, 300, 2, 0, 4, 3, None,
                               P, NS, None)), "padded K must cover K"),
    (('fga_gemm_recv_gqa_mx', (P, P, P, 512, P, P, 512, 4096, 512, P, P, P, P, TABLES, 8, 2, 0, 300, 2, 0, 4, 0, None,
                               P, NS, None)), 'roles'),
    (recv(num_in=2), 'three/four'),
    (recv(recv_rows=300), 'multiple of 256'),
    (recv(src_rows=0), 'Receive source rows'),
    (recv(src_rows=513), 'Receive source rows'),
    (recv(k=1000), 'split evenly'),
    (recv(n=100), 'tile N must divide'),
    (recv(split=3), 'FUSED_PUSH_SPLIT'),
    (recv(roles=0), 'roles'),
    (recv(roles=4), 'roles'),
    (recv(p=0), 'bad rank'),
    (local(n=100), 'multiple of 128'),
    (local(accumulate=1), 'FP32 output'),
    (local(lda=100), '16-byte aligned'),
    (local(ldc=128), '16-byte aligned'),
    (local(c=P + 2), '16-byte aligned'),
    (('fga_gemm_local_mx', (P, P, 256, P, P, 256, 256, 256, 100, P, 256, 0, 0, P, NS, None)), 'multiples of 128'),
    (('fga_gemm_local_mx', (P, P, 128, P, P, 256, 256, 256, 128, P, 256, 0, 0, P, NS, None)), 'padded'),
    (('fga_gemm_local_mx', (P, P, 256, P, P, 256, 256, 256, 128, P, 256, 0, 1, P, NS, None)), 'FP32 output'),
    (('fga_gemm_push_mx', (P, P, 512, 512, 512, P, P, 1536, None, 2, 512, TABLES, 512, 0, 1, P, NS, None)), 'three/four'),
    (('fga_gemm_push_mx', (P, P, 512, 100, 512, P, P, 1536, None, 3, 512, TABLES, 512, 0, 1, P, NS, None)), 'multiple of 128'),
    (('fga_gemm_push_mx', (P, P, 512, 512, 512, P, P, 1024, None, 3, 512, TABLES, 512, 0, 1, P, NS, None)), 'padded'),
    (('fga_barrier', (P, P, 2, 2, 0, None, 0, None, P, NS, None)), r'single-warp.*rank=2'),
    (('fga_barrier', (P, P, 0, 2, 1, None, 4, None, P, NS, None)), 'bump needs counters'),
    (('fga_copy_rank_rows', (TABLES, TABLES, 5, 1, 1, 1, 128, None, 128, 0, None)), 'segments'),
    (('fga_copy_rank_rows', (TABLES, TABLES, 1, 0, 1, 1, 128, None, 128, 0, None)), 'fga_copy_rank_rows'),
    (('fga_copy_rank_rows', (TABLES, TABLES, 1, 1, 1, 1, 100, P, 128, 0, None)), 'Bias must cover'),
    (('fga_bias_grad', (P, 0, 128, P, 0, 0, P, None)), 'Bias reduction requires'),
    (('fga_bias_grad', (P, 256 * 70000, 128, P, 0, 0, P, None)), 'too many rows'),
    (('fga_bias_grad_static', (P, 256 * 70000, 8, P, 0, 0, None)), 'too many rows'),
    (('fga_mx_quantize', (P, 100, 100, 3, 5, P, P, 256, 128, None)), '16-byte aligned rows or columns'),
    (('fga_mx_quantize', (P, 100, 100, 100, 1, P, P, 100, 128, None)), 'padded|multiple'),
    (('fga_symm_alloc', (0, ctypes.pointer(ctypes.c_void_p()))), 'fga_symm_alloc'),
]


@pytest.mark.parametrize('call,fragment', CASES, ids=[f'{c[0][0]}-{i}' for i, c in enumerate(CASES)])
def test_launchers_reject_bad_arguments_before_touching_cuda(call, fragment):
    import re
    name, args = call
    lib = _fga_native.lib()
    assert getattr(lib, name)(*args) == -1
    message = lib.fga_last_error().decode()
    assert re.search(fragment, message), message


def test_static_bias_gradient_states_its_limit():
    lib = _fga_native.lib()
    capacity = lib.fga_bias_grad_static_capacity_floats()
    assert capacity == 1 << 20
    rows, width = 256 * 1025, 1024          # 1025 partial rows x 1024 floats: one row too many
    assert lib.fga_bias_grad_static(P, rows, width, P, 0, 0, None) == -1
    message = lib.fga_last_error().decode()
    assert str(capacity) in message or '1048576' in message, message
