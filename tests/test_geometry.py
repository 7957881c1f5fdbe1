"""Host-side geometry rules of the fused kernels, no GPU.

Two kinds of checks. Known answers: the values and message fragments that the reference pins in its
own unit tests (tests/test_recv_plan.py, tests/test_row_blocks.py) are listed here as tables, so
that they hold on a machine without the reference checkout (where it exists,
test_reference_unit_tests_compat.py runs the reference's files themselves). Properties: what the
kernels of this build rely on, for every geometry in a sweep - a pusher job is a whole number of
rows, a raster group divides the tile count, a chosen tile always passes the validator.
"""
import os
import subprocess
import sys
from unittest.mock import patch

import pytest
import torch

import fused_gemm_a2a as fused
import fused_gemm_a2a_kernels as kernels

BF16 = torch.bfloat16


# ---------------------------------------------------------------------------- known answers
@pytest.mark.parametrize('fn,args,expected', [
    (kernels.mxfp8_tile_n, ('push', 4096, 16), 256),
    (kernels.mxfp8_tile_n, ('push', 4096, 32), 128),
    (kernels.mxfp8_tile_n, ('local', 384), 128),
    (kernels.tile_swizzle, (32, 8), 8),
    (kernels.tile_swizzle, (4, 8), 4),
    (kernels.tile_swizzle, (6, 8), 2),
    (kernels.push_split, (4096, 16, 1), 1),
    (kernels.push_split, (12288, 16, 3), 1),
    (kernels.push_split, (12288, 4, 3), 4),
    (kernels.push_split, (4096, 16, 1, 8), 8),
    (kernels.padded_rows, (7456, 256), 7680),
    (kernels.padded_rows, (7456, 128), 7552),
    (kernels.padded_rows, (8192, 256), 8192),
    (kernels.padded_rows, (1, 256), 256),
])
def test_values_pinned_by_the_reference_tests(fn, args, expected):
    assert fn(*args) == expected


@pytest.mark.parametrize('fn,args,fragment', [
    (kernels.validate_peer_count, (0,), 'single-warp'),
    (kernels.validate_peer_count, (-1,), 'single-warp'),
    (kernels.validate_peer_count, (33,), 'single-warp'),
    (kernels.validate_peer_count, (64,), 'single-warp'),
    (kernels.validate_tile_n, ('push', 256, 16384, 16, 4096, 4, 128), 'one N tile per head'),
    (kernels.validate_tile_n, ('push', 256, 4096, 32, 4096), r'CP \* tile N'),
    (kernels.validate_tile_n, ('recv', 256, 4095, 16), 'tile N must divide'),
    (kernels.validate_tile_n, ('recv', 256, 4097, 16), 'tile N must divide'),
    (kernels.validate_tile_n, ('recv', 0, 4096, 16), 'tile N must divide'),
    (kernels.validate_tile_n, ('recv', -128, 4096, 16), 'tile N must divide'),
    (kernels.validate_tile_n, ('local', 128, 4096, 1), 'push/recv'),
    (kernels.validate_tile_n, ('recv', 128, 4096, 1, 0, 2), 'three/four'),
    (kernels.validate_tile_n, ('recv', 128, 4096, 1, 0, 3, 0), 'positive head dimension'),
    (kernels.tile_swizzle, (0, 8), 'positive'),
    (kernels.tile_swizzle, (4, 0), 'positive'),
    (kernels.tile_swizzle, (4, -1), 'positive'),
    (kernels.push_split, (4096, 0, 1), 'split evenly'),
    (kernels.push_split, (4000, 16, 1), 'multiple of 64'),
    (kernels.push_split, (32 * 16, 16, 1), 'multiple of 64'),
    (kernels.padded_rows, (0, 256), 'positive'),
    (kernels.padded_rows, (7456, 0), 'positive'),
    (kernels.padded_rows, (-1, 128), 'positive'),
] + [(kernels.push_split, (4096, 16, 1, bad), 'FUSED_PUSH_SPLIT') for bad in (-1, 3, 6, 17, 64, 129)])
def test_rejections_pinned_by_the_reference_tests(fn, args, fragment):
    with pytest.raises(ValueError, match=fragment):
        fn(*args)


def test_accepted_geometries_of_the_reference_tests():
    for peers in (1, 4, 8, 16, 32):
        kernels.validate_peer_count(peers)
    kernels.validate_tile_n('recv', 256, 4096, 16, num_segments=4, head_dim=128)   # interleaved K, free N tile
    kernels.validate_tile_n('push', 128, 16384, 16, 4096, 4, 128)
    kernels.validate_tile_n('push', 256, 4096, 16, 4096)
    kernels.validate_tile_n('push', 128, 4096, 32, 4096)
    assert kernels.MMA_TILER_MN == (256, 128) and fused.MMA_TILER_MN == kernels.MMA_TILER_MN


# ---------------------------------------------------------------------------- properties
@pytest.mark.parametrize('peers', [1, 2, 4, 8, 16, 32])
def test_a_selected_mxfp8_tile_always_validates(peers):
    for heads_per_peer in (1, 2, 3, 4):
        hidden = peers * heads_per_peer * 128
        for segments in (1, 3, 4):
            tile = kernels.mxfp8_tile_n('push', hidden * segments, peers, segments)
            kernels.validate_tile_n('push', tile, hidden * segments, peers, hidden, segments, 128)
            assert tile == 128 or segments == 1
        kernels.validate_tile_n('recv', kernels.mxfp8_tile_n('recv', hidden, peers), hidden, peers)
        assert hidden % kernels.mxfp8_tile_n('local', hidden) == 0


def test_raster_groups_divide_the_tile_count():
    for clusters in range(1, 129):
        for requested in (1, 2, 3, 4, 8, 16):
            group = kernels.tile_swizzle(clusters, requested)
            assert clusters % group == 0 and 1 <= group <= requested


@pytest.mark.parametrize('segments', [1, 3, 4])
def test_pusher_jobs_tile_a_row_block(segments):
    """Whatever the width, a job is a whole number (>= 4) of the 128 rows, the split is a power of
    two, and the automatic choice keeps a job near 64 KB: never above it unless one row block per
    job already is, never below 32 KB unless the row limit of 16 jobs per block binds."""
    for width in range(64, 8193, 64):          # BF16 columns one source contributes
        split = kernels.push_split(width * 4 * segments, 4, segments)
        rows = kernels.CTA_M // split
        assert rows * split == kernels.CTA_M and rows % 4 == 0 and split & (split - 1) == 0
        job_bytes = rows * width * 2
        assert job_bytes >= 64 * 1024 or split == 1 or job_bytes * 2 > 64 * 1024 or split == 16
        assert job_bytes < 128 * 1024 or split == 16


def test_padding_is_the_next_multiple():
    for tile in (128, 256):
        for valid in list(range(1, 700)) + [8191, 8192, 8193]:
            padded = kernels.padded_rows(valid, tile)
            assert padded % tile == 0 and 0 <= padded - valid < tile


# ---------------------------------------------------------------------------- main_grad validation
def _mxfp8_main_grad_cases():
    shape = (384, 128)
    misaligned = torch.empty(384 * 128 + 1, dtype=torch.float32)[1:].view(shape)
    assert misaligned.is_contiguous() and misaligned.data_ptr() % 16
    return {
        'fewer rows': torch.empty(128, 128, dtype=torch.float32),
        'more columns': torch.empty(384, 256, dtype=torch.float32),
        'flattened': torch.empty(384 * 128, dtype=torch.float32),
        'other device': torch.empty(shape, device='meta', dtype=torch.float32),
        'misaligned view': misaligned,
        'bf16 storage': torch.empty(shape, dtype=BF16),
        'transposed strides': torch.empty(128, 384, dtype=torch.float32).T,
    }


@pytest.mark.parametrize('case', sorted(_mxfp8_main_grad_cases()))
def test_unusable_mxfp8_main_grad_is_rejected_before_any_kernel(case):
    """A main_grad the accumulating epilogue cannot write (shape, device, dtype, strides or
    alignment) must raise before the quantizers or the GEMM run: a silent truncation of the weight
    gradient would be worse than the error (the cases of reference tests/test_recv_plan.py:94-123)."""
    weight = torch.nn.Parameter(torch.empty(384, 128, dtype=BF16))
    weight.main_grad = _mxfp8_main_grad_cases()[case]
    with patch.object(fused, 'mxfp8_wgrad') as gemm:
        with pytest.raises(ValueError, match='main_grad'):
            fused._weight_grad(weight, torch.empty(33, 384, dtype=BF16), torch.empty(33, 128, dtype=BF16), 'mxfp8')
        gemm.assert_not_called()


# ---------------------------------------------------------------------------- construction
def test_modules_validate_on_the_host_and_only_the_workspace_needs_a_group():
    weight_qkv = torch.empty(768, 256, dtype=BF16)
    weight_out = torch.empty(256, 256, dtype=BF16)
    with patch.object(fused._Comm, 'get', side_effect=AssertionError('communication set up at construction')):
        qkv = fused.FusedQKVProjection(256, 2, weight=weight_qkv)
        out = fused.FusedOutputProjection(256, 2, weight=weight_out)
    assert qkv.weight is weight_qkv and out.weight is weight_out      # kept by reference, not copied
    assert (qkv.segments, out.segments, qkv.head_dim) == (3, 1, 128)
    assert fused.FusedQKVProjection.weight_layout == 'head_qkvg'
    with pytest.raises(RuntimeError, match='Initialize the CP process group'):
        fused.FusedGemmA2AWorkspace(256, 2, 128)


@pytest.mark.parametrize('build,error,fragment', [
    (lambda: fused.FusedQKVProjection(256, 2, weight=None), TypeError, 'caller-provided'),
    (lambda: fused.FusedQKVProjection(256, 2, weight=torch.empty(768, 256, dtype=BF16), bias=[0.0]),
     TypeError, 'caller-provided'),
    (lambda: fused.FusedQKVProjection(256, 2, weight=torch.empty(768, 256, dtype=BF16), bias_in_gemm=True,
                                      apply_bias=False), ValueError, 'bias_in_gemm'),
    (lambda: fused.FusedQKVProjection(256, 2, weight=torch.empty(768, 256)), ValueError, 'weight must be'),
    (lambda: fused.FusedQKVProjection(256, 2, weight=torch.empty(1024, 256, dtype=BF16)), ValueError, 'weight must be'),
    # grouped-query attention is accepted here (the reference's fused modules reject it): 2 query heads on
    # 1 key/value head need 2 + 2 head blocks of weight rows, and the head counts must nest
    (lambda: fused.FusedQKVProjection(256, 2, 1, weight=torch.empty(768, 256, dtype=BF16)), ValueError, 'weight must be'),
    (lambda: fused.FusedQKVProjection(384, 3, 2, weight=torch.empty(896, 384, dtype=BF16)), ValueError,
     'multiple of key/value heads'),
    (lambda: fused.FusedQKVProjection(256, 4, weight=torch.empty(768, 256, dtype=BF16)), ValueError,
     'one N tile per head'),
    (lambda: fused.FusedQKVProjection(250, 4, weight=torch.empty(750, 250, dtype=BF16)), ValueError, 'divisible'),
    (lambda: fused.FusedOutputProjection(256, 2, weight=torch.empty(256, 256, dtype=BF16),
                                         bias=torch.empty(255, dtype=BF16)), ValueError, 'bias must be'),
    (lambda: fused.FusedOutputProjection(256, 2, weight=torch.empty(256, 256, dtype=BF16),
                                         bias=torch.empty(256)), ValueError, 'bias must be'),
    (lambda: fused.FusedOutputProjection(256, 0, weight=torch.empty(256, 256, dtype=BF16)), ValueError, 'divisible'),
])
def test_constructor_errors(build, error, fragment):
    with pytest.raises(error, match=fragment):
        build()


def test_wgrad_backend_variable_is_validated_like_the_reference():
    """FUSED_WGRAD_BACKEND accepts the reference's two settings (both use the accumulating
    epilogue here) and rejects anything else at import (reference fused_gemm_a2a.py:34-36)."""
    package = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'fused-gemm-a2a_b200')
    code = f'import sys; sys.path.insert(0, {package!r}); import fused_gemm_a2a as f; print(f.WGRAD_BACKEND)'
    for value, ok in (('torch', True), ('fused_accum', True), ('cublas', False)):
        run = subprocess.run([sys.executable, '-c', code], env=dict(os.environ, FUSED_WGRAD_BACKEND=value),
                             capture_output=True, text=True, timeout=300)
        if ok:
            assert run.returncode == 0 and run.stdout.strip() == value, run.stderr[-500:]
        else:
            assert run.returncode != 0 and 'FUSED_WGRAD_BACKEND must be torch or fused_accum' in run.stderr


def test_grouped_query_projection_takes_grouped_weight_rows():
    module = fused.FusedQKVProjection(512, 4, 2, weight=torch.empty((4 + 2 * 2) * 128, 512, dtype=BF16))
    assert (module.num_kv_heads, module.n_q, module.n_kv, module.segments) == (2, 512, 256, 3)
    assert module.weight_layout == 'group_qkvg' and fused.FusedQKVProjection.weight_layout == 'head_qkvg'
    gated = fused.FusedQKVProjection(512, 4, 1, gate=True, weight=torch.empty((4 * 2 + 2) * 128, 512, dtype=BF16),
                                     bias=torch.empty((4 * 2 + 2) * 128, dtype=BF16))
    assert gated.segments == 4 and gated.weight.shape[0] == 1280
    same = fused.FusedQKVProjection(512, 4, 4, weight=torch.empty(3 * 512, 512, dtype=BF16))
    assert same.weight_layout == 'head_qkvg' and same.num_kv_heads == 4
