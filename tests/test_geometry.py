"""Host-side geometry rules of the fused kernels (no GPU): the values and error messages the
reference pins in tests/test_recv_plan.py and tests/test_row_blocks.py, checked on this build's
fused_gemm_a2a_kernels / fused_gemm_a2a modules."""
from unittest.mock import patch

import pytest
import torch

import fused_gemm_a2a as fused
from fused_gemm_a2a_kernels import (CTA_M, MMA_TILER_MN, mxfp8_tile_n, padded_rows, push_split,
                                    tile_swizzle, validate_peer_count, validate_tile_n)


def test_peer_limit_of_the_single_warp_barrier():
    for peers in (1, 4, 8, 16, 32):
        validate_peer_count(peers)
    for peers in (0, -1, 33, 64):
        with pytest.raises(ValueError, match='single-warp'):
            validate_peer_count(peers)


def test_tile_rules():
    validate_tile_n('recv', 256, 4096, 16, num_segments=4, head_dim=128)
    validate_tile_n('push', 128, 16384, 16, 4096, 4, 128)
    with pytest.raises(ValueError, match='one N tile per head'):
        validate_tile_n('push', 256, 16384, 16, 4096, 4, 128)
    validate_tile_n('push', 256, 4096, 16, 4096)
    with pytest.raises(ValueError, match=r'CP \* tile N'):
        validate_tile_n('push', 256, 4096, 32, 4096)
    validate_tile_n('push', 128, 4096, 32, 4096)
    for width in (4095, 4097):
        with pytest.raises(ValueError):
            validate_tile_n('recv', 256, width, 16)
    for tile in (0, -128):
        with pytest.raises(ValueError):
            validate_tile_n('recv', tile, 4096, 16)
    with pytest.raises(ValueError):
        validate_tile_n('local', 128, 4096, 1)
    with pytest.raises(ValueError, match='three/four'):
        validate_tile_n('recv', 128, 4096, 1, num_segments=2)


def test_mxfp8_tile_selection():
    for peers in (1, 2, 4, 8, 16, 32):
        for heads_per_peer in (1, 2, 3, 4):
            hidden = peers * heads_per_peer * 128
            for segments in (1, 3, 4):
                tile = mxfp8_tile_n('push', hidden * segments, peers, segments)
                validate_tile_n('push', tile, hidden * segments, peers, hidden, segments, 128)
            validate_tile_n('recv', mxfp8_tile_n('recv', hidden, peers), hidden, peers)
            assert hidden % mxfp8_tile_n('local', hidden) == 0
    assert mxfp8_tile_n('push', 4096, 16) == 256
    assert mxfp8_tile_n('push', 4096, 32) == 128
    assert mxfp8_tile_n('local', 384) == 128


def test_swizzle_never_pads():
    for clusters in range(1, 129):
        for requested in (1, 2, 3, 4, 8, 16):
            s = tile_swizzle(clusters, requested)
            assert clusters % s == 0 and s <= requested
    assert (tile_swizzle(32, 8), tile_swizzle(4, 8), tile_swizzle(6, 8)) == (8, 4, 2)
    for args in ((0, 8), (4, 0), (4, -1)):
        with pytest.raises(ValueError):
            tile_swizzle(*args)


def test_push_split():
    for width in range(64, 8193, 64):
        for segments in (1, 3):
            split = push_split(width * 4 * segments, 4, segments)
            rows = CTA_M // split
            assert rows * split == CTA_M and rows % 4 == 0
    assert push_split(4096, 16, 1) == 1
    assert push_split(12288, 16, 3) == 1
    assert push_split(12288, 4, 3) == 4
    assert push_split(4096, 16, 1, requested=8) == 8
    for requested in (-1, 3, 6, 17, 64, 129):
        with pytest.raises(ValueError):
            push_split(4096, 16, 1, requested)
    for args in ((4096, 0, 1), (4000, 16, 1), (32 * 16, 16, 1)):
        with pytest.raises(ValueError):
            push_split(*args)


def test_padded_rows():
    assert padded_rows(7456, 256) == 7680 and padded_rows(7456, 128) == 7552
    assert padded_rows(8192, 256) == 8192 and padded_rows(1, 256) == 256
    for args in ((0, 256), (7456, 0), (-1, 128)):
        with pytest.raises(ValueError):
            padded_rows(*args)
    assert MMA_TILER_MN == (256, 128) and fused.MMA_TILER_MN == MMA_TILER_MN


class TestMxfp8MainGrad:
    """main_grad validation happens before any kernel is touched
    (reference tests/test_recv_plan.py:94-123)."""

    def setup_method(self):
        self.weight = torch.nn.Parameter(torch.empty(384, 128, dtype=torch.bfloat16))
        self.dy = torch.empty(33, 384, dtype=torch.bfloat16)
        self.x = torch.empty(33, 128, dtype=torch.bfloat16)

    def reject(self, buffer):
        self.weight.main_grad = buffer
        with patch.object(fused, 'mxfp8_wgrad') as gemm:
            with pytest.raises(ValueError, match='main_grad'):
                fused._weight_grad(self.weight, self.dy, self.x, 'mxfp8')
            gemm.assert_not_called()

    def test_wrong_shape(self):
        for shape in ((128, 128), (384, 256), (384 * 128,)):
            self.reject(torch.empty(shape, dtype=torch.float32))

    def test_wrong_device(self):
        self.reject(torch.empty(self.weight.shape, device='meta', dtype=torch.float32))

    def test_misaligned_view(self):
        buffer = torch.empty(self.weight.numel() + 1, dtype=torch.float32)[1:].view(self.weight.shape)
        assert buffer.is_contiguous() and buffer.data_ptr() % 16
        self.reject(buffer)

    def test_dtype_and_strides(self):
        self.reject(torch.empty_like(self.weight))
        self.reject(torch.empty(128, 384, dtype=torch.float32).T)


def test_module_construction_needs_no_process_group_or_gpu_work():
    """Modules validate on the host only; the workspace is what touches the process group
    (reference tests/variable_length_driver.py:36-47)."""
    with patch.object(fused._Comm, 'get', side_effect=AssertionError('eager communication setup')):
        fused.FusedQKVProjection(256, 2, weight=torch.empty(768, 256, dtype=torch.bfloat16))
        fused.FusedOutputProjection(256, 2, weight=torch.empty(256, 256, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match='Initialize the CP process group'):
        fused.FusedGemmA2AWorkspace(256, 2, 128)
    with pytest.raises(TypeError):
        fused.FusedQKVProjection(256, 2, weight=None)
    with pytest.raises(ValueError, match='bias_in_gemm'):
        fused.FusedQKVProjection(256, 2, weight=torch.empty(768, 256, dtype=torch.bfloat16),
                                 bias_in_gemm=True, apply_bias=False)
    with pytest.raises(ValueError, match='weight must be'):
        fused.FusedQKVProjection(256, 2, weight=torch.empty(768, 256))
    with pytest.raises(ValueError, match='bias must be'):
        fused.FusedOutputProjection(256, 2, weight=torch.empty(256, 256, dtype=torch.bfloat16),
                                    bias=torch.empty(255, dtype=torch.bfloat16))
    assert fused.FusedQKVProjection.weight_layout == 'head_qkvg'


def test_wgrad_backend_variable_is_validated_like_the_reference():
    """FUSED_WGRAD_BACKEND accepts the reference's two settings (both use the accumulating
    epilogue here) and rejects anything else at import (reference fused_gemm_a2a.py:34-36)."""
    import os
    import subprocess
    import sys
    package = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'fused-gemm-a2a_b200')
    code = f'import sys; sys.path.insert(0, {package!r}); import fused_gemm_a2a as f; print(f.WGRAD_BACKEND)'
    for value, ok in (('torch', True), ('fused_accum', True), ('cublas', False)):
        run = subprocess.run([sys.executable, '-c', code], env=dict(os.environ, FUSED_WGRAD_BACKEND=value),
                             capture_output=True, text=True, timeout=300)
        if ok:
            assert run.returncode == 0 and run.stdout.strip() == value, run.stderr[-500:]
        else:
            assert run.returncode != 0 and 'FUSED_WGRAD_BACKEND must be torch or fused_accum' in run.stderr
