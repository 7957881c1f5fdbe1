"""Geometry rules and kernel wrappers of the fused projection path (B200 / sm_100a build).

Same importable names as the reference module fused_gemm_a2a_kernels.py, but nothing is JIT
compiled: every wrapper validates on the host and calls libfga.so (hand-written CUDA, see csrc/)
through ctypes on the current CUDA stream. There is no CPU or PyTorch fallback.

Geometry (reference fused_gemm_a2a_kernels.py:34-123): a CTA owns 128 output rows and one arrival
counter; a CTA pair owns a 256-row MMA tile; a QKV push maps one 128-column tile to one head.
"""
import math
import os

import torch

import _fga_native as _native

CTA_M = 128                 # rows per CTA and per receive counter
MMA_N = 128                 # one N tile per head in the QKV push
MMA_N_RECV = 256            # receive GEMMs tile the output freely
MMA_N_OUT_PUSH = MMA_N      # granularity at which the output-projection dgrad is routed to peers
MMA_TILER_MN = (256, MMA_N)  # rows of a CTA pair, columns routed as one unit
CLUSTER_MN = (2, 1)
USE_2CTA = True
PUSH_SPLIT = int(os.environ.get('FUSED_PUSH_SPLIT', 0))  # 0: about 64 KB per pusher job
# The reference's other launch parameters, which its benchmark records by name (benchmark/run.py
# reads them from this module). Here they are properties of the compiled library, listed with the
# values this build uses; the FGA_* variables of include/fga.h are the knobs that exist.
CLUSTER_N = 1                # CTAs along N per cluster: no operand is ever multicast
RASTER_ALONG_M = False       # N varies fastest inside a raster group
SWIZZLE = 4                  # pair tiles per raster group of a receive GEMM (FGA_GROUP_M_RECV)
SWIZZLE_PUSH = 16            # and of a push GEMM (FGA_GROUP_M_PUSH)
PUSHER_WARPS = 4             # pusher warps per CTA during the first two raster groups
PUSHER_STEADY_WARPS = 2      # afterwards, once most traffic crosses NVLink (FGA_PUSHER_WARPS); 4 for CP <= 2
PUSHER_CHUNK = 256           # 16-byte units per pusher chunk: one 4 KiB bulk copy through shared memory
PUSHER_STREAMING = True      # transport bypasses registers and L1 (bulk copies), like the reference's evict-first stores
DEVICE_TIMEOUT_NS = int(float(os.environ.get('FGA_TIMEOUT_S', 20)) * 1e9)  # bound of device waits


# ----------------------------------------------------------------------------- pure geometry
_BARRIER_LANES = 32          # the device barrier is one warp, one lane per peer
_JOB_BYTES = 64 * 1024       # target size of one pusher job (rows of one source for one destination)
_MIN_JOB_ROWS = 4            # a pusher job never has fewer rows than this


def _reject(message):
    raise ValueError(message)


def validate_peer_count(peers):
    """The device barrier gives one lane of a single warp to every peer."""
    if peers not in range(1, _BARRIER_LANES + 1):
        _reject('The single-warp device barrier supports CP sizes from 1 to 32')


def validate_tile_n(mode, tile_n, output_width, peers, segment_width=0, num_segments=1, head_dim=0):
    """A scheduler tile may neither be truncated nor, when pushed, straddle a peer or head
    boundary. Receive traffic only permutes K, so it does not constrain the output tile
    (reference fused_gemm_a2a_kernels.py:43-59)."""
    covers_width = tile_n > 0 and output_width > 0 and output_width % tile_n == 0
    if mode not in ('push', 'recv') or not covers_width:
        _reject('GEMM mode must be push/recv and tile N must divide output width')
    if num_segments not in (1, 3, 4):
        _reject('Expected one output projection or three/four QKV projections')
    interleaved = num_segments > 1       # QKV(/gate): weight rows interleaved per head
    if interleaved and head_dim <= 0:
        _reject('QKV needs a positive head dimension')
    if mode == 'recv':
        return
    routable = peers > 0 and segment_width > 0 and segment_width % (peers * tile_n) == 0
    if not routable:
        _reject('Push segment width must be a multiple of CP * tile N')
    if interleaved and tile_n != head_dim:
        _reject('QKV push needs one N tile per head')


def mxfp8_tile_n(mode, output_width, peers=1, num_segments=1):
    """256-wide tiles only where they keep peer and head boundaries intact
    (reference fused_gemm_a2a_kernels.py:62-68)."""
    if mode == 'push' and num_segments > 1:
        return 128                      # one tile per (head, segment) unit
    span = output_width // peers if mode == 'push' else output_width
    return 256 if span % 256 == 0 else 128


def tile_swizzle(grouped_clusters, requested):
    """Raster group size that divides the cluster count exactly (no padding tiles): the gcd
    (reference fused_gemm_a2a_kernels.py:71-78)."""
    if min(grouped_clusters, requested) < 1:
        _reject('Cluster extent and FUSED_SWIZZLE must be positive')
    return math.gcd(grouped_clusters, requested)


def push_split(k, peers, segments, requested=0):
    """Row sub-blocks per (row block, destination) pusher job: jobs of roughly 64 KB, a power of
    two so the sub-blocks tile all 128 rows, at least four rows each
    (reference fused_gemm_a2a_kernels.py:81-97)."""
    sources = peers * segments
    if peers < 1 or segments < 1 or k % sources:
        _reject('Receive K must split evenly over peers and input segments')
    width = k // sources                 # BF16 columns one source contributes to a row
    if width % 64:
        _reject('The per-peer segment width must be a multiple of 64 BF16 elements')
    if requested:
        split = requested
    else:
        block_bytes = CTA_M * width * 2
        wanted = min(CTA_M // 8, block_bytes // _JOB_BYTES)
        split = 1 << (wanted.bit_length() - 1) if wanted >= 1 else 1     # round down to a power of two
    whole_blocks = split >= 1 and CTA_M % split == 0
    if not whole_blocks or (CTA_M // split) % _MIN_JOB_ROWS:
        _reject('FUSED_PUSH_SPLIT must divide 128 and leave at least four rows per job')
    return split


def padded_rows(valid, tile_m):
    """Rows a per-rank buffer holds for `valid` logical rows: rounded up to whole tiles."""
    if min(valid, tile_m) < 1:
        _reject('Token count and tile height must be positive')
    tiles = (valid + tile_m - 1) // tile_m
    return tiles * tile_m


# ----------------------------------------------------------------------------- launch helpers
def _stream():
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise ValueError('The fused kernels only run on CUDA tensors; there is no CPU path')


def device_barrier(flags, peer_flags, rank, peers, status, *, bump=False, counters=None, epoch=None):
    """Group barrier on the current stream (reference barrier, fused_gemm_a2a_kernels.py:204-234)."""
    count = 0 if counters is None else counters.numel()
    _native.check(_native.lib().fga_barrier(
        flags.data_ptr(), peer_flags.data_ptr(), rank, peers, int(bump),
        0 if counters is None else counters.data_ptr(), count,
        0 if epoch is None else epoch.data_ptr(), status.data_ptr(), DEVICE_TIMEOUT_NS, _stream()))


def resize_rank_rows(tensors, peers, rows, *, copy=False, bias=None, head_dim=128, head_offset=0,
                     use_cute=False):
    """Resize every rank's row chunk of each [peers*in_rows, width] matrix to `rows` rows: extra
    rows are zero, surplus rows dropped. Storage is fresh whenever something changes or copy=True;
    otherwise the inputs are returned. An interleaved bias (per-head [q|k|v|g] order) can be added
    on the way, in FP32 with one BF16 rounding (reference fused_gemm_a2a_kernels.py:1145-1188).
    `use_cute` is accepted for call compatibility; one CUDA kernel serves both precisions."""
    tensors = tuple(tensors)
    first = tensors[0]
    if peers < 1 or rows < 1 or first.shape[0] % peers:
        raise ValueError('Positive row counts must split evenly across peers')
    if first.ndim != 2 or not first.is_cuda:
        raise ValueError('Rank copies require CUDA matrices')
    for t in tensors:
        if t.shape != first.shape or t.dtype != first.dtype or t.device != first.device or not t.is_contiguous():
            raise ValueError('Rank copies require matching contiguous tensors')
    if first.dtype != torch.bfloat16:
        raise ValueError('Rank copies require BF16 matrices')
    if len(tensors) > 4:
        raise ValueError('At most four segments are copied per call')
    in_rows, width = first.shape[0] // peers, first.shape[1]
    if bias is not None:
        covered = (head_offset * head_dim + width) * len(tensors)
        if (head_dim < 1 or width % head_dim or head_offset < 0 or bias.ndim != 1
                or not bias.is_contiguous() or bias.device != first.device
                or bias.dtype != first.dtype or bias.numel() < covered):
            raise ValueError('Bias must cover the interleaved heads being copied')
    if in_rows == rows and bias is None and not copy:
        return tensors
    outputs = tuple(torch.empty((peers * rows, width), device=first.device, dtype=first.dtype)
                    for _ in tensors)
    _native.check(_native.lib().fga_copy_rank_rows(
        _native.ptr_array([t.data_ptr() for t in tensors]),
        _native.ptr_array([t.data_ptr() for t in outputs]), len(tensors), peers, in_rows, rows,
        width, 0 if bias is None else bias.data_ptr(), head_dim, head_offset, _stream()))
    return outputs


def reduce_bias_grad(dy, out, *, accumulate=False, use_cute=False):
    """out[c] (=|+=) sum over rows of dy[:, c], summed in FP32 and rounded once
    (reference fused_gemm_a2a_kernels.py:1086-1103)."""
    if dy.ndim != 2:
        raise ValueError('Bias reduction requires contiguous BF16 rows and a BF16/FP32 output vector')
    rows, width = dy.shape
    if (rows < 1 or not dy.is_cuda or not dy.is_contiguous() or dy.dtype != torch.bfloat16
            or tuple(out.shape) != (width,) or out.device != dy.device or not out.is_contiguous()
            or out.dtype not in (torch.bfloat16, torch.float32)):
        raise ValueError('Bias reduction requires contiguous BF16 rows and a BF16/FP32 output vector')
    lib = _native.lib()
    scratch = torch.empty(lib.fga_bias_grad_scratch_floats(rows, width), device=dy.device,
                          dtype=torch.float32)
    _native.check(lib.fga_bias_grad(dy.data_ptr(), rows, width, out.data_ptr(),
                                    int(out.dtype == torch.float32), int(accumulate),
                                    scratch.data_ptr(), _stream()))
    return out


def mxfp8_quantize(a, *, k_multiple=256):
    """BF16 [rows, k] -> (E4M3 [pad256(rows), pad(k)], E8M0 scale bytes in the tcgen05 128x4
    layout), one scale per 32 elements along k. A transposed view (stride(0) == 1) is quantized
    along its strided axis without materializing the transpose
    (reference fused_gemm_a2a_kernels.py:1358-1376)."""
    if a.ndim != 2 or a.dtype != torch.bfloat16:
        raise ValueError('MXFP8 quantization requires a BF16 matrix')
    _require_cuda(a)
    transposed = a.stride(0) == 1 and a.stride(1) != 1
    minor, major = (a.stride(0), a.stride(1)) if transposed else (a.stride(1), a.stride(0))
    if minor != 1 or major % 8 or a.data_ptr() % 16:
        raise ValueError('MXFP8 quantization requires 16-byte aligned rows or columns')
    rows, k = a.shape
    rp, kp = padded_rows(rows, MMA_TILER_MN[0]), padded_rows(k, k_multiple)
    q = torch.empty((rp, kp), device=a.device, dtype=torch.float8_e4m3fn)
    sf = torch.empty((rp * kp // 32,), device=a.device, dtype=torch.uint8)
    _native.check(_native.lib().fga_mx_quantize(a.data_ptr(), rows, k, a.stride(0), a.stride(1),
                                                q.data_ptr(), sf.data_ptr(), rp, kp, _stream()))
    return q, sf


def bf16_wgrad(dy, x, out, status, *, accumulate=False):
    """out[N_out, K] (=|+=) dy[tokens, N_out]^T x[tokens, K] on the tensor cores; FP32 outputs may
    accumulate in place (Megatron main_grad), BF16 outputs are stored. Replaces the reference's
    cuBLAS call plus separate add (fused_gemm_a2a.py:264-275)."""
    tokens, n_out = dy.shape
    if x.shape[0] != tokens or tuple(out.shape) != (n_out, x.shape[1]):
        raise ValueError('Weight gradient shapes must be dy [T, N], x [T, K], out [N, K]')
    if dy.stride(1) != 1 or x.stride(1) != 1 or not out.is_contiguous():
        raise ValueError('Weight gradient operands need unit inner strides')
    if out.dtype not in (torch.bfloat16, torch.float32) or (accumulate and out.dtype != torch.float32):
        raise ValueError('Gradient accumulation requires FP32 output')
    _native.check(_native.lib().fga_gemm_local(
        dy.data_ptr(), 1, x.data_ptr(), 1, n_out, x.shape[1], tokens, dy.stride(0), x.stride(0),
        out.data_ptr(), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
        status.data_ptr(), DEVICE_TIMEOUT_NS, _stream()))
    return out


_local_status = {}


def _status_word(device):
    """A per-device status word for kernels launched outside a CP group (bounded-wait reports)."""
    word = _local_status.get(device)
    if word is None:
        word = _local_status[device] = torch.zeros(4, dtype=torch.int32, device=device)
    return word


def mxfp8_gemm(a, sa, b, sb, out, m, n, status, *, accumulate=False):
    """out[m, n] (=|+=) dequant(a) @ dequant(b)^T for operands produced by mxfp8_quantize (same
    padded K); block-scaled tcgen05 MMAs with FP32 accumulation."""
    if a.shape[1] != b.shape[1]:
        raise ValueError('MXFP8 operands must be quantized over the same padded K')
    _native.check(_native.lib().fga_gemm_local_mx(
        a.data_ptr(), sa.data_ptr(), a.shape[0], b.data_ptr(), sb.data_ptr(), b.shape[0], m, n, a.shape[1],
        out.data_ptr(), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
        status.data_ptr(), DEVICE_TIMEOUT_NS, _stream()))
    return out


def mxfp8_wgrad(dy, x, out, *, accumulate=False, status=None):
    """MXFP8 weight gradient out[N_out, K] (=|+=) dy[T, N_out]^T x[T, K]: both operands are
    requantized from BF16 along the token axis (the new reduction axis; FP8 payloads are never
    transposed) and multiplied by the block-scaled GEMM; FP32 outputs may accumulate in place
    (reference fused_gemm_a2a_kernels.py:1398-1421). `status` is the device status word that a
    bounded wait reports to; without one a per-device word is used, which _Comm.check_status() and
    clear_status() of any group on that device also cover. Returns the object that stands for the
    launched kernel (see _InlinePtx below), as the reference does."""
    if accumulate and out.dtype != torch.float32:
        raise ValueError('MXFP8 gradient accumulation requires FP32 output')
    if out.dtype not in (torch.bfloat16, torch.float32) or not out.is_contiguous():
        raise ValueError('MXFP8 weight gradient needs a contiguous BF16 or FP32 output')
    dq, ds = mxfp8_quantize(dy.T)
    xq, xs = mxfp8_quantize(x.T)
    mxfp8_gemm(dq, ds, xq, xs, out, out.shape[0], out.shape[1],
               _status_word(out.device) if status is None else status, accumulate=accumulate)
    # The reference returns the kernel it launched, and its acceptance driver reads that object's
    # `__ptx__` (tests/mxfp8_driver.py:239-244 of the reference); the result itself is in `out`.
    return _native_mxfp8_kernels[0] if _native_mxfp8_kernels else None


class _InlinePtx:
    """Stands where the reference keeps its JIT-compiled MXFP8 kernels, whose PTX text its benchmark
    and driver search for `tcgen05.mma` and `block_scale` (benchmark/run.py:366-371). Nothing is
    compiled at run time here: `__ptx__` is the text of the inline-PTX wrappers that libfga.so is
    built from, which hold the block-scaled MMA the MXFP8 kernels issue."""

    def __init__(self, path):
        with open(path) as source:
            self.__ptx__ = source.read()


_PTX_SOURCE = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'csrc', 'ptx.cuh')
_native_mxfp8_kernels = [_InlinePtx(_PTX_SOURCE)] if os.path.exists(_PTX_SOURCE) else []
