"""CPU restatement of the reference's MXFP8 quantizer (E4M3 payload, one E8M0 scale per 32).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and bench.py's CPU baseline, never
by the library.

The reference quantizer is a GPU-only CuTe-DSL kernel, so this file restates its arithmetic in
numpy integer/float32 operations, function by function:

  mx_scale        <- _mx_scale           (fused_gemm_a2a_kernels.py:1200-1219)
  scale_offset    <- _mx_scale_offset    (fused_gemm_a2a_kernels.py:1195-1197, 1283)
  quantize        <- _mx_quant_kernel + mxfp8_quantize padding rules
                                          (fused_gemm_a2a_kernels.py:1222-1292, 1358-1368)
  e4m3_encode     <- the float32 -> float8_e4m3fn conversion (round to nearest even, finite
                     saturation at 448, NaN -> NaN); the OCP FP8 E4M3 format, restated here from its
                     published definition: 1 sign, 4 exponent bits (bias 7), 3 mantissa bits,
                     no infinities, S.1111.111 is NaN, largest finite 448.

Parity pin: the reference's tests only hold known answers for this path, no golden tensors; the
pins reproduced in tests/test_oracle_mxfp8.py are
  - a group containing +-Inf gets scale byte 255, its Inf elements a NaN payload and its finite
    elements a finite payload, at scale offsets [0, 16, 33] for non-finite inputs at (0,0), (1,31),
    (2,32) of a [128, 33] source (tests/mxfp8_local_driver.py:63-77),
  - an all-zero group gets scale byte 127 and zero payload,
  - every finite BF16 magnitude 0x0000..0x7f7f in a constant-magnitude group, both signs,
    dequantizes within E4M3 precision (tests/mxfp8_driver.py:184-204),
and e4m3_encode is additionally checked against torch's CPU float8_e4m3fn cast on all inputs that
do not saturate. The scale chosen for a group that holds NaN but no Inf is not pinned by any
reference test ("parity unpinned" for that single case): this oracle lets NaN elements not raise
the group maximum, which is what a max.f32-style reduction does.
"""
import numpy as np

E4M3_MAX = 448.0


def bf16_to_f32(bits16):
    """uint16 BF16 bit patterns -> float32."""
    return (np.asarray(bits16, dtype=np.uint32) << 16).view(np.float32)


def _e4m3_table():
    codes = np.arange(127, dtype=np.uint8)  # non-negative finite codes 0x00..0x7e
    exp = (codes >> 3).astype(np.int32)
    man = (codes & 7).astype(np.float64)
    values = np.where(exp == 0, man / 8.0 * 2.0 ** -6, (1.0 + man / 8.0) * 2.0 ** (exp - 7))
    return values


_E4M3_VALUES = _e4m3_table()
_E4M3_MID = (_E4M3_VALUES[:-1] + _E4M3_VALUES[1:]) / 2.0


def e4m3_encode(x):
    """float32 array -> uint8 E4M3 codes: round to nearest, ties to the even code, magnitudes above
    448 saturate to 448 (finite saturation), NaN -> 0x7f with the sign bit kept."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x.astype(np.float64))
    sign = (x.view(np.uint32) >> 24).astype(np.uint8) & 0x80
    finite = np.minimum(mag, E4M3_MAX)
    finite = np.where(np.isnan(finite), 0.0, finite)
    idx = np.searchsorted(_E4M3_MID, finite, side='left')  # first midpoint >= value
    # value == midpoint: tie between code idx and idx+1 -> choose the even one
    on_tie = (idx < _E4M3_MID.size) & (finite == _E4M3_MID[np.minimum(idx, _E4M3_MID.size - 1)])
    code = np.where(on_tie & (idx % 2 == 1), idx + 1, idx).astype(np.uint8)
    code = np.where(np.isnan(x), np.uint8(0x7f), code)
    return (code | sign).astype(np.uint8)


def e4m3_decode(codes):
    """uint8 E4M3 codes -> float32 (NaN for S.1111.111)."""
    codes = np.asarray(codes, dtype=np.uint8)
    mag = codes & 0x7f
    vals = np.where(mag == 0x7f, np.nan, _E4M3_VALUES[np.minimum(mag, 126)])
    return np.where(codes & 0x80, -vals, vals).astype(np.float32)


def mx_scale(peak):
    """Group maximum (float32, >= 0 or +Inf) -> (E8M0 exponent e, float32 multiplier 2**-e).
    e = ceil(log2(peak / 448)) computed from the float32 exponent and mantissa (448 = 1.75 * 2**8,
    mantissa 0x600000), clamped to [-126, 127]; zero -> e = 0; +Inf -> e = 128 (byte 255, the E8M0
    NaN) with multiplier 0."""
    peak = np.asarray(peak, dtype=np.float32)
    bits = peak.view(np.uint32).astype(np.int64)
    e = (bits >> 23) - 135
    e = e + ((bits & 0x7fffff) > 0x600000)
    e = np.clip(e, -126, 127)
    e = np.where(peak > 0, e, 0)
    inv = ((127 - e).astype(np.uint32) << 23).view(np.float32)
    is_inf = np.isposinf(peak)
    e = np.where(is_inf, 128, e)
    inv = np.where(is_inf, np.float32(0), inv).astype(np.float32)
    return e.astype(np.int32), inv


def scale_offset(row, group, groups):
    """Byte offset of the scale of (row, 32-group) in the tcgen05 128-row x 4-group layout."""
    row, group = np.asarray(row, dtype=np.int64), np.asarray(group, dtype=np.int64)
    return (((row // 128) * (groups // 4) + group // 4) * 512 + (row % 32) * 16
            + (row % 128 // 32) * 4 + group % 4)


def padded(value, multiple):
    return -(-value // multiple) * multiple


def quantize(a_bits, k_multiple=256, row_multiple=256):
    """a_bits: uint16 [rows, k] BF16 bit patterns (the logical matrix, already in the orientation
    whose second axis is quantized). Returns (q uint8 [rp, kp], sf uint8 [rp*kp/32]); padding rows
    and columns are quantized as zeros (payload 0, scale byte 127)."""
    a_bits = np.asarray(a_bits, dtype=np.uint16)
    rows, k = a_bits.shape
    rp, kp = padded(rows, row_multiple), padded(k, k_multiple)
    if rp % 128 or kp % 128:
        raise ValueError('the scale layout needs padded extents in multiples of 128')
    vals = np.zeros((rp, kp), dtype=np.float32)
    vals[:rows, :k] = bf16_to_f32(a_bits)
    groups = kp // 32
    g = vals.reshape(rp, groups, 32)
    with np.errstate(invalid='ignore'):
        peak = np.fmax.reduce(np.abs(g), axis=2, initial=np.float32(0))  # fmax drops NaN
    e, inv = mx_scale(peak)
    with np.errstate(invalid='ignore', over='ignore'):
        scaled = (g * inv[:, :, None]).astype(np.float32)  # Inf * 0 = NaN, finite * 0 = 0
    q = e4m3_encode(scaled).reshape(rp, kp)
    sf = np.zeros(rp * groups, dtype=np.uint8)
    r, c = np.meshgrid(np.arange(rp), np.arange(groups), indexing='ij')
    sf[scale_offset(r, c, groups)] = (e + 127).astype(np.uint8)
    return q, sf


def unswizzle_scales(sf, rp, kp):
    """Scale bytes in the tcgen05 layout -> plain [rp, kp/32] matrix."""
    groups = kp // 32
    r, c = np.meshgrid(np.arange(rp), np.arange(groups), indexing='ij')
    return np.asarray(sf, dtype=np.uint8)[scale_offset(r, c, groups)]


def dequantize(q, sf, rp, kp):
    """(payload, swizzled scales) -> float64 matrix [rp, kp]; scale byte 255 gives NaN."""
    s = unswizzle_scales(sf, rp, kp).astype(np.int32)
    scale = np.where(s == 255, np.nan, np.ldexp(1.0, s - 127))
    return e4m3_decode(q).astype(np.float64).reshape(rp, kp // 32, 32) * scale[:, :, None]


def mx_matmul(a_bits, b_bits):
    """Reference value of the block-scaled GEMM a [M, K] x b [N, K]^T: quantize both along K,
    dequantize exactly, multiply in float64."""
    qa, sa = quantize(a_bits)
    qb, sb = quantize(b_bits)
    da = dequantize(qa, sa, *qa.shape).reshape(qa.shape)
    db = dequantize(qb, sb, *qb.shape).reshape(qb.shape)
    return (da @ db.T)[:a_bits.shape[0], :b_bits.shape[0]]
