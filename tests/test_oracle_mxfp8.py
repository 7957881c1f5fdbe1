"""Known answers that pin the CPU restatement of the MXFP8 quantizer (oracle/mxfp8_oracle.py)."""
import numpy as np
import torch

from oracle import mxfp8_oracle as mx


def bits_of(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def test_e4m3_encode_matches_torch_cast_on_all_bf16_inputs_below_saturation():
    """Every finite BF16 value with |v| <= 448 and both signs: round to nearest even onto E4M3."""
    codes = np.arange(0x8000, dtype=np.uint16)
    vals = mx.bf16_to_f32(codes)
    keep = np.isfinite(vals) & (np.abs(vals) <= 448)
    for sign in (1.0, -1.0):
        v = (vals[keep] * sign).astype(np.float32)
        want = torch.from_numpy(v).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        got = mx.e4m3_encode(v)
        zero = v == 0
        assert np.array_equal(got[~zero], want[~zero])
        assert np.all((got[zero] & 0x7f) == 0)


def test_e4m3_saturates_and_keeps_nan():
    got = mx.e4m3_encode(np.array([448, 449, 464, 480, 1e9, -1e9, np.nan], dtype=np.float32))
    assert got[:5].tolist() == [0x7e] * 5 and got[5] == 0xfe and (got[6] & 0x7f) == 0x7f
    dec = mx.e4m3_decode(np.arange(256, dtype=np.uint8))
    assert dec[0x7e] == 448 and np.isnan(dec[0x7f]) and dec[0x01] == 2.0 ** -9 and dec[0x88] == -2.0 ** -6


def test_scale_rule():
    peaks = np.array([0, 448, 448.0001, 1, 1.75, 1.76, 2.0 ** -140, 3.0e38, np.inf], dtype=np.float32)
    e, inv = mx.mx_scale(peaks)
    # 448 = 1.75 * 2^8 fits exactly at e=0; just above needs e=1; 1.75 -> 2^-8; above -> 2^-7
    assert e.tolist() == [0, 0, 1, -8, -8, -7, -126, 120, 128]
    assert inv[0] == 1 and inv[3] == 256 and inv[-1] == 0 and inv[6] == 2.0 ** 126
    # the scaled maximum never exceeds 448
    rng = np.random.default_rng(0)
    p = np.abs(rng.standard_normal(10000).astype(np.float32)) * np.float32(10.0) ** rng.integers(-30, 30, 10000).astype(np.float32)
    e, inv = mx.mx_scale(p)
    assert np.all(p * inv <= 448) and np.all((p * inv > 224) | (e == -126))


def test_scale_layout_offsets():
    """128-row x 4-group tiles of 512 bytes, 16 bytes per row-of-32 and 4 per 32-row slab."""
    assert mx.scale_offset(0, 0, 8) == 0 and mx.scale_offset(1, 0, 8) == 16 and mx.scale_offset(2, 1, 8) == 33
    assert mx.scale_offset(32, 0, 8) == 4 and mx.scale_offset(0, 4, 8) == 512 and mx.scale_offset(128, 0, 8) == 1024
    rows, groups = 256, 8
    r, c = np.meshgrid(np.arange(rows), np.arange(groups), indexing='ij')
    assert sorted(mx.scale_offset(r, c, groups).reshape(-1).tolist()) == list(range(rows * groups))


def test_inf_groups_known_answer():
    """Reference tests/mxfp8_local_driver.py:63-77: [128, 33] source, non-finite at (0,0), (1,31),
    (2,32): scale byte 255 exactly at offsets [0, 16, 33]; NaN payload only at those elements."""
    a = torch.ones(128, 33)
    a[0, 0], a[1, 31], a[2, 32] = float('inf'), float('-inf'), float('inf')
    q, sf = mx.quantize(bits_of(a))
    assert q.shape == (256, 256) and sf.shape == (256 * 8,)
    assert np.nonzero(sf == 255)[0].tolist() == [0, 16, 33]
    nan = (q & 0x7f) == 0x7f
    assert sorted(zip(*np.nonzero(nan))) == [(0, 0), (1, 31), (2, 32)]
    assert np.all(q[0, 1:32] == 0)           # finite members of an Inf group become 0
    assert q[3, 0] == mx.e4m3_encode(np.float32(1.0) * np.float32(256))  # ordinary group of ones: e = -8


def test_zero_groups_and_padding():
    a = torch.randn(5, 70)
    a[2, 32:64] = 0
    q, sf = mx.quantize(bits_of(a), k_multiple=128)
    assert q.shape == (256, 128)
    plain = mx.unswizzle_scales(sf, 256, 128)
    assert plain[2, 1] == 127 and not q[2, 32:64].any()
    assert np.all(plain[5:] == 127) and not q[5:].any() and not q[:, 70:].any() and np.all(plain[:, 3] == 127)


def test_exhaustive_constant_magnitude_groups():
    """Reference tests/mxfp8_driver.py:184-204: every finite BF16 magnitude, both signs, in a
    constant-magnitude group dequantizes back within E4M3 precision (2^-4 relative), exactly for
    values E4M3 can hold after scaling."""
    mags = np.arange(0x7f80, dtype=np.uint16)
    for sign in (0, 0x8000):
        a = np.repeat((mags | sign)[:, None], 32, axis=1)
        q, sf = mx.quantize(a, k_multiple=128, row_multiple=128)
        back = mx.dequantize(q, sf, *q.shape).reshape(q.shape)[:mags.size, :32]
        want = mx.bf16_to_f32(a).astype(np.float64)
        tiny = np.abs(want) < 2.0 ** -126 * 2.0 ** -9   # below the smallest scaled E4M3 step
        err = np.abs(back - want)
        assert np.all(err[~tiny] <= np.abs(want[~tiny]) * 2.0 ** -4 + 2.0 ** -136)
        assert np.all(np.sign(back[~tiny]) == np.sign(want[~tiny]))


def test_nan_does_not_raise_the_group_scale():
    a = torch.ones(1, 32)
    a[0, 3] = float('nan')
    q, sf = mx.quantize(bits_of(a), k_multiple=128, row_multiple=128)
    assert sf[0] == 127 - 8 and (q[0, 3] & 0x7f) == 0x7f and q[0, 0] == q[0, 31] != 0


def test_block_scaled_matmul_is_close_to_exact():
    rng = torch.Generator().manual_seed(3)
    a, b = torch.randn(48, 256, generator=rng), torch.randn(40, 256, generator=rng)
    got = mx.mx_matmul(bits_of(a), bits_of(b))
    want = a.to(torch.bfloat16).double() @ b.to(torch.bfloat16).double().t()
    rel = np.linalg.norm(got - want.numpy()) / np.linalg.norm(want.numpy())
    assert rel < 0.05
