"""The kernel's index arithmetic on the CPU. csrc/schedule.cuh holds the integer functions that the
CUDA kernel, its launchers and nothing else use to decide which tile a CTA pair computes, which K
steps a work unit covers, where a finished head tile goes on which peer, and which rows a pusher
job moves. tests/native/schedule_host.cpp compiles the same header with g++; here every function is
checked for the properties the kernel depends on (each tile, K step, job and byte exactly once; a
persistent grid's stride schedule; both pusher schedules) and the routing is compared with the
oracle's buffer layouts, for the benchmark geometries and a sweep of small ones.
"""
import ctypes
import itertools
import os
import subprocess

import pytest
import torch

from oracle import mxfp8_oracle
from oracle.ulysses_oracle import GroupedQueryOracle, UlyssesOracle

HERE = os.path.dirname(os.path.abspath(__file__))
I = ctypes.c_int
L = ctypes.c_longlong


@pytest.fixture(scope='module')
def sched(tmp_path_factory):
    out = tmp_path_factory.mktemp('sched') / 'libsched.so'
    subprocess.run(['g++', '-O1', '-std=c++17', '-shared', '-fPIC', '-Wall', '-Werror', '-x', 'c++',
                    os.path.join(HERE, 'native', 'schedule_host.cpp'), '-o', str(out)], check=True)
    lib = ctypes.CDLL(str(out))
    for name in ('sched_push_element', 'sched_push_jobs_total', 'sched_first_phase_jobs', 'sched_recv_column',
                 'sched_push_element_grouped', 'sched_recv_column_grouped'):
        getattr(lib, name).restype = L
    lib.sched_push_element_grouped.argtypes = [I, I, I, I, I, I, L, I]
    lib.sched_push_element.argtypes = [I, I, I, I, L, I, L]
    lib.sched_decode_push_job.argtypes = [L, I, I, I, I, ctypes.POINTER(I)]
    lib.sched_pick_k_splits.argtypes = [L, I, I, I]
    lib.rule_mx_scale_offset.restype = L
    lib.rule_mx_scale_offset.argtypes = [L, I, I]
    return lib


def tile_of(lib, m_tiles, n_tiles, group_m, t):
    m, n = I(), I()
    lib.sched_tile_coords(m_tiles, n_tiles, group_m, t, ctypes.byref(m), ctypes.byref(n))
    return m.value, n.value


def unit_of(lib, k_tiles, k_splits, total, u):
    t, a, b = I(), I(), I()
    lib.sched_unit_coords(k_tiles, k_splits, total, u, ctypes.byref(t), ctypes.byref(a), ctypes.byref(b))
    return t.value, a.value, b.value


def job_of(lib, job, num_in, p, split, rank):
    out = (I * 5)()
    lib.sched_decode_push_job(job, num_in, p, split, rank, out)
    return tuple(out)     # mi, t, d, q, row0


def chunking(lib, hpr, sub_rows, buffer_bytes=4096):
    units, rows = I(), I()
    lib.sched_push_chunking(hpr, sub_rows, buffer_bytes, ctypes.byref(units), ctypes.byref(rows))
    return units.value, rows.value


# ------------------------------------------------------------------------------------ tiles
@pytest.mark.parametrize('m_tiles,n_tiles,group_m', [(64, 48, 16), (64, 16, 4), (48, 16, 8), (16, 16, 8), (512, 48, 16),
                                                     (1, 1, 4), (5, 3, 4), (7, 2, 3), (9, 5, 1), (3, 7, 16)])
def test_raster_visits_every_tile_once_and_groups_rows(sched, m_tiles, n_tiles, group_m):
    total = m_tiles * n_tiles
    seen = [tile_of(sched, m_tiles, n_tiles, group_m, t) for t in range(total)]
    assert sorted(seen) == sorted(itertools.product(range(m_tiles), range(n_tiles)))
    # a raster group never mixes row tiles of different groups, and group g comes before g + 1
    groups = [m // group_m for m, _ in seen]
    assert groups == sorted(groups)
    # inside a group the row tile varies fastest: consecutive tiles share the weight tile
    first_group = [pair for pair in seen if pair[0] < group_m]
    rows = min(group_m, m_tiles)
    assert first_group[:rows] == [(m, 0) for m in range(rows)]


@pytest.mark.parametrize('pairs', [1, 7, 71, 74])
@pytest.mark.parametrize('total,k_tiles,k_splits', [(256, 256, 1), (256, 2048, 2), (768, 2048, 2), (10, 257, 8),
                                                    (3, 64, 2), (1, 96, 3)])
def test_units_cover_every_k_step_of_every_tile_once(sched, pairs, total, k_tiles, k_splits):
    """The persistent grid's stride schedule (pair, pair + pairs, ...) over tiles x shares: each
    (tile, K step) belongs to exactly one unit, shares are contiguous, balanced and never empty."""
    covered = {}
    for pair in range(pairs):
        for u in range(pair, total * k_splits, pairs):
            t, kt0, kt1 = unit_of(sched, k_tiles, k_splits, total, u)
            assert 0 <= t < total and 0 <= kt0 < kt1 <= k_tiles
            assert abs((kt1 - kt0) - k_tiles / k_splits) < 1
            for kt in range(kt0, kt1):
                assert covered.setdefault((t, kt), u) == u
    assert len(covered) == total * k_tiles


def test_rotation_is_a_permutation_that_starts_ranks_on_different_peers(sched):
    for n_tiles, p in ((48, 8), (16, 8), (16, 2), (12, 4), (3, 1)):
        for rank in range(p):
            rotate = rank * (n_tiles // p)
            order = [sched.sched_rotated_n(n, rotate, n_tiles) for n in range(n_tiles)]
            assert sorted(order) == list(range(n_tiles)) and order[0] == rotate


def test_share_count_selection(sched):
    pick = sched.sched_pick_k_splits
    assert pick(256, 2048, 74, 0) == 2      # 4096x4096 gradient over 131072 tokens: 3.46 waves -> 6.92
    assert pick(768, 2048, 74, 0) == 2      # 12288x4096: 10.4 waves -> 20.8
    assert pick(3072, 64, 74, 0) == 1       # already 98.8 % efficient
    assert pick(256, 63, 74, 0) == 1        # a share must keep 32 K steps
    assert pick(1, 256, 74, 0) == 8         # a single tile: as many shares as allowed
    assert pick(256, 2048, 74, 4) == 4 and pick(256, 100, 74, 4) == 3 and pick(256, 40, 74, 4) == 1
    for tiles, k_tiles in itertools.product((1, 5, 74, 75, 256, 768, 1000), (32, 64, 100, 256, 4096)):
        s = pick(tiles, k_tiles, 74, 0)
        assert 1 <= s <= 8 and (s == 1 or k_tiles // s >= 32)


# ------------------------------------------------------------------------------------ push routing
class _CodedOracle(UlyssesOracle):
    """The oracle with the QKV GEMM replaced by a table: rank r's projection output is codes[r], so
    that its head-side buffers show, element by element, which output element belongs where."""

    def __init__(self, codes, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.codes = codes

    def qkv_sequence_side(self, x):
        table = self.codes[int(x[0, 0])]
        out = torch.zeros(x.shape[0], table.shape[1])
        out[:table.shape[0]] = table
        return out


@pytest.mark.parametrize('p,hidden,heads,segments', [(1, 512, 4, 3), (2, 512, 4, 3), (4, 1024, 8, 4), (8, 1024, 8, 3),
                                                     (2, 512, 4, 1), (8, 1024, 8, 1),
                                                     # the benchmark geometries at CP = 8: 4, 3, 5 heads per rank
                                                     (8, 4096, 32, 3), (8, 3072, 24, 4), (8, 5120, 40, 3),
                                                     (8, 3072, 24, 1), (8, 5120, 40, 1)])
def test_push_routing_matches_the_oracle_layout(sched, p, hidden, heads, segments):
    """Every output element of every source rank lands where the oracle's head-side buffers have it.
    The GEMM output of rank r is a table of distinct codes (through a stand-in for the QKV GEMM, or an
    identity weight for the output-projection dgrad), so equality of the buffers is equality of the
    routing."""
    tokens, capacity = 3, 256
    hpr, width = heads // p, hidden // p
    n = segments * hidden
    codes = [torch.arange(1, tokens * n + 1, dtype=torch.float32).reshape(tokens, n) + 100000 * r for r in range(p)]
    if segments > 1:
        oracle = _CodedOracle(codes, p, hidden, heads, segments, dtype=torch.float32)
        xs = [torch.full((tokens, hidden), float(r)) for r in range(p)]
        expected = oracle.qkv_heads_buffers(xs, capacity)
    else:
        oracle = UlyssesOracle(p, hidden, heads, 1, weight_out=torch.eye(hidden), dtype=torch.float32)
        expected = [[buffer] for buffer in oracle.out_dhead_buffers(codes, capacity)]
    got = [[torch.zeros(p * capacity, width) for _ in range(segments)] for _ in range(p)]
    out = (I * 3)()
    for r in range(p):
        for col in range(n):
            sched.sched_push_route(col, segments, hpr, out)
            seg, dest, column = tuple(out)
            assert 0 <= seg < segments and 0 <= dest < p and 0 <= column < width
            for row in range(tokens):
                element = sched.sched_push_element(col, segments, hpr, r, capacity, row, width)
                assert element == (r * capacity + row) * width + column
                got[dest][seg].view(-1)[element] = codes[r][row, col]
    for dest in range(p):
        for seg in range(segments):
            assert torch.equal(got[dest][seg], expected[dest][seg]), (dest, seg)


# ------------------------------------------------------------------------------------ pusher jobs
@pytest.mark.parametrize('m_tiles,num_in,p,split,group_m', [(64, 3, 8, 2, 4), (64, 1, 8, 2, 4), (2, 3, 2, 4, 4),
                                                            (5, 4, 4, 1, 1), (11, 1, 1, 8, 4), (1, 3, 8, 2, 4)])
@pytest.mark.parametrize('grid', [148, 4, 2])
def test_both_pusher_phases_run_every_job_once(sched, m_tiles, num_in, p, split, group_m, grid):
    """All CTAs x 4 warps take the first two raster groups; then `push_warps` warps of every CTA
    take the rest. Every job exactly once, for any rank."""
    total = sched.sched_push_jobs_total(m_tiles, num_in, p, split)
    first = sched.sched_first_phase_jobs(m_tiles, group_m, num_in, p, split)
    assert total == m_tiles * 2 * num_in * p * split
    assert first == min(total, min(2 * group_m, m_tiles) * 2 * num_in * p * split)
    runs = [0] * total
    for cta in range(grid):
        for warp in range(4):
            for job in range(cta * 4 + warp, first, grid * 4):
                runs[job] += 1
    for push_warps in (1, 2, 4):
        again = list(runs)
        for cta in range(grid):
            for warp in range(push_warps):
                for job in range(first + cta * push_warps + warp, total, grid * push_warps):
                    again[job] += 1
        assert again == [1] * total
    # decoding: a bijection onto (row block, segment, destination, sub-block), destinations rotated by rank
    for rank in range(p):
        decoded = [job_of(sched, job, num_in, p, split, rank) for job in range(total)]
        assert sorted(d[:4] for d in decoded) == sorted(itertools.product(range(m_tiles * 2), range(num_in), range(p), range(split)))
        assert all(row0 == mi * 128 + q * (128 // split) for mi, _, _, q, row0 in decoded)
        assert decoded[0][2] == rank and [d[0] for d in decoded] == sorted(d[0] for d in decoded)


@pytest.mark.parametrize('hpr,num_in,split', [(4, 3, 2), (4, 1, 2), (16, 3, 4), (32, 1, 8), (1, 4, 1), (3, 3, 1), (20, 1, 4),
                                              (17, 1, 4), (3, 4, 1), (3, 1, 1), (5, 3, 2), (5, 1, 2), (40, 3, 16)])
def test_chunks_move_every_byte_of_a_job_once_and_zero_the_missing_rows(sched, hpr, num_in, split):
    sub_rows = 128 // split
    units, rows = chunking(sched, hpr, sub_rows)
    assert units * rows * 256 <= 4096 and hpr % units == 0 and sub_rows % rows == 0
    assert rows == 1 or units == hpr
    count = sched.sched_push_chunks_per_job(hpr, units, rows, sub_rows)
    out = (I * 3)()
    for src_rows, row0 in ((10 ** 6, 0), (sub_rows + 3, sub_rows), (5, 0), (128, 128)):
        moved = torch.zeros(sub_rows, hpr, dtype=torch.int32)
        zeros = torch.zeros(sub_rows, hpr, dtype=torch.int32)
        for c in range(count):
            sched.sched_push_chunk(c, hpr, units, rows, src_rows, row0, out)
            r0, u0, valid = tuple(out)
            assert 0 <= valid <= rows
            moved[r0:r0 + rows, u0:u0 + units] += 1
            zeros[r0 + valid:r0 + rows, u0:u0 + units] += 1
        assert bool((moved == 1).all())
        exists = (torch.arange(sub_rows) + row0 < src_rows).int().view(-1, 1).expand(-1, hpr)
        assert torch.equal(zeros, 1 - exists)


@pytest.mark.parametrize('p,hidden,heads,num_in', [(2, 512, 4, 3), (4, 1024, 8, 4), (8, 1024, 8, 3), (8, 1024, 8, 1)])
def test_receive_columns_match_the_oracle_layout(sched, p, hidden, heads, num_in):
    """Where the pushers of every rank put each head unit in a destination's receive buffer, against
    the oracle's receive buffers built from tensors that encode (rank, segment, row, column)."""
    tokens, hpr = 2, heads // p
    oracle = UlyssesOracle(p, hidden, heads, max(num_in, 1))
    sources = [tuple(torch.arange(p * tokens * hpr * 128, dtype=torch.float32).reshape(p * tokens, hpr, 128)
                     + 1e6 * r + 1e5 * t for t in range(num_in)) for r in range(p)]
    for dest in range(p):
        want = (oracle.qkv_recv_buffer(sources, dest) if num_in > 1
                else oracle.out_recv_buffer([s[0] for s in sources], dest))
        got = torch.full_like(want, -1.0)
        for r in range(p):
            for t in range(num_in):
                block = sources[r][t][dest * tokens:(dest + 1) * tokens]        # rows this rank sends to dest
                for unit in range(hpr):
                    column = sched.sched_recv_column(r, hpr, unit, num_in, t)
                    got[:, column:column + 128] = block[:, unit]
        assert torch.equal(got, want)


# ------------------------------------------------------------------------------------ grouped-query layouts
class _CodedGroupedOracle(GroupedQueryOracle):
    """The grouped-query oracle with the QKV GEMM replaced by a table of codes (see _CodedOracle)."""

    def __init__(self, codes, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.codes = codes

    def qkv_sequence_side(self, x):
        table = self.codes[int(x[0, 0])]
        out = torch.zeros(x.shape[0], table.shape[1])
        out[:table.shape[0]] = table
        return out


@pytest.mark.parametrize('p,heads,kv_heads,gate', [(1, 8, 2, False), (2, 8, 2, True), (2, 8, 4, False), (4, 32, 8, False),
                                                   (8, 64, 8, True), (8, 32, 8, False), (2, 6, 6, True)])
def test_grouped_push_routing_and_receive_columns_match_the_oracle(sched, p, heads, kv_heads, gate):
    """More query heads than key/value heads: every output element of every source rank lands in the
    head-side buffer (kind, destination, column, row pitch) where the grouped-query oracle has it, and
    the pushers' receive columns rebuild the oracle's receive buffer. The oracle itself is pinned by the
    reference's unfused modules run with num_kv_heads < num_heads."""
    d, tokens, capacity = 128, 2, 256
    hidden = heads * d
    r, gpr = heads // kv_heads, kv_heads // p
    layout = (r, 1, r if gate else 0, gpr)
    kinds = 4 if gate else 3
    n = kv_heads * (r * (2 if gate else 1) + 2) * d
    codes = [torch.arange(1, tokens * n + 1, dtype=torch.float32).reshape(tokens, n) + 1e7 * rank for rank in range(p)]
    oracle = _CodedGroupedOracle(codes, p, hidden, heads, kv_heads, gate, dtype=torch.float32)
    xs = [torch.full((tokens, hidden), float(rank)) for rank in range(p)]
    expected = oracle.qkv_heads_buffers(xs, capacity)
    got = [[torch.zeros_like(expected[dest][kind]) for kind in range(kinds)] for dest in range(p)]
    out = (I * 4)()
    for rank in range(p):
        for col in range(0, n, 128):                      # one unit at a time: 128 columns move together
            sched.sched_push_route_grouped(col, *layout, out)
            kind, dest, column, pitch = tuple(out)
            assert 0 <= kind < kinds and 0 <= dest < p and pitch == expected[dest][kind].shape[1]
            assert pitch == 128 * sched.sched_kind_pitch_units(*layout, kind) and 0 <= column <= pitch - 128
            for row in range(tokens):
                element = sched.sched_push_element_grouped(col, *layout, rank, capacity, row)
                assert element == (rank * capacity + row) * pitch + column
                got[dest][kind].view(-1)[element:element + 128] = codes[rank][row, col:col + 128]
    for dest in range(p):
        for kind in range(kinds):
            assert torch.equal(got[dest][kind], expected[dest][kind]), (dest, kind)
    # receive side: rank `rank` pushes unit u of its kind-`kind` input for destination dest
    widths = [gpr * (r if kind in (0, 3) else 1) for kind in range(kinds)]
    sources = [tuple(torch.arange(p * tokens * widths[kind] * d, dtype=torch.float32).reshape(p * tokens, widths[kind], d)
                     + 1e7 * rank + 1e6 * kind for kind in range(kinds)) for rank in range(p)]
    for dest in range(p):
        want = oracle.qkv_recv_buffer(sources, dest)
        rebuilt = torch.full_like(want, -1.0)
        for rank in range(p):
            for kind in range(kinds):
                block = sources[rank][kind][dest * tokens:(dest + 1) * tokens]
                assert sched.sched_kind_pitch_units(*layout, kind) == widths[kind]
                for unit in range(widths[kind]):
                    column = sched.sched_recv_column_grouped(rank, *layout, kind, unit)
                    rebuilt[:, column:column + d] = block[:, unit]
        assert torch.equal(rebuilt, want)


def test_uniform_layout_is_the_grouped_layout_with_one_query_head_per_group(sched):
    out3, out4 = (I * 3)(), (I * 4)()
    for segments, hpr in ((1, 4), (3, 4), (4, 3), (3, 5)):
        layout = (1, 1 if segments > 1 else 0, 1 if segments == 4 else 0, hpr)
        for col in range(0, 2 * segments * hpr * 128, 64):
            sched.sched_push_route(col, segments, hpr, out3)
            sched.sched_push_route_grouped(col, *layout, out4)
            assert tuple(out3) == tuple(out4)[:3] and out4[3] == hpr * 128
        for rank in range(2):
            for t in range(segments):
                for unit in range(hpr):
                    assert sched.sched_recv_column(rank, hpr, unit, segments, t) == \
                        sched.sched_recv_column_grouped(rank, *layout, t, unit)


# ------------------------------------------------------------------------------------ MXFP8 rule
def test_scale_rule_equals_the_oracle_on_every_bf16_magnitude_and_around_every_threshold(sched):
    """The CUDA quantizer's scale rule (csrc/mx_rule.cuh, compiled here for the host) against the
    oracle, which is pinned by the reference tests' known answers: all BF16 magnitudes including
    zero, subnormals and +Inf, and for every binade the FP32 values at and next to the rounding
    threshold (mantissa 0x600000) and the binade's ends."""
    import numpy as np
    bf16 = np.arange(0x0000, 0x7f81, dtype=np.int64) << 16
    exponents = np.arange(0, 255, dtype=np.int64) << 23
    around = np.concatenate([exponents + m for m in (0, 1, 0x5fffff, 0x600000, 0x600001, 0x7fffff)])
    patterns = np.concatenate([bf16, around]).astype(np.int32)
    got_e = np.zeros(len(patterns), dtype=np.int32)
    got_m = np.zeros(len(patterns), dtype=np.int32)
    sched.rule_mx_scale(patterns.ctypes.data_as(ctypes.POINTER(I)), len(patterns),
                        got_e.ctypes.data_as(ctypes.POINTER(I)), got_m.ctypes.data_as(ctypes.POINTER(I)))
    want_e, want_m = mxfp8_oracle.mx_scale(patterns.view(np.float32))
    assert np.array_equal(got_e, want_e)
    assert np.array_equal(got_m, want_m.view(np.int32))
    assert got_e[0] == 0 and got_m[0] == 0x3f800000                  # zero group: scale 1
    assert got_e[0x7f80] == 128 and got_m[0x7f80] == 0               # +Inf group: NaN scale, multiplier 0
    assert got_e.min() == -126 and got_e[:0x7f80].max() == 120      # clamped below; the largest finite BF16 needs 2^120


def test_scale_bytes_fill_the_tcgen05_blocks_exactly(sched):
    import numpy as np
    for rows, groups in ((256, 4), (256, 16), (512, 40), (1024, 8)):
        offsets = np.array([[sched.rule_mx_scale_offset(r, g, groups) for g in range(groups)] for r in range(rows)])
        want = mxfp8_oracle.scale_offset(np.arange(rows)[:, None], np.arange(groups)[None, :], groups)
        assert np.array_equal(offsets, want)
        assert sorted(offsets.ravel().tolist()) == list(range(rows * groups))     # a bijection onto the buffer
        # one 512-byte block per (128 rows, 4 groups); the four groups of a row are adjacent bytes
        assert np.array_equal(offsets // 512, (np.arange(rows)[:, None] // 128) * (groups // 4) + np.arange(groups)[None, :] // 4)
        assert np.array_equal(offsets[:, 1] - offsets[:, 0], np.ones(rows, dtype=offsets.dtype))


# ------------------------------------------------------------------------------------ randomized sweeps
def test_random_geometries_keep_the_exactly_once_properties(sched):
    """300 random geometries (fixed seed): raster and K shares cover every (tile, K step) once under a
    random grid size; the pusher schedule with a random number of pushing-only pairs runs every job
    once; a job's chunks cover its rows and units once."""
    import random
    rng = random.Random(20251125)
    for _ in range(300):
        m_tiles, n_tiles = rng.randint(1, 40), rng.randint(1, 24)
        group_m, pairs = rng.randint(1, 20), rng.randint(1, 80)
        k_splits = rng.choice([1, 1, 2, 3, 5, 8])
        k_tiles = rng.randint(k_splits, 40)
        total = m_tiles * n_tiles
        seen = set()
        for pair in range(min(pairs, total * k_splits)):
            for u in range(pair, total * k_splits, pairs):
                t, kt0, kt1 = unit_of(sched, k_tiles, k_splits, total, u)
                m, n = tile_of(sched, m_tiles, n_tiles, group_m, t)
                assert 0 <= m < m_tiles and 0 <= n < n_tiles and kt0 < kt1
                for kt in range(kt0, kt1):
                    assert (m, n, kt) not in seen
                    seen.add((m, n, kt))
        assert len(seen) == total * k_tiles

        p, num_in = rng.choice([1, 2, 4, 8]), rng.choice([1, 3, 4])
        split = rng.choice([1, 2, 4, 8, 16])
        jobs = sched.sched_push_jobs_total(m_tiles, num_in, p, split)
        first = sched.sched_first_phase_jobs(m_tiles, group_m, num_in, p, split)
        grid = 2 * rng.randint(1, 74)
        runs = [0] * jobs
        for cta in range(grid):
            for warp in range(4):
                for job in range(cta * 4 + warp, first, grid * 4):
                    runs[job] += 1
        warps = rng.randint(1, 4)
        for cta in range(grid):
            for warp in range(warps):
                for job in range(first + cta * warps + warp, jobs, grid * warps):
                    runs[job] += 1
        assert runs == [1] * jobs

        hpr, sub_rows = rng.randint(1, 40), 128 // split
        units, rows = chunking(sched, hpr, sub_rows)
        assert 1 <= units <= 16 and hpr % units == 0 and units * rows * 256 <= 4096 and sub_rows % rows == 0
        covered = torch.zeros(sub_rows, hpr, dtype=torch.int32)
        out = (I * 3)()
        src_rows, row0 = rng.randint(1, 400), rng.choice([0, 128, 256]) + rng.randrange(0, 128, sub_rows)
        for c in range(sched.sched_push_chunks_per_job(hpr, units, rows, sub_rows)):
            sched.sched_push_chunk(c, hpr, units, rows, src_rows, row0, out)
            r0, u0, valid = tuple(out)
            covered[r0:r0 + rows, u0:u0 + units] += 1
            assert valid == max(0, min(rows, src_rows - (row0 + r0)))
        assert bool((covered == 1).all())
