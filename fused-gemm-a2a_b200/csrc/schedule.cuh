// Index arithmetic of the persistent GEMM: which tile a CTA pair works on, which K steps a work
// unit covers, where a finished head tile is stored on which peer, which rows a pusher job moves.
// Pure integer functions, compiled for the device by the kernel and for the host by the launchers
// and by the CPU tests (tests/native/schedule_host.cpp builds them with g++ and checks coverage,
// exactly-once properties and the routing against the oracle's layout), so that the schedule can be
// verified without a GPU.
#pragma once

#if defined(__CUDACC__)
#define FGA_HD __host__ __device__ __forceinline__
#else
#define FGA_HD inline
#endif

namespace fga {
namespace sched {

FGA_HD int imin(int a, int b) { return a < b ? a : b; }
FGA_HD int imax(int a, int b) { return a > b ? a : b; }
FGA_HD long long lmin(long long a, long long b) { return a < b ? a : b; }

// ---- tiles ------------------------------------------------------------------------------------
// Tile t of the raster -> (pair tile along M, tile along N). N varies fastest inside a group of
// `group_m` pair tiles, so a wave of CTA pairs stays within a few row blocks (the recv GEMM can
// start before later blocks arrive; a push wave spreads its stores over all destinations) and
// each weight tile is reused across the group out of L2. The last group may be shorter.
FGA_HD void tile_coords(int m_tiles, int n_tiles, int group_m, int t, int& m, int& n) {
  const int per_group = group_m * n_tiles;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int gm = imin(group_m, m_tiles - g * group_m);
  n = r / gm;
  m = g * group_m + (r - n * gm);
}

// Work unit u -> (output tile, K-step range). With k_splits > 1 the split index varies slowest, so
// a wave of CTA pairs works on one K range and the operands it shares stay in L2; every unit adds
// its partial tile into the FP32 output with bulk reductions.
FGA_HD void unit_coords(int k_tiles, int k_splits, int total_tiles, int u, int& t, int& kt0, int& kt1) {
  if (k_splits <= 1) {
    t = u;
    kt0 = 0;
    kt1 = k_tiles;
    return;
  }
  const int s = u / total_tiles;
  t = u - s * total_tiles;
  kt0 = static_cast<int>(static_cast<long long>(s) * k_tiles / k_splits);
  kt1 = static_cast<int>(static_cast<long long>(s + 1) * k_tiles / k_splits);
}

// N tile after the per-rank rotation of push mode (ranks start on different peers).
FGA_HD int rotated_n(int n, int n_rotate, int n_tiles) {
  n += n_rotate;
  return n >= n_tiles ? n - n_tiles : n;
}

// ---- head layout --------------------------------------------------------------------------------
// The output columns of a projection (= its weight rows) are 128-wide units, one per (head, kind).
// Units come in groups, one group per key/value head: `q_units` query heads, then the key head and
// the value head (`kv_units` = 1, or 0 for the output projection, which has neither), then
// `gate_units` gate heads (0 or q_units). With one query head per key/value head this is Megatron's
// per-head order [q_h; k_h; v_h; (g_h)]; with several it is its grouped-query order
// [q_g0 .. q_g(r-1); k_g; v_g; (gate_g0 .. gate_g(r-1))]. Every rank owns `groups_per_rank`
// consecutive groups. Kinds are numbered like the head-side buffers: 0 = q, 1 = k, 2 = v, 3 = gate.
struct HeadLayout {
  int q_units, kv_units, gate_units, groups_per_rank;
};

FGA_HD HeadLayout uniform_layout(int segments, int heads_per_rank) {
  HeadLayout l;
  l.q_units = 1;
  l.kv_units = segments > 1 ? 1 : 0;
  l.gate_units = segments == 4 ? 1 : 0;
  l.groups_per_rank = heads_per_rank;
  return l;
}

FGA_HD int group_units(const HeadLayout& l) { return l.q_units + 2 * l.kv_units + l.gate_units; }

// Units of kind `kind` per group, and where they start inside the group.
FGA_HD int kind_units(const HeadLayout& l, int kind) {
  return kind == 0 ? l.q_units : (kind == 3 ? l.gate_units : l.kv_units);
}
FGA_HD int kind_offset(const HeadLayout& l, int kind) {
  return kind == 0 ? 0 : (kind == 1 ? l.q_units : (kind == 2 ? l.q_units + l.kv_units : l.q_units + 2 * l.kv_units));
}
// 128-wide units per row of one rank's head-side buffer of that kind (its row pitch in units).
FGA_HD int kind_pitch_units(const HeadLayout& l, int kind) { return l.groups_per_rank * kind_units(l, kind); }

// ---- push routing -----------------------------------------------------------------------------
// Output column `col` of a push GEMM belongs to unit col/128 = group*group_units + position. The
// group lives on peer group/groups_per_rank, in that peer's buffer of the unit's kind, whose rows are
// `pitch` elements long, at column ((group % groups_per_rank)*kind_units + index in kind)*128 +
// col%128; the rows of source rank r start at r*head_rows.
struct PushRoute {
  int segment, dest, column, pitch;
};

FGA_HD PushRoute push_route(int col, const HeadLayout& l) {
  const int unit = col >> 7;
  const int per_group = group_units(l);
  const int group = unit / per_group;
  const int position = unit - group * per_group;
  PushRoute r;
  r.segment = position < l.q_units ? 0
              : (position < l.q_units + l.kv_units ? 1 : (position < l.q_units + 2 * l.kv_units ? 2 : 3));
  const int within = position - kind_offset(l, r.segment);
  const int per_kind = kind_units(l, r.segment);
  r.dest = group / l.groups_per_rank;
  r.column = ((group - r.dest * l.groups_per_rank) * per_kind + within) * 128 + (col & 127);
  r.pitch = l.groups_per_rank * per_kind * 128;
  return r;
}

FGA_HD PushRoute push_route(int col, int segments, int heads_per_rank) {
  return push_route(col, uniform_layout(segments, heads_per_rank));
}

FGA_HD long long push_element(const PushRoute& r, int rank, long long head_rows, int row) {
  return (static_cast<long long>(rank) * head_rows + row) * r.pitch + r.column;
}

// ---- pusher jobs (recv mode) --------------------------------------------------------------------
// Job = (row block mi of 128 rows, input segment t, destination d, row sub-block q). Jobs are
// numbered row-block-major; inside a block the sub-block varies fastest, then the destination,
// rotated by the rank so that ranks do not all start on the same peer, then the segment.
struct PushJob {
  int mi, t, d, q, row0;
};

FGA_HD int push_jobs_per_block(int num_in, int p, int split) { return num_in * p * split; }

FGA_HD long long push_jobs_total(int m_tiles, int num_in, int p, int split) {
  return static_cast<long long>(m_tiles) * 2 * push_jobs_per_block(num_in, p, split);
}

FGA_HD PushJob decode_push_job(long long job, int num_in, int p, int split, int rank) {
  const int per_block = push_jobs_per_block(num_in, p, split);
  PushJob j;
  j.mi = static_cast<int>(job / per_block);
  int rest = static_cast<int>(job - static_cast<long long>(j.mi) * per_block);
  j.q = rest % split;
  rest /= split;
  j.d = (rest % p + rank) % p;
  j.t = rest / p;
  j.row0 = j.mi * 128 + j.q * (128 / split);
  return j;
}

// Jobs of the first two raster groups, which the GEMM cannot start without: every pusher warp of
// every CTA works on them; the rest is the steady phase.
FGA_HD long long first_phase_jobs(int m_tiles, int group_m, int num_in, int p, int split) {
  const long long per_block = push_jobs_per_block(num_in, p, split);
  return lmin(push_jobs_total(m_tiles, num_in, p, split),
              static_cast<long long>(imin(2 * group_m, m_tiles)) * 2 * per_block);
}

// A job is moved in chunks of `rows_per_chunk` rows x `units_per_chunk` 256-byte head units (one
// shared buffer). Chunk c -> first row r0 within the job, first unit u0 within the row, and the
// number of its rows that exist in the source (the others travel as zeros).
struct PushChunk {
  int r0, u0, valid;
};

FGA_HD int push_chunks_per_job(int heads_per_rank, int units_per_chunk, int rows_per_chunk, int sub_rows) {
  const int pieces_per_row = heads_per_rank / units_per_chunk;
  return pieces_per_row == 1 ? sub_rows / rows_per_chunk : sub_rows * pieces_per_row;
}

FGA_HD PushChunk push_chunk(int c, int heads_per_rank, int units_per_chunk, int rows_per_chunk, int src_rows,
                            int row0) {
  const int pieces_per_row = heads_per_rank / units_per_chunk;
  PushChunk k;
  if (pieces_per_row == 1) {
    k.r0 = c * rows_per_chunk;
    k.u0 = 0;
  } else {
    k.r0 = c / pieces_per_row;
    k.u0 = (c - k.r0 * pieces_per_row) * units_per_chunk;
  }
  k.valid = imax(0, imin(rows_per_chunk, src_rows - (row0 + k.r0)));
  return k;
}

// Chunk shape for a buffer of `buffer_bytes`: whole rows when a row of heads_per_rank units fits
// (then as many rows as fit, a power of two, at most the job's rows), else equal pieces of whole
// units.
FGA_HD void push_chunking(int heads_per_rank, int sub_rows, int buffer_bytes, int& units, int& rows) {
  units = heads_per_rank;
  while (units > buffer_bytes / 256 || heads_per_rank % units) --units;
  rows = 1;
  if (units == heads_per_rank)
    while (rows * 2 * units * 256 <= buffer_bytes && rows * 2 <= sub_rows) rows *= 2;
}

// First BF16 column, in the receive buffer, of unit `unit` (0 .. kind_pitch_units - 1) of the input of
// kind `kind` pushed by `rank`: the receive buffer is in weight-row order, group after group.
FGA_HD long long recv_column(int rank, const HeadLayout& l, int kind, int unit) {
  const int per_kind = kind_units(l, kind);
  const int group_local = unit / per_kind;
  const int within = unit - group_local * per_kind;
  const long long group = static_cast<long long>(rank) * l.groups_per_rank + group_local;
  return (group * group_units(l) + kind_offset(l, kind) + within) * 128;
}

FGA_HD long long recv_column(int rank, int heads_per_rank, int unit, int num_in, int t) {
  return recv_column(rank, uniform_layout(num_in, heads_per_rank), t, unit);
}

// ---- K shares of an FP32 gradient GEMM ----------------------------------------------------------
// Wave efficiency of `units` work units on `pairs` CTA pairs.
FGA_HD double wave_efficiency(long long units, int pairs) {
  const long long waves = (units + pairs - 1) / pairs;
  return static_cast<double>(units) / (static_cast<double>(waves) * pairs);
}

// forced = 0: the smallest share count (<= 8, every share keeping >= 32 K steps) that reaches 97 %
// wave efficiency, else the most efficient one. forced > 1: that count, lowered until every share
// keeps 32 K steps.
FGA_HD int pick_k_splits(long long tiles, int k_tiles, int pairs, int forced) {
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 8; ++s) {
    if (s > 1 && k_tiles / s < 32) break;
    if (forced > 0) {
      best = s;
      if (s == forced) break;
      continue;
    }
    const double eff = wave_efficiency(tiles * s, pairs);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = s;
    }
    if (eff >= 0.97) break;
  }
  return best;
}

}  // namespace sched
}  // namespace fga
