// Host build of the kernel's index arithmetic (csrc/schedule.cuh) for the CPU tests: plain C
// entry points over the same inline functions the CUDA kernel and its launchers compile.
// Built by tests/test_schedule_native.py with g++; not part of libfga.so.
#include "../../fused-gemm-a2a_b200/csrc/schedule.cuh"
#include "../../fused-gemm-a2a_b200/csrc/mx_rule.cuh"

using namespace fga::sched;

extern "C" {

void sched_tile_coords(int m_tiles, int n_tiles, int group_m, int t, int* m, int* n) {
  tile_coords(m_tiles, n_tiles, group_m, t, *m, *n);
}

void sched_unit_coords(int k_tiles, int k_splits, int total_tiles, int u, int* t, int* kt0, int* kt1) {
  unit_coords(k_tiles, k_splits, total_tiles, u, *t, *kt0, *kt1);
}

int sched_rotated_n(int n, int n_rotate, int n_tiles) { return rotated_n(n, n_rotate, n_tiles); }

// out: segment, dest, column
void sched_push_route(int col, int segments, int heads_per_rank, int* out) {
  const PushRoute r = push_route(col, segments, heads_per_rank);
  out[0] = r.segment;
  out[1] = r.dest;
  out[2] = r.column;
}

long long sched_push_element(int col, int segments, int heads_per_rank, int rank, long long head_rows, int row,
                             long long head_pitch) {
  const PushRoute r = push_route(col, segments, heads_per_rank);
  return r.pitch == head_pitch ? push_element(r, rank, head_rows, row) : -1;
}

// Grouped layouts (more query heads than key/value heads). out: segment, dest, column, pitch
void sched_push_route_grouped(int col, int q_units, int kv_units, int gate_units, int groups_per_rank, int* out) {
  const HeadLayout l{q_units, kv_units, gate_units, groups_per_rank};
  const PushRoute r = push_route(col, l);
  out[0] = r.segment;
  out[1] = r.dest;
  out[2] = r.column;
  out[3] = r.pitch;
}

long long sched_push_element_grouped(int col, int q_units, int kv_units, int gate_units, int groups_per_rank, int rank,
                                     long long head_rows, int row) {
  const HeadLayout l{q_units, kv_units, gate_units, groups_per_rank};
  return push_element(push_route(col, l), rank, head_rows, row);
}

long long sched_recv_column_grouped(int rank, int q_units, int kv_units, int gate_units, int groups_per_rank, int kind,
                                    int unit) {
  const HeadLayout l{q_units, kv_units, gate_units, groups_per_rank};
  return recv_column(rank, l, kind, unit);
}

int sched_kind_pitch_units(int q_units, int kv_units, int gate_units, int groups_per_rank, int kind) {
  const HeadLayout l{q_units, kv_units, gate_units, groups_per_rank};
  return kind_pitch_units(l, kind);
}

long long sched_push_jobs_total(int m_tiles, int num_in, int p, int split) {
  return push_jobs_total(m_tiles, num_in, p, split);
}

long long sched_first_phase_jobs(int m_tiles, int group_m, int num_in, int p, int split) {
  return first_phase_jobs(m_tiles, group_m, num_in, p, split);
}

// out: mi, t, d, q, row0
void sched_decode_push_job(long long job, int num_in, int p, int split, int rank, int* out) {
  const PushJob j = decode_push_job(job, num_in, p, split, rank);
  out[0] = j.mi;
  out[1] = j.t;
  out[2] = j.d;
  out[3] = j.q;
  out[4] = j.row0;
}

int sched_push_chunks_per_job(int heads_per_rank, int units, int rows, int sub_rows) {
  return push_chunks_per_job(heads_per_rank, units, rows, sub_rows);
}

// out: r0, u0, valid
void sched_push_chunk(int c, int heads_per_rank, int units, int rows, int src_rows, int row0, int* out) {
  const PushChunk k = push_chunk(c, heads_per_rank, units, rows, src_rows, row0);
  out[0] = k.r0;
  out[1] = k.u0;
  out[2] = k.valid;
}

void sched_push_chunking(int heads_per_rank, int sub_rows, int buffer_bytes, int* units, int* rows) {
  push_chunking(heads_per_rank, sub_rows, buffer_bytes, *units, *rows);
}

long long sched_recv_column(int rank, int heads_per_rank, int unit, int num_in, int t) {
  return recv_column(rank, heads_per_rank, unit, num_in, t);
}

int sched_pick_k_splits(long long tiles, int k_tiles, int pairs, int forced) {
  return pick_k_splits(tiles, k_tiles, pairs, forced);
}

// MXFP8 scale rule on `count` FP32 bit patterns: exponents[i] (128 = the NaN scale) and the bit
// patterns of the multipliers.
void rule_mx_scale(const int* peak_bits, int count, int* exponents, int* multiplier_bits) {
  for (int i = 0; i < count; ++i) {
    float inv;
    fga::rule::mx_scale(fga::rule::bits_float(peak_bits[i]), exponents[i], inv);
    multiplier_bits[i] = fga::rule::float_bits(inv);
  }
}

long long rule_mx_scale_offset(long long row, int group, int groups) {
  return fga::rule::mx_scale_offset(row, group, groups);
}

}  // extern "C"
