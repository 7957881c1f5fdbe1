// Persistent 2-CTA tcgen05 GEMM for sm_100a with the Ulysses all-to-all fused in.
//
// One kernel, three modes (the reference's UlyssesGemm, fused_gemm_a2a_kernels.py:400-929):
//   local : C = A * B^T, plain store or FP32 accumulate (weight gradients)
//   push  : the epilogue stores every finished 128x128 head tile straight into the owning peer's
//           head-side buffer over NVLink (QKV forward, output-projection dgrad)
//   recv  : pusher warps move this rank's head-side input into the peers' receive buffers with
//           bulk copies (global -> shared -> peer global) and bump per-row-block arrival counters;
//           the TMA producer polls its own counters before loading a row block
//           (output-projection forward, QKV dgrad)
//
// Layout of one CTA pair (cluster 2x1x1): the pair owns a 256 x BN output tile, each CTA 128 rows.
// Each CTA TMA-loads its own 128 rows of A and its half (BN/2) of B per 64-wide K step; one thread
// of the leader CTA issues tcgen05.mma.cta_group::2 into TMEM of both CTAs (2 accumulator stages
// of BN columns each). Four epilogue warps per CTA read TMEM (thread = row), convert, write their
// own 128-byte row piece to shared memory and ship it with a 1-D bulk copy (cp.async.bulk) to
// local or peer global memory; FP32 gradient accumulation uses the bulk reduce-add. No TMA load
// uses cluster multicast. Every wait is bounded: on expiry the waiter records an error in the
// caller's status word, all roles drain, TMEM is freed and the kernel returns.
//
// Shared memory (220 KiB): local/push run 6 pipeline stages of 32 KiB; recv runs 5 stages and
// gives the sixth to the pusher warps (4 warps x 2 buffers x 4 KiB); 18 KiB of epilogue staging.
#pragma once
#include "ptx.cuh"
#include "common.cuh"
#include "mx_quant.cuh"
#include "schedule.cuh"

namespace fga {

constexpr int kMaxStages = 6;
constexpr int kTileM = 128;             // rows per CTA
constexpr int kTileK = 64;              // BF16 elements per K step (128 bytes = one swizzle span)
constexpr int kABytes = kTileM * 128;   // 16 KiB
constexpr int kBBytes = 128 * 128;      // 16 KiB (BN/2 <= 128 rows)
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kPieceBytes = 128;        // epilogue row piece: 64 BF16 or 32 FP32 columns
constexpr int kSlotPitch = kPieceBytes + 16;  // 16-byte skew: conflict-free 16-byte stores
constexpr int kStagingBytes = 128 * kSlotPitch;
constexpr int kBarrierBytes = 256;
constexpr int kSfStageBytes = 1536;     // MXFP8: 512 B of A scales + 2 x 512 B of B scales per stage
constexpr int kQuantWarps = 2;          // MXFP8 recv: warps that quantize arrived BF16 row blocks
constexpr int kGemmWarps = 6;           // TMA, MMA, 4 epilogue
constexpr int kPusherWarps = 4;
constexpr int kPushBufBytes = 4096;     // per pusher warp: two of these
constexpr int kSmemBytes =
    kMaxStages * (kStageBytes + kSfStageBytes) + kStagingBytes + kBarrierBytes + 1024;
static_assert(kPusherWarps * 2 * kPushBufBytes == kStageBytes, "pusher buffers reuse one stage");

enum GemmMode : int { kLocal = 0, kPush = 1, kRecv = 2 };
enum EpiMode : int { kEpiBf16 = 0, kEpiF32Store = 1, kEpiF32Add = 2 };

struct GemmParams {
  // geometry
  int m_tiles, n_tiles, k_tiles;  // 256-row pair tiles, BN-column tiles, 64-element K steps
  int bn;                         // 128 or 256
  int stages;                     // pipeline stages in use (<= kMaxStages)
  int group_m;                    // pair tiles per raster group (N varies fastest inside a group)
  int k_splits;                   // work units per output tile, each a contiguous share of the K steps
                                  // (> 1 only with the FP32 reduce-add epilogue)
  int a_mn, b_mn;                 // 1 = operand is MN-major in global memory (transposed read)
  uint32_t idesc;                 // tcgen05 instruction descriptor
  int mode, epi;
  int rank, p;
  // local / recv output
  void* c;
  long long c_pitch;  // elements per output row
  int c_rows;         // rows of c that exist; others are not stored
  // push
  const uint16_t* bias;            // BF16 bias indexed by weight row, added in FP32, or null
  const long long* peer_heads[4];  // device int64[P]: peers' head-side buffer base per kind (q, k, v, gate)
  sched::HeadLayout layout;        // how the output columns (push) / receive-buffer columns (recv) are
                                   // grouped into heads and which rank owns which group
  long long head_rows;             // rows of one rank block in the head-side buffers (capacity)
  int n_rotate;                    // N-tile rotation so that ranks start on different peers
  // recv
  int* counters;                   // this rank's arrival counters, one per 128 rows
  int target;                      // arrivals that complete a row block
  const long long* peer_recv;      // device int64[P]
  const long long* peer_counters;  // device int64[P]
  const void* src[4];              // head-side inputs [P*src_rows, in_units[t]*128] BF16
  int num_in, src_rows, split;
  int in_units[4];                 // 128-wide units per row of input t (q and gate: groups_per_rank*q_units,
                                   // k and v: groups_per_rank)
  int push_units[4];               // 256-byte units per pusher chunk row of input t (divides in_units[t])
  int push_rows[4];                // rows per pusher chunk (1 unless push_units[t] == in_units[t])
  long long recv_k;                // elements per receive-buffer row
  int roles;                       // bit 0: GEMM roles run, bit 1: pusher warps run
  int push_warps;                  // pusher warps that take jobs (1..kPusherWarps)
  int* progress;                   // 1 + the highest pair tile this rank's GEMM has started; the launcher
                                   // zeroes it on the stream before a paced launch
  int push_lead;                   // raster groups the pushers may run ahead of the GEMM (0 = unlimited)
  // MXFP8 (E4M3 operands, one E8M0 scale per 32 K elements, K step = 128 elements)
  int acc_stages;                  // TMEM accumulator stages: 2, or 1 when MXFP8 uses BN = 256
  int sfa_kblocks, sfb_kblocks;    // 128-element K blocks per 128-row block in the A / B scale layouts
  const uint16_t* quant_src;       // recv: this rank's BF16 receive buffer (source of the quantizer warps)
  uint8_t* quant_q;                // recv: local E4M3 copy of the receive buffer (the GEMM's A operand)
  uint8_t* quant_sf;               // recv: its E8M0 scales in the tcgen05 layout
  int quant_arrivals;              // recv: counter value at which a row block is complete in BF16
  // bounded waits
  int* status;
  unsigned long long timeout_ns;
};

struct WaitCtx {
  int* status;
  unsigned long long timeout_ns;
  uint32_t abort_flag;  // shared address of this CTA's abort word
  bool dead;
};

__device__ __forceinline__ void report(WaitCtx& w, int code, int where, int detail) {
  if (atomicCAS(w.status, 0, code) == 0) {
    w.status[1] = where;
    w.status[2] = detail;
  }
  asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(w.abort_flag), "r"(1u) : "memory");
  w.dead = true;
}

__device__ __forceinline__ bool should_abort(WaitCtx& w) {
  uint32_t f;
  asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(f) : "r"(w.abort_flag) : "memory");
  if (f != 0 || ld_relaxed_sys_s32(w.status) != 0) {
    w.dead = true;
    return true;
  }
  return false;
}

// Bounded mbarrier wait. Returns false when the kernel is aborting.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, WaitCtx& w, int where) {
  if (w.dead) return false;
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 0x3ff) == 0) {
      if (should_abort(w)) return false;
      if (globaltimer_ns() - t0 > w.timeout_ns) {
        report(w, kErrPipelineTimeout, where, static_cast<int>(bar));
        return false;
      }
    }
  }
  return true;
}

// Bounded acquire-poll of a global counter until it reaches `target`.
__device__ __forceinline__ bool counter_wait(const int* ctr, int target, WaitCtx& w, int where,
                                             int detail) {
  if (w.dead) return false;
  if (ld_acquire_sys_s32(ctr) >= target) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (ld_acquire_sys_s32(ctr) < target) {
    nanosleep(256);
    if ((++it & 0xff) == 0) {
      if (should_abort(w)) return false;
      if (globaltimer_ns() - t0 > w.timeout_ns) {
        report(w, kErrCounterTimeout, where, detail);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// The index arithmetic lives in schedule.cuh (shared with the host and the CPU tests); these are
// the kernel's views of it.
__device__ __forceinline__ void tile_coords(const GemmParams& P, int t, int& m, int& n) {
  sched::tile_coords(P.m_tiles, P.n_tiles, P.group_m, t, m, n);
}

__device__ __forceinline__ void unit_coords(const GemmParams& P, int u, int total_tiles, int& t, int& kt0,
                                            int& kt1) {
  sched::unit_coords(P.k_tiles, P.k_splits, total_tiles, u, t, kt0, kt1);
}

// First B row (weight row / output column) of N tile n. Push mode rotates the N order by rank.
__device__ __forceinline__ int b_row0_of(const GemmParams& P, int n) {
  if (P.mode == kPush) n = sched::rotated_n(n, P.n_rotate, P.n_tiles);
  return n * P.bn;
}

// ---------------------------------------------------------------------------------------------
// Pusher warps (recv mode). Job = (row block, input segment, destination, row sub-block): move
// rows [row0, row0 + 128/split) of this rank's head-side input for destination d into d's receive
// buffer, columns in Megatron order [head][q|k|v|g][D], rows past src_rows as zeros; then one
// release-increment of d's counter for that row block (fused_gemm_a2a_kernels.py:291-380 is the
// reference's register-copy version). Here one lane per warp drives the TMA unit: a chunk of up
// to 4 KiB is bulk-loaded from local memory into one of the warp's two shared buffers and
// bulk-stored to the peer in 256-byte head units (or whole rows when the columns are contiguous),
// so the data never passes through registers and remote stores queue in the copy engine.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void run_pushers(const GemmParams& P, int pusher, int lane, uint32_t buf0,
                                            uint32_t bar0, WaitCtx& w) {
  const int sub_rows = kTileM / P.split;
  const int jobs_per_block = P.num_in * P.p * P.split;
  const long long num_jobs = static_cast<long long>(P.m_tiles) * 2 * jobs_per_block;
  const bool paced = P.push_lead > 0 && P.progress != nullptr;
  uint32_t issued = 0;          // chunks issued by this warp (selects the buffer)
  uint32_t loads[2] = {0, 0};   // completed-load count per buffer (selects the barrier phase)
  auto do_job = [&](long long job) {
    const sched::PushJob j = sched::decode_push_job(job, P.num_in, P.p, P.split, P.rank);
    const int mi = j.mi, t = j.t, d = j.d, row0 = j.row0;
    // Geometry of this input: its rows are in_units[t] head units wide (the same for every input
    // unless query heads outnumber key/value heads).
    const int hpr = P.in_units[t];
    const int row_bytes = hpr * 256;
    const int upp = P.push_units[t], rpc = P.push_rows[t];
    const int chunk_row_bytes = upp * 256;
    const int chunks_per_job = sched::push_chunks_per_job(hpr, upp, rpc, sub_rows);
    if (paced) {
      // Pacing: stay at most push_lead raster groups ahead of this rank's own GEMM. Every rank runs
      // the same schedule, so the peers consume at about this rank's pace; pushing faster only
      // saturates the NVLink egress queue, behind which the GEMM's own loads then wait.
      const int need = ((mi >> 1) / P.group_m - P.push_lead) * P.group_m;  // pair tile that must have started
      if (need > 0 && lane == 0) {
        const uint64_t t0 = globaltimer_ns();
        uint32_t it = 0;
        while (ld_relaxed_sys_s32(P.progress) <= need) {
          nanosleep(200);
          if ((++it & 0xff) == 0) {
            if (should_abort(w)) break;
            if (globaltimer_ns() - t0 > w.timeout_ns) {
              report(w, kErrCounterTimeout, 41, mi);
              break;
            }
          }
        }
      }
      __syncwarp();
    }
    const char* src = static_cast<const char*>(P.src[t]) +
                      (static_cast<long long>(d) * P.src_rows + row0) * row_bytes;
    char* dst = reinterpret_cast<char*>(P.peer_recv[d]) + static_cast<long long>(row0) * P.recv_k * 2;
    for (int c = 0; c < chunks_per_job; ++c) {
      const sched::PushChunk ch = sched::push_chunk(c, hpr, upp, rpc, P.src_rows, row0);
      const int r0 = ch.r0, u0 = ch.u0, valid = ch.valid;  // valid: rows that exist in the source
      const int b = issued & 1;
      const uint32_t buf = buf0 + b * kPushBufBytes, bar = bar0 + 8 * b;
      if (lane == 0) bulk_wait_read<1>();  // the group that used this buffer last has left shared memory
      __syncwarp();
      if (lane == 0 && valid > 0) {
        mbar_arrive_expect_tx(bar, valid * chunk_row_bytes);
        bulk_load(buf, src + static_cast<long long>(r0) * row_bytes + u0 * 256, valid * chunk_row_bytes, bar);
      }
      if (valid < rpc) {  // rows beyond the logical count travel as exact zeros
        for (int o = valid * chunk_row_bytes + lane * 16; o < rpc * chunk_row_bytes; o += 512)
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(buf + o), "r"(0u) : "memory");
        fence_proxy_async_shared();
      }
      __syncwarp();
      if (lane == 0) {
        bool ok = true;
        if (valid > 0) {
          ok = mbar_wait(bar, loads[b] & 1, w, 40);
          ++loads[b];
        }
        if (ok) {
          for (int r = 0; r < rpc; ++r) {
            char* drow = dst + static_cast<long long>(r0 + r) * P.recv_k * 2;
            if (P.num_in == 1) {
              bulk_store(drow + sched::recv_column(P.rank, P.layout, 0, u0) * 2, buf + r * chunk_row_bytes,
                         chunk_row_bytes);
            } else {
              for (int u = 0; u < upp; ++u) {
                const long long col = sched::recv_column(P.rank, P.layout, t, u0 + u);
                bulk_store(drow + col * 2, buf + r * chunk_row_bytes + u * 256, 256);
              }
            }
          }
        }
        bulk_commit();
      }
      ++issued;
    }
    if (lane == 0) {
      // All of this job's bulk stores have been performed; the release makes them visible to
      // whoever acquires the counter.
      bulk_wait_all();
      fence_proxy_async_all();
      if (!w.dead) {
        int* ctr = reinterpret_cast<int*>(P.peer_counters[d]) + mi;
        red_release_sys_add(ctr, 1);
      }
    }
    w.dead = __shfl_sync(0xffffffffu, w.dead ? 1 : 0, 0) != 0;
  };
  // Two phases (as in fused_gemm_a2a_kernels.py:358-380): every pusher warp works on the first two
  // raster groups, which the GEMM cannot start without; afterwards only `push_warps` warps per CTA
  // continue, enough to stay ahead of the GEMM without saturating the NVLink egress queue that
  // the GEMM's own loads share.
  const long long first_jobs = sched::first_phase_jobs(P.m_tiles, P.group_m, P.num_in, P.p, P.split);
  for (long long job = blockIdx.x * kPusherWarps + pusher; job < first_jobs && !w.dead;
       job += static_cast<long long>(gridDim.x) * kPusherWarps)
    do_job(job);
  if (pusher < P.push_warps)
    for (long long job = first_jobs + blockIdx.x * P.push_warps + pusher; job < num_jobs && !w.dead;
         job += static_cast<long long>(gridDim.x) * P.push_warps)
      do_job(job);
  if (lane == 0) bulk_wait_all();
}

// ---------------------------------------------------------------------------------------------
// Receive-side quantizer warps (MXFP8 recv mode; the reference's _mx_quantize_received,
// fused_gemm_a2a_kernels.py:1295-1343). Only BF16 crosses the links. Job = 8 rows of a 128-row
// block: wait until the block's counter shows every BF16 arrival, quantize the rows along K into
// the local E4M3 copy and its scale bytes, then add one completion to the same counter; the TMA
// producer waits for arrivals + 16 completions before it loads the block.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void run_quantizers(const GemmParams& P, int worker_in_cta, int lane, WaitCtx& w) {
  const long long k = P.recv_k;
  const int groups = static_cast<int>(k >> 5);
  const long long jobs = static_cast<long long>(P.m_tiles) * 2 * 16;
  for (long long job = blockIdx.x * kQuantWarps + worker_in_cta; job < jobs && !w.dead;
       job += static_cast<long long>(gridDim.x) * kQuantWarps) {
    const int blk = static_cast<int>(job >> 4);
    bool ok = true;
    if (lane == 0) ok = counter_wait(P.counters + blk, P.quant_arrivals, w, 50, blk);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    __syncwarp();  // lane 0's acquire orders the other lanes' loads of the block behind it
    if (!ok) {
      w.dead = true;
      break;
    }
    for (int r = 0; r < 8; ++r) {
      const long long row = job * 8 + r;
      for (long long c0 = 0; c0 < k; c0 += 256) {
        const long long col = c0 + lane * 8;
        const bool active = col < k;  // K is a multiple of 32: whole 4-lane groups drop out together
        uint4 x = make_uint4(0, 0, 0, 0);
        if (active) x = __ldcg(reinterpret_cast<const uint4*>(P.quant_src + row * k + col));
        int sf_byte;
        const uint2 q = mx_quantize8(x, sf_byte);
        if (active) {
          *reinterpret_cast<uint2*>(P.quant_q + row * k + col) = q;
          if ((lane & 3) == 0)
            P.quant_sf[mx_scale_offset(row, static_cast<int>(col >> 5), groups)] = static_cast<uint8_t>(sf_byte);
        }
      }
    }
    __syncwarp();
    if (lane == 0) red_release_sys_add(P.counters + blk, 1);
  }
}

// ---------------------------------------------------------------------------------------------
// Epilogue for one 128-row x BN accumulator of this CTA. Thread = output row; the row leaves in
// 128-byte pieces (64 BF16 or 32 FP32 columns), each staged in the thread's own shared slot and
// shipped with one bulk copy, so no thread ever waits for another.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void epilogue_tile(const GemmParams& P, uint32_t tmem_acc, int quarter,
                                              int lane, uint32_t slot, int row, int b_row0,
                                              uint32_t tempty_leader, bool& stores_pending) {
  const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
  const bool bf16_out = P.epi == kEpiBf16;
  const int piece_cols = bf16_out ? 64 : 32;
  const int chunks = piece_cols >> 5;
  const int pieces = P.bn / piece_cols;
  for (int pc = 0; pc < pieces; ++pc) {
    const int col0 = pc * piece_cols;
    char* dst = nullptr;
    if (P.mode == kPush) {
      const sched::PushRoute route = sched::push_route(b_row0 + col0, P.layout);
      dst = reinterpret_cast<char*>(P.peer_heads[route.segment][route.dest]) +
            sched::push_element(route, P.rank, P.head_rows, row) * 2;
    } else if (row < P.c_rows) {
      dst = static_cast<char*>(P.c) +
            (static_cast<long long>(row) * P.c_pitch + b_row0 + col0) * (bf16_out ? 2 : 4);
    }
    if (stores_pending) bulk_wait_read_all();
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(tmem_acc + lane_base + col0 + c * 32, r);
      tmem_ld_wait();
      if (pc == pieces - 1 && c == chunks - 1) {
        // Last TMEM read of this accumulator stage: hand it back to the MMA thread.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader);
      }
      if (bf16_out) {
        if (P.bias != nullptr) {
          const uint4* bp = reinterpret_cast<const uint4*>(P.bias + b_row0 + col0 + c * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 b = __ldg(bp + v);
            const uint32_t wv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              r[v * 8 + e * 2] = __float_as_uint(__uint_as_float(r[v * 8 + e * 2]) +
                                                 bf16_bits_to_f32(wv[e] & 0xffffu));
              r[v * 8 + e * 2 + 1] = __float_as_uint(__uint_as_float(r[v * 8 + e * 2 + 1]) +
                                                     bf16_bits_to_f32(wv[e] >> 16));
            }
          }
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint32_t a0 = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
          const uint32_t a1 = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
          const uint32_t a2 = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
          const uint32_t a3 = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(slot + c * 64 + v * 16),
                       "r"(a0), "r"(a1), "r"(a2), "r"(a3)
                       : "memory");
        }
      } else {
#pragma unroll
        for (int v = 0; v < 8; ++v)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(slot + v * 16), "r"(r[v * 4]),
                       "r"(r[v * 4 + 1]), "r"(r[v * 4 + 2]), "r"(r[v * 4 + 3])
                       : "memory");
      }
    }
    fence_proxy_async_shared();
    if (dst != nullptr) {
      if (P.epi == kEpiF32Add)
        bulk_reduce_add_f32(dst, slot, kPieceBytes);
      else
        bulk_store(dst, slot, kPieceBytes);
      bulk_commit();
      stores_pending = true;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The kernel. blockDim = 192 (local, push), 320 (recv: + 4 pusher warps) or 384 (MXFP8 recv: + 2
// quantizer warps). Grid = 2 * pairs.
// ---------------------------------------------------------------------------------------------
template <bool kMx>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(32 * (kGemmWarps + kPusherWarps + kQuantWarps), 1)
    ulysses_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_sfa,
                        const __grid_constant__ CUtensorMap tmap_sfb,
                        const __grid_constant__ GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t push_bufs = smem_base + (kMaxStages - 1) * kStageBytes;  // recv mode: sixth stage
  const uint32_t staging = smem_base + kMaxStages * kStageBytes;
  const uint32_t sf0 = staging + kStagingBytes;  // MXFP8 scale stages
  const uint32_t bars = sf0 + kMaxStages * kSfStageBytes;
  // barrier layout (8 bytes each): full[6], empty[6], tfull[2], tempty[2], pusher[4][2]
  const uint32_t full0 = bars, empty0 = bars + 8 * kMaxStages, tfull0 = bars + 16 * kMaxStages,
                 tempty0 = tfull0 + 16, push_bar0 = tempty0 + 16,
                 tmem_slot = push_bar0 + 16 * kPusherWarps, abort_word = tmem_slot + 8;
  static_assert(16 * kMaxStages + 32 + 16 * kPusherWarps + 16 <= kBarrierBytes, "barrier area");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int total_tiles = P.m_tiles * P.n_tiles;
  const int total_units = total_tiles * max(1, P.k_splits);
  const bool gemm_on = (P.roles & 1) != 0;
  const int stages = P.stages;

  // A device error recorded by an earlier kernel is sticky: every role starts out aborted, so no
  // peer memory is touched (the peer that never answered may be gone) until the host clears it.
  WaitCtx w{P.status, P.timeout_ns, abort_word, ld_relaxed_sys_s32(P.status) != 0};

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(full0 + 8 * i, 1);   // leader producer's arrive.expect_tx (+ both CTAs' bytes)
      mbar_init(empty0 + 8 * i, 1);  // one tcgen05.commit arrival per use
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull0 + 8 * i, 1);   // one tcgen05.commit arrival per tile
      mbar_init(tempty0 + 8 * i, 8);  // 4 epilogue warps x 2 CTAs
    }
    for (int i = 0; i < 2 * kPusherWarps; ++i) mbar_init(push_bar0 + 8 * i, 1);
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_word), "r"(0u) : "memory");
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0 && gemm_on) {
      const uint32_t tx_bytes =
          2u * (kABytes + (P.bn >> 1) * 128u + (kMx ? 512u + (P.bn >> 7) * 512u : 0u));
      const int b_half = P.bn >> 1;
      int s = 0;
      uint32_t ph = 0;
      for (int u = pair; u < total_units && !w.dead; u += pairs) {
        int t, kt0, kt1, m, n;
        unit_coords(P, u, total_tiles, t, kt0, kt1);
        tile_coords(P, t, m, n);
        const int a_row0 = m * 256 + static_cast<int>(cta_rank) * kTileM;
        const int b_row0 = b_row0_of(P, n) + static_cast<int>(cta_rank) * b_half;
        if (P.mode == kRecv) {
          // Acquire this CTA's row block from every source, then order the TMA reads after it.
          const int blk = m * 2 + static_cast<int>(cta_rank);
          if (!counter_wait(P.counters + blk, P.target, w, 10, blk)) break;
          fence_proxy_async_global();
          if (P.push_lead > 0 && P.progress != nullptr) atomicMax(P.progress, m + 1);
        }
        for (int kt = kt0; kt < kt1; ++kt) {
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1, w, 11)) break;
          const uint32_t a_dst = smem_base + s * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const uint32_t full_leader = mapa(full0 + 8 * s, 0);
          if (leader) mbar_arrive_expect_tx(full0 + 8 * s, tx_bytes);
          const int k0 = kt * (kMx ? 128 : kTileK);
          if constexpr (kMx) {
            // Scale blocks of this K step: 512 B for this CTA's 128 rows of A, and one block per
            // 128 columns of the whole N tile (both CTAs multiply their rows by every column).
            const uint32_t sf_dst = sf0 + s * kSfStageBytes;
            tma_load_2d_pair(sf_dst, &tmap_sfa, full_leader, 0, (a_row0 >> 7) * P.sfa_kblocks + kt);
            const int nb0 = b_row0_of(P, n) >> 7;
            for (int i = 0; i < (P.bn >> 7); ++i)
              tma_load_2d_pair(sf_dst + 512 + i * 512, &tmap_sfb, full_leader, 0, (nb0 + i) * P.sfb_kblocks + kt);
          }
          if (!P.a_mn) {
            tma_load_2d_pair(a_dst, &tmap_a, full_leader, k0, a_row0);
          } else {
            tma_load_2d_pair(a_dst, &tmap_a, full_leader, a_row0, k0);
            tma_load_2d_pair(a_dst + 8192, &tmap_a, full_leader, a_row0 + 64, k0);
          }
          if (!P.b_mn) {
            tma_load_2d_pair(b_dst, &tmap_b, full_leader, k0, b_row0);
          } else {
            tma_load_2d_pair(b_dst, &tmap_b, full_leader, b_row0, k0);
            if (b_half > 64) tma_load_2d_pair(b_dst + 8192, &tmap_b, full_leader, b_row0 + 64, k0);
          }
          if (++s == stages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (lane == 0 && leader && gemm_on) {
      // Shared-memory matrix descriptors: SWIZZLE_128B, descriptor version 1.
      //   K-major : 8-row groups 1024 B apart (SBO); one UMMA_K (16 elements) = 32 bytes.
      //   MN-major: 64-element chunks 8192 B apart (LBO), 8-K-row groups 1024 B apart (SBO);
      //             one UMMA_K = 16 K rows = 2048 bytes.
      const uint64_t desc_hi = (static_cast<uint64_t>(64u | (1u << 14) | (2u << 29))) << 32;
      const uint32_t a_lbo = P.a_mn ? 512u : 1u, b_lbo = P.b_mn ? 512u : 1u;
      const uint32_t a_step = P.a_mn ? 128u : 2u, b_step = P.b_mn ? 128u : 2u;
      int s = 0, as = 0;
      uint32_t ph = 0, aph = 0;
      for (int u = pair; u < total_units && !w.dead; u += pairs) {
        int t, kt0, kt1;
        unit_coords(P, u, total_tiles, t, kt0, kt1);
        if (!mbar_wait(tempty0 + 8 * as, aph ^ 1, w, 20)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * P.bn;
        for (int kt = kt0; kt < kt1; ++kt) {
          if (!mbar_wait(full0 + 8 * s, ph, w, 21)) break;
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * kStageBytes;
          const uint32_t b_addr = a_addr + kABytes;
          const uint64_t adesc = desc_hi | ((a_addr >> 4) & 0x3fffu) | (a_lbo << 16);
          const uint64_t bdesc = desc_hi | ((b_addr >> 4) & 0x3fffu) | (b_lbo << 16);
          if constexpr (kMx) {
            // Scales: shared -> TMEM (lane = row % 32, column = row / 32, byte = K group), then four
            // K = 32 MMAs whose descriptors select byte 0..3 of those columns.
            const uint32_t sf_addr = sf0 + s * kSfStageBytes;
            const uint64_t sf_hi = (static_cast<uint64_t>(8u | (1u << 14))) << 32;  // SBO 128 B, no swizzle
            const uint32_t sfa_t = tmem_base + 256, sfb_t = tmem_base + 260;
            tc_cp_sf_pair(sfa_t, sf_hi | ((sf_addr >> 4) & 0x3fffu) | (1u << 16));
            for (int i = 0; i < (P.bn >> 7); ++i)
              tc_cp_sf_pair(sfb_t + 4 * i, sf_hi | (((sf_addr + 512 + i * 512) >> 4) & 0x3fffu) | (1u << 16));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_mxf8_pair(d_tmem, adesc + k * 2, bdesc + k * 2,
                            P.idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29), sfa_t,
                            sfb_t, (kt != kt0 || k != 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_bf16_pair(d_tmem, adesc + k * a_step, bdesc + k * b_step, P.idesc,
                            (kt != kt0 || k != 0) ? 1u : 0u);
          }
          tc_commit_pair(empty0 + 8 * s, 3);  // frees the stage in both CTAs when the MMAs retire
          if (++s == stages) {
            s = 0;
            ph ^= 1;
          }
        }
        if (w.dead) break;
        tc_commit_pair(tfull0 + 8 * as, 3);  // accumulator ready in both CTAs
        if (++as == P.acc_stages) {
          as = 0;
          aph ^= 1;
        }
      }
    }
  } else if (warp < kGemmWarps) {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    if (gemm_on) {
      const int quarter = warp & 3;  // TMEM lane quarter this warp may read
      const int row_in_cta = quarter * 32 + lane;
      const uint32_t slot = staging + row_in_cta * kSlotPitch;
      bool stores_pending = false;
      int as = 0;
      uint32_t aph = 0;
      for (int u = pair; u < total_units; u += pairs) {
        int t, kt0, kt1, m, n;
        unit_coords(P, u, total_tiles, t, kt0, kt1);
        tile_coords(P, t, m, n);
        const bool ok = mbar_wait(tfull0 + 8 * as, aph, w, 30);
        // All lanes take the same branch: the barrier state is CTA-wide and aborts are sticky.
        if (!__all_sync(0xffffffffu, ok)) {
          w.dead = true;
          break;
        }
        tc_fence_after();
        const int row = m * 256 + static_cast<int>(cta_rank) * kTileM + row_in_cta;
        epilogue_tile(P, tmem_base + as * P.bn, quarter, lane, slot, row, b_row0_of(P, n),
                      mapa(tempty0 + 8 * as, 0), stores_pending);
        if (++as == P.acc_stages) {
          as = 0;
          aph ^= 1;
        }
      }
      // Writes (local or remote) are complete before the kernel ends; the group barrier that
      // follows a push publishes them with a system-scope release.
      bulk_wait_all();
      if (P.mode == kPush) fence_acq_rel_sys();
    }
  } else if (warp < kGemmWarps + kPusherWarps) {
    // ------------------------------------------------------------------ pusher warps (recv mode)
    if (P.mode == kRecv && (P.roles & 2) != 0) {
      const int pusher = warp - kGemmWarps;
      run_pushers(P, pusher, lane, push_bufs + pusher * 2 * kPushBufBytes, push_bar0 + 16 * pusher, w);
    }
  } else {
    // ------------------------------------------------------------------ quantizer warps (MXFP8 recv)
    if constexpr (kMx) {
      if (P.mode == kRecv && gemm_on) run_quantizers(P, warp - kGemmWarps - kPusherWarps, lane, w);
    }
  }

  // Teardown: nobody leaves while the pair may still touch this CTA's shared memory or TMEM.
  __syncwarp();
  if (should_abort(w)) {
    // Loads that were issued but never consumed may still be landing in shared memory.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) nanosleep(1000);
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace fga
