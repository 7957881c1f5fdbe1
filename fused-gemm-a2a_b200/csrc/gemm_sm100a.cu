// Host launchers of the persistent tcgen05 GEMM (gemm_sm100a.cuh): argument validation, TMA
// descriptor encoding per call (a few hundred nanoseconds of host work, so a changing token count
// never recompiles anything), grid sizing from the number of co-resident CTA pairs.
#include <cstdlib>
#include <cstring>
#include "../../include/fga.h"
#include "gemm_sm100a.cuh"

namespace fga {

static int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  const int x = atoi(v);
  return x > 0 ? x : fallback;
}

// CTA pairs that can be resident at once. A persistent grid never exceeds it: in recv mode the
// resident CTAs wait for pusher jobs of every CTA of every rank, so a CTA that is not resident
// would deadlock the group.
static int resident_pairs(bool mx, int threads, int* out) {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices][2][3];  // 0 = not queried yet; racing threads compute the same value
  int dev = 0;
  FGA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return set_error(kUnsupported, "device index %d out of range", dev);
  const int slot = threads <= 32 * kGemmWarps ? 0 : (threads <= 32 * (kGemmWarps + kPusherWarps) ? 1 : 2);
  int& slot_ref = cached[dev][mx ? 1 : 0][slot];
  int entry = __atomic_load_n(&slot_ref, __ATOMIC_RELAXED);
  if (entry == 0) {
    const void* fn = mx ? reinterpret_cast<const void*>(ulysses_gemm_kernel<true>)
                        : reinterpret_cast<const void*>(ulysses_gemm_kernel<false>);
    FGA_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    FGA_CUDA(cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg));
    if (clusters < 1) return set_error(kCudaError, "no CTA pair of the GEMM kernel fits on this device");
    entry = clusters;
    __atomic_store_n(&slot_ref, entry, __ATOMIC_RELAXED);
  }
  *out = entry;
  return kSuccess;
}

static uint32_t make_idesc(int a_mn, int b_mn, int bn) {
  // FP32 accumulate, BF16 x BF16, M = 256 across the CTA pair, N = bn.
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn) << 15) |
         (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(bn >> 3) << 17) |
         (static_cast<uint32_t>(256 >> 4) << 24);
}

// A/B descriptors. K-major operand [rows, k]: box = 64 K-elements x `box_rows` rows.
// MN-major operand stored as [k, rows]: box = 64 rows-elements x 64 K rows.
static int encode_operand(CUtensorMap* map, const void* base, int mn_major, long long rows,
                          long long k, long long pitch, int box_rows) {
  if (!mn_major)
    return encode_tmap_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, k, pitch, box_rows, 64);
  return encode_tmap_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, rows, pitch, 64, 64);
}

static int launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams P, cudaStream_t stream,
                  const CUtensorMap* tsa = nullptr, const CUtensorMap* tsb = nullptr) {
  const bool mx = tsa != nullptr;
  const int forced_stages = env_int("FGA_STAGES", 0);  // tuning knob: fewer pipeline stages
  if (forced_stages >= 2 && forced_stages <= P.stages) P.stages = forced_stages;
  if (P.acc_stages == 0) P.acc_stages = 2;
  if (P.k_splits < 1) P.k_splits = 1;
  const int threads =
      32 * (kGemmWarps + (P.mode == kRecv ? kPusherWarps + (mx ? kQuantWarps : 0) : 0));
  int pairs = 0;
  const int rc = resident_pairs(mx, threads, &pairs);
  if (rc != kSuccess) return rc;
  const long long units = static_cast<long long>(P.m_tiles) * P.n_tiles * P.k_splits;
  if (P.mode != kRecv && units < pairs) pairs = static_cast<int>(units);
  if (mx)
    ulysses_gemm_kernel<true><<<2 * pairs, threads, kSmemBytes, stream>>>(ta, tb, *tsa, *tsb, P);
  else
    ulysses_gemm_kernel<false><<<2 * pairs, threads, kSmemBytes, stream>>>(ta, tb, ta, tb, P);
  FGA_LAUNCHED();
  return kSuccess;
}

// Shares of the K steps per output tile for an FP32 gradient GEMM. A persistent grid of `pairs`
// CTA pairs runs ceil(tiles / pairs) waves and the last one may be mostly empty (256 tiles on 74
// pairs: 3.46 waves, 86 % efficiency). Cutting K multiplies the work units and fills the last wave;
// every unit adds its partial tile with bulk reductions, so no second pass is needed.
// FGA_WGRAD_SPLITS selects it: unset or 1 = one unit per tile (the default), N = N shares,
// "auto" = the smallest count that reaches 97 % wave efficiency. A share keeps at least 32 K steps.
static int choose_k_splits(long long tiles, int k_tiles, int pairs) {
  const char* v = getenv("FGA_WGRAD_SPLITS");
  if (v == nullptr || *v == '\0') return 1;
  if (strcmp(v, "auto") == 0) return sched::pick_k_splits(tiles, k_tiles, pairs, 0);
  const int forced = atoi(v);
  return forced <= 1 ? 1 : sched::pick_k_splits(tiles, k_tiles, pairs, forced);
}

// Optional pacing of the recv pushers (FGA_PUSH_LEAD = raster groups they may run ahead of this
// rank's own GEMM; off by default). The GEMM publishes 1 + the pair tile it has started in
// `progress`, which is zeroed on the stream in front of the launch (a memset node under capture).
// Only launches that run both roles are paced: pushers without a GEMM would wait for nothing.
static int pace_pushers(GemmParams& P, int32_t* progress, cudaStream_t stream) {
  P.progress = nullptr;
  P.push_lead = 0;
  const int lead = env_int("FGA_PUSH_LEAD", 0);
  if (lead <= 0 || progress == nullptr || P.roles != 3) return kSuccess;
  FGA_CUDA(cudaMemsetAsync(progress, 0, sizeof(int32_t), stream));
  P.progress = progress;
  P.push_lead = lead;
  return kSuccess;
}

// N tile of a block-scaled GEMM: 256 columns where the widths allow it, with a single accumulator
// stage (the scale columns take the TMEM that a second 256-column stage would need, so a tile's
// epilogue does not overlap the next tile's mainloop), else 128 columns with two stages.
// FGA_MX_TILE_N=128 forces the narrow, double-buffered form everywhere, for measuring one against
// the other; both forms are the same code path with different tile counts.
static int mx_tile_n(bool wide_allowed) {
  return wide_allowed && env_int("FGA_MX_TILE_N", 256) != 128 ? 256 : 128;
}

// Block-scaled instruction descriptor: E4M3 x E4M3, E8M0 scales, M = 256 across the pair, N = bn.
// The scale-byte selectors (bits 4-5 and 29-30) are filled in per K block by the kernel.
static uint32_t make_idesc_mx(int bn) {
  return (static_cast<uint32_t>(bn >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(256 >> 4) << 24);
}

// E4M3 operand [rows, kp] (K-major, 128-byte K steps) and its scale blocks [blocks, 512 B].
static int encode_mx_operand(CUtensorMap* data, CUtensorMap* scales, const void* q, const void* sf,
                             long long rows_padded, long long kp, int box_rows) {
  int rc = encode_tmap_2d(data, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows_padded, kp, kp, box_rows, 128);
  if (rc != kSuccess) return rc;
  const long long blocks = (rows_padded / 128) * (kp / 128);
  return encode_tmap_2d(scales, sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, blocks, 128, 128, 1, 128, false);
}

// Push-mode fields shared by the BF16 and MXFP8 launchers and by the uniform and grouped-query head
// layouts: `n` output columns = p * layout.groups_per_rank groups of group_units 128-wide units.
static void fill_push(GemmParams& P, int n, const sched::HeadLayout& layout, const int64_t* const* peer_heads,
                      int kinds, int64_t head_rows, int rank, int p, const void* bias, int32_t* status,
                      uint64_t timeout_ns) {
  P.mode = kPush;
  P.epi = kEpiBf16;
  P.n_tiles = n / P.bn;
  P.group_m = env_int("FGA_GROUP_M_PUSH", 16);
  P.stages = kMaxStages;
  P.rank = rank;
  P.p = p;
  P.bias = static_cast<const uint16_t*>(bias);
  for (int s = 0; s < 4; ++s)
    P.peer_heads[s] = reinterpret_cast<const long long*>(peer_heads[s < kinds ? s : 0]);
  P.layout = layout;
  P.head_rows = head_rows;
  P.n_rotate = (P.n_tiles % p == 0) ? rank * (P.n_tiles / p) : 0;
  P.roles = 1;
  P.status = status;
  P.timeout_ns = timeout_ns;
}

// Recv-mode fields shared the same way. Input t (t < num_in) is of kind t; its rows are
// kind_pitch_units(layout, t) head units wide.
static void fill_recv(GemmParams& P, int recv_rows, int k, int n, void* c, const sched::HeadLayout& layout,
                      const int64_t* peer_recv, const int64_t* peer_counters, int32_t* counters,
                      const void* const* srcs, int num_in, int src_rows, int split, int rank, int p, int roles,
                      int32_t* status, uint64_t timeout_ns) {
  P.mode = kRecv;
  P.epi = kEpiBf16;
  P.m_tiles = recv_rows / 256;
  P.n_tiles = n / P.bn;
  P.group_m = env_int("FGA_GROUP_M_RECV", 4);
  P.stages = kMaxStages - 1;  // the sixth stage's shared memory holds the pusher buffers
  P.rank = rank;
  P.p = p;
  P.c = c;
  P.c_pitch = n;
  P.c_rows = recv_rows;
  P.layout = layout;
  P.counters = counters;
  P.peer_recv = reinterpret_cast<const long long*>(peer_recv);
  P.peer_counters = reinterpret_cast<const long long*>(peer_counters);
  for (int t = 0; t < 4; ++t) {
    const int kind = t < num_in ? t : 0;
    P.src[t] = srcs[kind];
    P.in_units[t] = sched::kind_pitch_units(layout, kind);
    // Pusher chunking: a chunk is `push_rows` rows of `push_units` 256-byte head units, at most
    // one 4 KiB buffer. Rows wider than a buffer are cut into equal pieces of whole units.
    sched::push_chunking(P.in_units[t], 128 / split, kPushBufBytes, P.push_units[t], P.push_rows[t]);
  }
  P.num_in = num_in;
  P.src_rows = src_rows;
  P.split = split;
  P.recv_k = k;
  P.roles = roles;
  // Warps per CTA that keep pushing after the first groups: all of them while at least half of the
  // traffic stays on this GPU, two once most of it crosses NVLink (more only congest the egress
  // queue that the GEMM's own loads share).
  P.push_warps = env_int("FGA_PUSHER_WARPS", p <= 2 ? kPusherWarps : 2);
  if (P.push_warps > kPusherWarps) P.push_warps = kPusherWarps;
  P.status = status;
  P.timeout_ns = timeout_ns;
}

// The grouped-query layout of kv_heads groups over p ranks (q_per_kv query heads per key/value head).
static sched::HeadLayout grouped_layout(int kv_heads, int q_per_kv, int gate, int p) {
  sched::HeadLayout l;
  l.q_units = q_per_kv;
  l.kv_units = 1;
  l.gate_units = gate ? q_per_kv : 0;
  l.groups_per_rank = kv_heads / p;
  return l;
}

}  // namespace fga

using namespace fga;

extern "C" {

int fga_gemm_push(const void* a, int m, int k, int a_rows, const void* b, int b_is_kn,
                  const void* bias, int segments, int n_segment, const int64_t* const* peer_heads,
                  int64_t head_rows, int rank, int p, int32_t* status, uint64_t timeout_ns,
                  void* stream) {
  FGA_REQUIRE(a && b && peer_heads && status, "fga_gemm_push: null operand, peer table or status");
  FGA_REQUIRE(segments == 1 || segments == 3 || segments == 4,
              "Expected one output projection or three/four QKV projections");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_push: bad rank %d of %d", rank, p);
  FGA_REQUIRE(m >= 1 && k >= 8 && k % 8 == 0, "fga_gemm_push: m >= 1 and k a multiple of 8");
  FGA_REQUIRE(a_rows >= m && a_rows % 256 == 0 && a_rows <= head_rows,
              "a_rows must be a tile multiple >= the rows of a and fit the head-side rank block");
  FGA_REQUIRE(n_segment > 0 && n_segment % (p * 128) == 0,
              "Push segment width must be a multiple of CP * tile N");
  for (int s = 0; s < segments; ++s) FGA_REQUIRE(peer_heads[s], "fga_gemm_push: null peer table %d", s);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(bias) % 16 == 0, "fga_gemm_push: the bias must be 16-byte aligned");
  const int n = segments * n_segment;
  GemmParams P{};
  P.bn = (n / 128) % 2 == 0 ? 256 : 128;
  P.m_tiles = a_rows / 256;
  P.k_tiles = (k + kTileK - 1) / kTileK;
  P.a_mn = 0;
  P.b_mn = b_is_kn ? 1 : 0;
  P.idesc = make_idesc(P.a_mn, P.b_mn, P.bn);
  fill_push(P, n, sched::uniform_layout(segments, n_segment / p / 128), peer_heads, segments, head_rows, rank, p,
            bias, status, timeout_ns);
  CUtensorMap ta, tb;
  int rc = encode_operand(&ta, a, 0, m, k, k, 128);
  if (rc != kSuccess) return rc;
  rc = b_is_kn ? encode_operand(&tb, b, 1, n, k, n, 0) : encode_operand(&tb, b, 0, n, k, k, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream));
}

int fga_gemm_recv(const void* recv, int recv_rows, int k, const void* b, int b_is_kn, int n,
                  void* c, const int64_t* peer_recv, const int64_t* peer_counters,
                  int32_t* counters, const void* const* srcs, int num_in, int src_rows, int split,
                  int rank, int p, int roles, const int64_t* epoch, int32_t* progress, int32_t* status,
                  uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(recv && b && c && peer_recv && peer_counters && counters && srcs && status,
              "fga_gemm_recv: null argument");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_recv: bad rank %d of %d", rank, p);
  FGA_REQUIRE(num_in == 1 || num_in == 3 || num_in == 4,
              "Expected one output projection or three/four QKV projections");
  FGA_REQUIRE(recv_rows >= 256 && recv_rows % 256 == 0, "fga_gemm_recv: receive rows must be a multiple of 256");
  FGA_REQUIRE(src_rows >= 1 && src_rows <= recv_rows,
              "Receive source rows must be positive and fit the receive buffer");
  FGA_REQUIRE(k % (p * num_in * 128) == 0, "Receive K must split evenly over peers and input segments");
  FGA_REQUIRE(n >= 128 && n % 128 == 0, "GEMM mode must be push/recv and tile N must divide output width");
  FGA_REQUIRE(split >= 1 && 128 % split == 0, "FUSED_PUSH_SPLIT must divide 128");
  FGA_REQUIRE((roles & 3) != 0 && (roles & ~3) == 0, "fga_gemm_recv: roles is a mask of 1 (GEMM) and 2 (pushers)");
  for (int t = 0; t < num_in; ++t)
    FGA_REQUIRE(srcs[t] && reinterpret_cast<uintptr_t>(srcs[t]) % 16 == 0,
                "fga_gemm_recv: source %d must be a 16-byte aligned device pointer", t);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(c) % 16 == 0, "fga_gemm_recv: output must be 16-byte aligned");
  GemmParams P{};
  P.bn = n % 256 == 0 ? 256 : 128;
  P.k_tiles = k / kTileK;
  P.a_mn = 0;
  P.b_mn = b_is_kn ? 1 : 0;
  P.idesc = make_idesc(P.a_mn, P.b_mn, P.bn);
  fill_recv(P, recv_rows, k, n, c, sched::uniform_layout(num_in, k / (p * num_in * 128)), peer_recv, peer_counters,
            counters, srcs, num_in, src_rows, split, rank, p, roles, status, timeout_ns);
  P.target = p * num_in * split;
  (void)epoch;
  int rc = pace_pushers(P, progress, static_cast<cudaStream_t>(stream));
  if (rc != kSuccess) return rc;
  P.status = status;
  P.timeout_ns = timeout_ns;
  CUtensorMap ta, tb;
  rc = encode_operand(&ta, recv, 0, recv_rows, k, k, 128);
  if (rc != kSuccess) return rc;
  rc = b_is_kn ? encode_operand(&tb, b, 1, n, k, n, 0) : encode_operand(&tb, b, 0, n, k, k, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream));
}

// ---- grouped-query attention: more query heads than key/value heads -----------------------------
// Same kernels, with the output columns (push) / receive-buffer columns (recv) grouped per
// key/value head: [q_g0 .. q_g(r-1); k_g; v_g; (gate_g0 .. gate_g(r-1))], r = q_per_kv.

int fga_gemm_push_gqa(const void* a, int m, int k, int a_rows, const void* b, const void* bias, int kv_heads,
                      int q_per_kv, int gate, const int64_t* const* peer_heads, int64_t head_rows, int rank,
                      int p, int32_t* status, uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(a && b && peer_heads && status, "fga_gemm_push_gqa: null operand, peer table or status");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_push_gqa: bad rank %d of %d", rank, p);
  FGA_REQUIRE(kv_heads >= 1 && kv_heads % p == 0 && q_per_kv >= 1 && q_per_kv <= 64,
              "Key/value heads must split evenly over CP ranks (kv_heads=%d, q_per_kv=%d, p=%d)", kv_heads,
              q_per_kv, p);
  FGA_REQUIRE(m >= 1 && k >= 8 && k % 8 == 0, "fga_gemm_push_gqa: m >= 1 and k a multiple of 8");
  FGA_REQUIRE(a_rows >= m && a_rows % 256 == 0 && a_rows <= head_rows,
              "a_rows must be a tile multiple >= the rows of a and fit the head-side rank block");
  const int kinds = gate ? 4 : 3;
  for (int s = 0; s < kinds; ++s) FGA_REQUIRE(peer_heads[s], "fga_gemm_push_gqa: null peer table %d", s);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(bias) % 16 == 0, "fga_gemm_push_gqa: the bias must be 16-byte aligned");
  const sched::HeadLayout layout = grouped_layout(kv_heads, q_per_kv, gate, p);
  const long long units = static_cast<long long>(kv_heads) * sched::group_units(layout);
  FGA_REQUIRE(units * 128 <= 2147483647LL, "fga_gemm_push_gqa: too many output columns");
  const int n = static_cast<int>(units) * 128;
  GemmParams P{};
  P.bn = units % 2 == 0 ? 256 : 128;
  P.m_tiles = a_rows / 256;
  P.k_tiles = (k + kTileK - 1) / kTileK;
  P.a_mn = 0;
  P.b_mn = 0;
  P.idesc = make_idesc(P.a_mn, P.b_mn, P.bn);
  fill_push(P, n, layout, peer_heads, kinds, head_rows, rank, p, bias, status, timeout_ns);
  CUtensorMap ta, tb;
  int rc = encode_operand(&ta, a, 0, m, k, k, 128);
  if (rc != kSuccess) return rc;
  rc = encode_operand(&tb, b, 0, n, k, k, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream));
}

int fga_gemm_recv_gqa(const void* recv, int recv_rows, const void* b, int n, void* c, const int64_t* peer_recv,
                      const int64_t* peer_counters, int32_t* counters, const void* const* srcs, int kv_heads,
                      int q_per_kv, int gate, int src_rows, int split, int rank, int p, int roles,
                      int32_t* progress, int32_t* status, uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(recv && b && c && peer_recv && peer_counters && counters && srcs && status,
              "fga_gemm_recv_gqa: null argument");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_recv_gqa: bad rank %d of %d", rank, p);
  FGA_REQUIRE(kv_heads >= 1 && kv_heads % p == 0 && q_per_kv >= 1 && q_per_kv <= 64,
              "Key/value heads must split evenly over CP ranks (kv_heads=%d, q_per_kv=%d, p=%d)", kv_heads,
              q_per_kv, p);
  FGA_REQUIRE(recv_rows >= 256 && recv_rows % 256 == 0, "fga_gemm_recv_gqa: receive rows must be a multiple of 256");
  FGA_REQUIRE(src_rows >= 1 && src_rows <= recv_rows,
              "Receive source rows must be positive and fit the receive buffer");
  FGA_REQUIRE(n >= 128 && n % 128 == 0, "GEMM mode must be push/recv and tile N must divide output width");
  FGA_REQUIRE(split >= 1 && 128 % split == 0, "FUSED_PUSH_SPLIT must divide 128");
  FGA_REQUIRE((roles & 3) != 0 && (roles & ~3) == 0, "fga_gemm_recv_gqa: roles is a mask of 1 (GEMM) and 2 (pushers)");
  const int num_in = gate ? 4 : 3;
  for (int t = 0; t < num_in; ++t)
    FGA_REQUIRE(srcs[t] && reinterpret_cast<uintptr_t>(srcs[t]) % 16 == 0,
                "fga_gemm_recv_gqa: source %d must be a 16-byte aligned device pointer", t);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(c) % 16 == 0, "fga_gemm_recv_gqa: output must be 16-byte aligned");
  const sched::HeadLayout layout = grouped_layout(kv_heads, q_per_kv, gate, p);
  const long long units = static_cast<long long>(kv_heads) * sched::group_units(layout);
  FGA_REQUIRE(units * 128 <= 2147483647LL, "fga_gemm_recv_gqa: receive rows too wide");
  const int k = static_cast<int>(units) * 128;
  GemmParams P{};
  P.bn = n % 256 == 0 ? 256 : 128;
  P.k_tiles = k / kTileK;
  P.a_mn = 0;
  P.b_mn = 1;   // the weight is [k, n]: dX = dY * W
  P.idesc = make_idesc(P.a_mn, P.b_mn, P.bn);
  fill_recv(P, recv_rows, k, n, c, layout, peer_recv, peer_counters, counters, srcs, num_in, src_rows, split, rank,
            p, roles, status, timeout_ns);
  P.target = p * num_in * split;
  int rc = pace_pushers(P, progress, static_cast<cudaStream_t>(stream));
  if (rc != kSuccess) return rc;
  CUtensorMap ta, tb;
  rc = encode_operand(&ta, recv, 0, recv_rows, k, k, 128);
  if (rc != kSuccess) return rc;
  rc = encode_operand(&tb, b, 1, n, k, n, 0);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream));
}

int fga_gemm_local(const void* a, int a_is_km, const void* b, int b_is_kn, int m, int n, int k,
                   int64_t lda, int64_t ldb, void* c, int64_t ldc, int out_f32, int accumulate,
                   int32_t* status, uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(a && b && c && status, "fga_gemm_local: null argument");
  FGA_REQUIRE(m >= 1 && k >= 1 && n >= 128 && n % 128 == 0,
              "fga_gemm_local: n must be a positive multiple of 128");
  FGA_REQUIRE(!accumulate || out_f32, "MXFP8 gradient accumulation requires FP32 output");
  FGA_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldc >= n && (ldc * (out_f32 ? 4 : 2)) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(c) % 16 == 0,
              "fga_gemm_local: operands need 16-byte aligned rows");
  GemmParams P{};
  P.mode = kLocal;
  P.epi = out_f32 ? (accumulate ? kEpiF32Add : kEpiF32Store) : kEpiBf16;
  P.bn = n % 256 == 0 ? 256 : 128;
  P.m_tiles = (m + 255) / 256;
  P.n_tiles = n / P.bn;
  P.k_tiles = (k + kTileK - 1) / kTileK;
  P.group_m = env_int("FGA_GROUP_M_LOCAL", 8);
  P.stages = kMaxStages;
  P.a_mn = a_is_km ? 1 : 0;
  P.b_mn = b_is_kn ? 1 : 0;
  P.idesc = make_idesc(P.a_mn, P.b_mn, P.bn);
  P.p = 1;
  P.c = c;
  P.c_pitch = ldc;
  P.c_rows = m;
  P.roles = 1;
  P.status = status;
  P.timeout_ns = timeout_ns;
  CUtensorMap ta, tb;
  int rc = encode_operand(&ta, a, P.a_mn, m, k, lda, 128);
  if (rc != kSuccess) return rc;
  rc = encode_operand(&tb, b, P.b_mn, n, k, ldb, P.bn / 2);
  if (rc != kSuccess) return rc;
  if (out_f32) {
    int pairs = 0;
    rc = resident_pairs(false, 32 * kGemmWarps, &pairs);
    if (rc != kSuccess) return rc;
    P.k_splits = choose_k_splits(static_cast<long long>(P.m_tiles) * P.n_tiles, P.k_tiles, pairs);
    if (P.k_splits > 1 && !accumulate) {
      // The shares add into the output, so a plain store becomes zero fill + accumulate.
      FGA_CUDA(cudaMemset2DAsync(c, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(n) * 4,
                                 static_cast<size_t>(m), static_cast<cudaStream_t>(stream)));
      P.epi = kEpiF32Add;
    }
  }
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream));
}

// ---- MXFP8 variants: operands are E4M3 [rows_padded, kp] with E8M0 scales in the tcgen05 layout,
// exactly what fga_mx_quantize writes (rows padded to 256, kp to 128).

int fga_gemm_local_mx(const void* aq, const void* sfa, int64_t a_rows_padded, const void* bq,
                      const void* sfb, int64_t b_rows_padded, int m, int n, int kp, void* c, int64_t ldc,
                      int out_f32, int accumulate, int32_t* status, uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(aq && sfa && bq && sfb && c && status, "fga_gemm_local_mx: null argument");
  FGA_REQUIRE(m >= 1 && n >= 128 && n % 128 == 0 && kp >= 128 && kp % 128 == 0,
              "fga_gemm_local_mx: n and the padded K must be positive multiples of 128");
  FGA_REQUIRE(a_rows_padded >= m && a_rows_padded % 256 == 0 && b_rows_padded >= n && b_rows_padded % 128 == 0,
              "fga_gemm_local_mx: operand rows must be padded as the quantizer pads them");
  FGA_REQUIRE(!accumulate || out_f32, "MXFP8 gradient accumulation requires FP32 output");
  FGA_REQUIRE(ldc >= n && (ldc * (out_f32 ? 4 : 2)) % 16 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0,
              "fga_gemm_local_mx: output needs 16-byte aligned rows");
  GemmParams P{};
  P.mode = kLocal;
  P.epi = out_f32 ? (accumulate ? kEpiF32Add : kEpiF32Store) : kEpiBf16;
  P.bn = mx_tile_n(n % 256 == 0 && b_rows_padded % 256 == 0);
  P.acc_stages = P.bn == 256 ? 1 : 2;
  P.m_tiles = (m + 255) / 256;
  P.n_tiles = n / P.bn;
  P.k_tiles = kp / 128;
  P.group_m = env_int("FGA_GROUP_M_LOCAL", 8);
  P.stages = kMaxStages;
  P.idesc = make_idesc_mx(P.bn);
  P.p = 1;
  P.c = c;
  P.c_pitch = ldc;
  P.c_rows = m;
  P.roles = 1;
  P.sfa_kblocks = P.sfb_kblocks = kp / 128;
  P.status = status;
  P.timeout_ns = timeout_ns;
  CUtensorMap ta, tb, tsa, tsb;
  int rc = encode_mx_operand(&ta, &tsa, aq, sfa, a_rows_padded, kp, 128);
  if (rc != kSuccess) return rc;
  rc = encode_mx_operand(&tb, &tsb, bq, sfb, b_rows_padded, kp, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream), &tsa, &tsb);
}

int fga_gemm_push_mx(const void* aq, const void* sfa, int64_t a_rows_padded, int kp, int a_rows,
                     const void* bq, const void* sfb, int64_t b_rows_padded, const void* bias, int segments,
                     int n_segment, const int64_t* const* peer_heads, int64_t head_rows, int rank, int p,
                     int32_t* status, uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(aq && sfa && bq && sfb && peer_heads && status, "fga_gemm_push_mx: null argument");
  FGA_REQUIRE(segments == 1 || segments == 3 || segments == 4,
              "Expected one output projection or three/four QKV projections");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_push_mx: bad rank %d of %d", rank, p);
  FGA_REQUIRE(kp >= 128 && kp % 128 == 0, "fga_gemm_push_mx: padded K must be a multiple of 128");
  FGA_REQUIRE(a_rows % 256 == 0 && a_rows <= a_rows_padded && a_rows <= head_rows,
              "a_rows must be a tile multiple within the quantized rows and the head-side rank block");
  FGA_REQUIRE(n_segment > 0 && n_segment % (p * 128) == 0,
              "Push segment width must be a multiple of CP * tile N");
  const int n = segments * n_segment;
  FGA_REQUIRE(b_rows_padded >= n && b_rows_padded % 128 == 0, "fga_gemm_push_mx: weight rows must be padded");
  for (int s = 0; s < segments; ++s) FGA_REQUIRE(peer_heads[s], "fga_gemm_push_mx: null peer table %d", s);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(bias) % 16 == 0, "fga_gemm_push_mx: the bias must be 16-byte aligned");
  GemmParams P{};
  P.bn = mx_tile_n((n / 128) % 2 == 0 && b_rows_padded % 256 == 0);
  P.acc_stages = P.bn == 256 ? 1 : 2;
  P.m_tiles = a_rows / 256;
  P.k_tiles = kp / 128;
  P.idesc = make_idesc_mx(P.bn);
  fill_push(P, n, sched::uniform_layout(segments, n_segment / p / 128), peer_heads, segments, head_rows, rank, p,
            bias, status, timeout_ns);
  P.sfa_kblocks = P.sfb_kblocks = kp / 128;
  CUtensorMap ta, tb, tsa, tsb;
  int rc = encode_mx_operand(&ta, &tsa, aq, sfa, a_rows_padded, kp, 128);
  if (rc != kSuccess) return rc;
  rc = encode_mx_operand(&tb, &tsb, bq, sfb, b_rows_padded, kp, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream), &tsa, &tsb);
}

int fga_gemm_recv_mx(const void* recv, void* mx_recv, void* mx_scale, int recv_rows, int k, const void* bq,
                     const void* sfb, int64_t b_rows_padded, int b_kp, int n, void* c,
                     const int64_t* peer_recv, const int64_t* peer_counters, int32_t* counters,
                     const void* const* srcs, int num_in, int src_rows, int split, int rank, int p,
                     int roles, const int64_t* epoch, int32_t* progress, int32_t* status,
                     uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(recv && mx_recv && mx_scale && bq && sfb && c && peer_recv && peer_counters && counters && srcs &&
                  status,
              "fga_gemm_recv_mx: null argument");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_recv_mx: bad rank %d of %d", rank, p);
  FGA_REQUIRE(num_in == 1 || num_in == 3 || num_in == 4,
              "Expected one output projection or three/four QKV projections");
  FGA_REQUIRE(recv_rows >= 256 && recv_rows % 256 == 0, "fga_gemm_recv_mx: receive rows must be a multiple of 256");
  FGA_REQUIRE(src_rows >= 1 && src_rows <= recv_rows,
              "Receive source rows must be positive and fit the receive buffer");
  FGA_REQUIRE(k % (p * num_in * 128) == 0, "Receive K must split evenly over peers and input segments");
  FGA_REQUIRE(b_kp >= k && b_kp % 128 == 0, "fga_gemm_recv_mx: the weight's padded K must cover K");
  FGA_REQUIRE(n >= 128 && n % 128 == 0 && b_rows_padded >= n && b_rows_padded % 128 == 0,
              "GEMM mode must be push/recv and tile N must divide output width");
  FGA_REQUIRE(split >= 1 && 128 % split == 0, "FUSED_PUSH_SPLIT must divide 128");
  FGA_REQUIRE((roles & 3) != 0 && (roles & ~3) == 0, "fga_gemm_recv_mx: roles is a mask of 1 (GEMM) and 2 (pushers)");
  for (int t = 0; t < num_in; ++t)
    FGA_REQUIRE(srcs[t] && reinterpret_cast<uintptr_t>(srcs[t]) % 16 == 0,
                "fga_gemm_recv_mx: source %d must be a 16-byte aligned device pointer", t);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(c) % 16 == 0, "fga_gemm_recv_mx: output must be 16-byte aligned");
  GemmParams P{};
  P.bn = mx_tile_n(n % 256 == 0 && b_rows_padded % 256 == 0);
  P.acc_stages = P.bn == 256 ? 1 : 2;
  P.k_tiles = k / 128;
  P.idesc = make_idesc_mx(P.bn);
  fill_recv(P, recv_rows, k, n, c, sched::uniform_layout(num_in, k / (p * num_in * 128)), peer_recv, peer_counters,
            counters, srcs, num_in, src_rows, split, rank, p, roles, status, timeout_ns);
  P.quant_arrivals = p * num_in * split;
  P.target = P.quant_arrivals + 16;
  (void)epoch;
  int rc = pace_pushers(P, progress, static_cast<cudaStream_t>(stream));
  if (rc != kSuccess) return rc;
  P.quant_src = static_cast<const uint16_t*>(recv);
  P.quant_q = static_cast<uint8_t*>(mx_recv);
  P.quant_sf = static_cast<uint8_t*>(mx_scale);
  P.sfa_kblocks = k / 128;
  P.sfb_kblocks = b_kp / 128;
  P.status = status;
  P.timeout_ns = timeout_ns;
  CUtensorMap ta, tb, tsa, tsb;
  rc = encode_mx_operand(&ta, &tsa, mx_recv, mx_scale, recv_rows, k, 128);
  if (rc != kSuccess) return rc;
  rc = encode_mx_operand(&tb, &tsb, bq, sfb, b_rows_padded, b_kp, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream), &tsa, &tsb);
}

// ---- grouped-query attention with MXFP8 operands: the block-scaled launches above with the grouped
// column layout of fga_gemm_push_gqa / fga_gemm_recv_gqa.

int fga_gemm_push_gqa_mx(const void* aq, const void* sfa, int64_t a_rows_padded, int kp, int a_rows, const void* bq,
                         const void* sfb, int64_t b_rows_padded, const void* bias, int kv_heads, int q_per_kv,
                         int gate, const int64_t* const* peer_heads, int64_t head_rows, int rank, int p,
                         int32_t* status, uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(aq && sfa && bq && sfb && peer_heads && status, "fga_gemm_push_gqa_mx: null argument");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_push_gqa_mx: bad rank %d of %d", rank, p);
  FGA_REQUIRE(kv_heads >= 1 && kv_heads % p == 0 && q_per_kv >= 1 && q_per_kv <= 64,
              "Key/value heads must split evenly over CP ranks (kv_heads=%d, q_per_kv=%d, p=%d)", kv_heads,
              q_per_kv, p);
  FGA_REQUIRE(kp >= 128 && kp % 128 == 0, "fga_gemm_push_gqa_mx: padded K must be a multiple of 128");
  FGA_REQUIRE(a_rows >= 256 && a_rows % 256 == 0 && a_rows <= a_rows_padded && a_rows <= head_rows,
              "a_rows must be a tile multiple within the quantized rows and the head-side rank block");
  const int kinds = gate ? 4 : 3;
  for (int s = 0; s < kinds; ++s) FGA_REQUIRE(peer_heads[s], "fga_gemm_push_gqa_mx: null peer table %d", s);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(bias) % 16 == 0, "fga_gemm_push_gqa_mx: the bias must be 16-byte aligned");
  const sched::HeadLayout layout = grouped_layout(kv_heads, q_per_kv, gate, p);
  const long long units = static_cast<long long>(kv_heads) * sched::group_units(layout);
  FGA_REQUIRE(units * 128 <= 2147483647LL, "fga_gemm_push_gqa_mx: too many output columns");
  const int n = static_cast<int>(units) * 128;
  FGA_REQUIRE(b_rows_padded >= n && b_rows_padded % 128 == 0, "fga_gemm_push_gqa_mx: weight rows must be padded");
  GemmParams P{};
  P.bn = mx_tile_n(units % 2 == 0 && b_rows_padded % 256 == 0);
  P.acc_stages = P.bn == 256 ? 1 : 2;
  P.m_tiles = a_rows / 256;
  P.k_tiles = kp / 128;
  P.idesc = make_idesc_mx(P.bn);
  fill_push(P, n, layout, peer_heads, kinds, head_rows, rank, p, bias, status, timeout_ns);
  P.sfa_kblocks = P.sfb_kblocks = kp / 128;
  CUtensorMap ta, tb, tsa, tsb;
  int rc = encode_mx_operand(&ta, &tsa, aq, sfa, a_rows_padded, kp, 128);
  if (rc != kSuccess) return rc;
  rc = encode_mx_operand(&tb, &tsb, bq, sfb, b_rows_padded, kp, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream), &tsa, &tsb);
}

int fga_gemm_recv_gqa_mx(const void* recv, void* mx_recv, void* mx_scale, int recv_rows, const void* bq,
                         const void* sfb, int64_t b_rows_padded, int b_kp, int n, void* c, const int64_t* peer_recv,
                         const int64_t* peer_counters, int32_t* counters, const void* const* srcs, int kv_heads,
                         int q_per_kv, int gate, int src_rows, int split, int rank, int p, int roles,
                         int32_t* progress, int32_t* status, uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(recv && mx_recv && mx_scale && bq && sfb && c && peer_recv && peer_counters && counters && srcs &&
                  status,
              "fga_gemm_recv_gqa_mx: null argument");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p, "fga_gemm_recv_gqa_mx: bad rank %d of %d", rank, p);
  FGA_REQUIRE(kv_heads >= 1 && kv_heads % p == 0 && q_per_kv >= 1 && q_per_kv <= 64,
              "Key/value heads must split evenly over CP ranks (kv_heads=%d, q_per_kv=%d, p=%d)", kv_heads,
              q_per_kv, p);
  FGA_REQUIRE(recv_rows >= 256 && recv_rows % 256 == 0,
              "fga_gemm_recv_gqa_mx: receive rows must be a multiple of 256");
  FGA_REQUIRE(src_rows >= 1 && src_rows <= recv_rows,
              "Receive source rows must be positive and fit the receive buffer");
  FGA_REQUIRE(split >= 1 && 128 % split == 0, "FUSED_PUSH_SPLIT must divide 128");
  FGA_REQUIRE((roles & 3) != 0 && (roles & ~3) == 0,
              "fga_gemm_recv_gqa_mx: roles is a mask of 1 (GEMM) and 2 (pushers)");
  const int num_in = gate ? 4 : 3;
  for (int t = 0; t < num_in; ++t)
    FGA_REQUIRE(srcs[t] && reinterpret_cast<uintptr_t>(srcs[t]) % 16 == 0,
                "fga_gemm_recv_gqa_mx: source %d must be a 16-byte aligned device pointer", t);
  FGA_REQUIRE(reinterpret_cast<uintptr_t>(c) % 16 == 0, "fga_gemm_recv_gqa_mx: output must be 16-byte aligned");
  const sched::HeadLayout layout = grouped_layout(kv_heads, q_per_kv, gate, p);
  const long long units = static_cast<long long>(kv_heads) * sched::group_units(layout);
  FGA_REQUIRE(units * 128 <= 2147483647LL, "fga_gemm_recv_gqa_mx: receive rows too wide");
  const int k = static_cast<int>(units) * 128;
  FGA_REQUIRE(b_kp >= k && b_kp % 128 == 0, "fga_gemm_recv_gqa_mx: the weight's padded K must cover K");
  FGA_REQUIRE(n >= 128 && n % 128 == 0 && b_rows_padded >= n && b_rows_padded % 128 == 0,
              "GEMM mode must be push/recv and tile N must divide output width");
  GemmParams P{};
  P.bn = mx_tile_n(n % 256 == 0 && b_rows_padded % 256 == 0);
  P.acc_stages = P.bn == 256 ? 1 : 2;
  P.k_tiles = k / 128;
  P.idesc = make_idesc_mx(P.bn);
  fill_recv(P, recv_rows, k, n, c, layout, peer_recv, peer_counters, counters, srcs, num_in, src_rows, split, rank,
            p, roles, status, timeout_ns);
  P.quant_arrivals = p * num_in * split;
  P.target = P.quant_arrivals + 16;
  int rc = pace_pushers(P, progress, static_cast<cudaStream_t>(stream));
  if (rc != kSuccess) return rc;
  P.quant_src = static_cast<const uint16_t*>(recv);
  P.quant_q = static_cast<uint8_t*>(mx_recv);
  P.quant_sf = static_cast<uint8_t*>(mx_scale);
  P.sfa_kblocks = k / 128;
  P.sfb_kblocks = b_kp / 128;
  CUtensorMap ta, tb, tsa, tsb;
  rc = encode_mx_operand(&ta, &tsa, mx_recv, mx_scale, recv_rows, k, 128);
  if (rc != kSuccess) return rc;
  rc = encode_mx_operand(&tb, &tsb, bq, sfb, b_rows_padded, b_kp, P.bn / 2);
  if (rc != kSuccess) return rc;
  return launch(ta, tb, P, static_cast<cudaStream_t>(stream), &tsa, &tsb);
}

}  // extern "C"
