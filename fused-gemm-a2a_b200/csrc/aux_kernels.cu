// Auxiliary sm_100a kernels of the fused projection path: the group barrier, the per-rank row
// copy (ownership copy / pad strip / interleaved bias), the bias-gradient reduction and the
// standalone MXFP8 quantizer. All are HBM-bound byte movers: 16-byte accesses, grids sized from
// the SM count.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "common.cuh"
#include "ptx.cuh"
#include "aux_kernels.cuh"
#include "mx_quant.cuh"

namespace fga {

// ---------------------------------------------------------------------------------------------
// Group barrier: one warp, lane t talks to peer t. Monotone epochs read from device memory keep
// CUDA-graph replays consistent. With `bump`, this rank's arrival counters are zeroed before its
// entry is published, so no peer can increment them before the reset.
// Follows fused_gemm_a2a_kernels.py:204-228 (_barrier_kernel); the spin is bounded here.
// ---------------------------------------------------------------------------------------------
__global__ void barrier_kernel(long long* flags, const long long* peer_flags, int rank, int p,
                               int bump, int* counters, int count, int* epoch_out, int* status,
                               unsigned long long timeout_ns) {
  const int lane = threadIdx.x;
  // A recorded device error is sticky: a peer that never answered may be gone together with its
  // memory, so nothing is written to any peer until the host has cleared the status word.
  if (ld_relaxed_sys_s32(status) != 0) return;
  if (bump) {
    for (int i = lane; i < count; i += 32) counters[i] = 0;
    __syncwarp();
  }
  const long long epoch = ld_acquire_sys_s64(flags + rank) + 1;
  if (lane < p) {
    long long* slot = reinterpret_cast<long long*>(peer_flags[lane]) + rank;
    st_release_sys_s64(slot, epoch);
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (ld_acquire_sys_s64(flags + lane) < epoch) {
      nanosleep(256);
      if ((++it & 0xff) == 0) {
        if (ld_relaxed_sys_s32(status) != 0) break;
        if (globaltimer_ns() - t0 > timeout_ns) {
          if (atomicCAS(status, 0, kErrBarrierTimeout) == 0) {
            status[1] = lane;
            status[2] = static_cast<int>(epoch);
          }
          break;
        }
      }
    }
  }
  __syncwarp();
  if (bump && lane == 0 && epoch_out != nullptr) epoch_out[0] = epoch_out[0] + 1;
}

int launch_barrier(long long* flags, const long long* peer_flags, int rank, int p, int bump,
                   int* counters, int count, int* epoch_out, int* status,
                   unsigned long long timeout_ns, cudaStream_t stream) {
  barrier_kernel<<<1, 32, 0, stream>>>(flags, peer_flags, rank, p, bump, counters, count,
                                       epoch_out, status, timeout_ns);
  FGA_LAUNCHED();
  return kSuccess;
}

// ---------------------------------------------------------------------------------------------
// Per-rank row copy. out[s][r*rows_out + i, :] = in[s][r*rows_in + i, :] for i < min(rows_in,
// rows_out), zero otherwise; optional interleaved bias bias[((head_off + c/D)*S + s)*D + c%D]
// added in FP32 and rounded to BF16 once (GEMM -> BF16 -> +bias -> BF16), never on added rows.
// Follows fused_gemm_a2a_kernels.py:1106-1142 and 1424-1475.
// ---------------------------------------------------------------------------------------------
struct CopyRowsArgs {
  const uint16_t* in[4];
  uint16_t* out[4];
};

template <bool kVec>
__global__ void copy_rank_rows_kernel(const __grid_constant__ CopyRowsArgs a, long long rows_in, long long rows_out,
                                      int width, const uint16_t* bias, int head_dim, int head_off,
                                      int segments) {
  const int r = blockIdx.y, s = blockIdx.z;
  const uint16_t* in = a.in[s] + static_cast<long long>(r) * rows_in * width;
  uint16_t* out = a.out[s] + static_cast<long long>(r) * rows_out * width;
  constexpr int kE = kVec ? 8 : 1;
  const long long n_out = rows_out * width / kE, n_in = rows_in * width / kE;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < n_out;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    if constexpr (kVec) {
      uint4 val = make_uint4(0, 0, 0, 0);
      if (v < n_in) {
        val = ld_cs_v4(in + v * 8);
        if (bias != nullptr) {
          const int col = static_cast<int>((v * 8) % width);
          const int idx = ((head_off + col / head_dim) * segments + s) * head_dim + col % head_dim;
          const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias + idx));
          uint32_t x[4] = {val.x, val.y, val.z, val.w};
          const uint32_t y[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float lo = __uint_as_float(x[e] << 16) + __uint_as_float(y[e] << 16);
            const float hi = __uint_as_float(x[e] & 0xffff0000u) + __uint_as_float(y[e] & 0xffff0000u);
            uint32_t packed;
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
            x[e] = packed;
          }
          val = make_uint4(x[0], x[1], x[2], x[3]);
        }
      }
      *reinterpret_cast<uint4*>(out + v * 8) = val;
    } else {
      uint16_t val = 0;
      if (v < n_in) {
        val = in[v];
        if (bias != nullptr) {
          const int col = static_cast<int>(v % width);
          const int idx = ((head_off + col / head_dim) * segments + s) * head_dim + col % head_dim;
          const float f = __uint_as_float(static_cast<uint32_t>(val) << 16) +
                          __uint_as_float(static_cast<uint32_t>(bias[idx]) << 16);
          val = __bfloat16_as_ushort(__float2bfloat16_rn(f));
        }
      }
      out[v] = val;
    }
  }
}

int launch_copy_rank_rows(const void* const* in, void* const* out, int segments, int peers,
                          long long rows_in, long long rows_out, int width, const void* bias,
                          int head_dim, int head_off, cudaStream_t stream) {
  CopyRowsArgs a{};
  for (int i = 0; i < segments; ++i) {
    a.in[i] = static_cast<const uint16_t*>(in[i]);
    a.out[i] = static_cast<uint16_t*>(out[i]);
  }
  bool vec = width % 8 == 0 && (bias == nullptr || (head_dim % 8 == 0 &&
                                                    reinterpret_cast<uintptr_t>(bias) % 16 == 0));
  for (int i = 0; i < segments && vec; ++i)
    vec = reinterpret_cast<uintptr_t>(in[i]) % 16 == 0 && reinterpret_cast<uintptr_t>(out[i]) % 16 == 0;
  const long long n = rows_out * width / (vec ? 8 : 1);
  const int threads = 256;
  long long blocks = (n + threads * 4 - 1) / (threads * 4);  // ~4 vectors per thread
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  dim3 grid(static_cast<unsigned>(blocks), peers, segments);
  if (vec)
    copy_rank_rows_kernel<true><<<grid, threads, 0, stream>>>(
        a, rows_in, rows_out, width, static_cast<const uint16_t*>(bias), head_dim, head_off, segments);
  else
    copy_rank_rows_kernel<false><<<grid, threads, 0, stream>>>(
        a, rows_in, rows_out, width, static_cast<const uint16_t*>(bias), head_dim, head_off, segments);
  FGA_LAUNCHED();
  return kSuccess;
}

// ---------------------------------------------------------------------------------------------
// Bias gradient: FP32 column sums of BF16 rows. Pass 1 sums 256-row parts into partial[part][col]
// (a caller-provided FP32 scratch of parts*width floats); pass 2 sums the parts in order, adds the
// previous value when accumulating, and writes FP32 or rounds once to BF16. Deterministic.
// Follows fused_gemm_a2a_kernels.py:1053-1103 and 1489-1523. Row offsets are 64-bit.
// ---------------------------------------------------------------------------------------------
constexpr int kBiasPartRows = 256;

__global__ void bias_grad_partial_kernel(const uint16_t* dy, float* partial, long long rows,
                                         int width, bool vec) {
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (col >= width) return;
  const long long r0 = static_cast<long long>(blockIdx.y) * kBiasPartRows;
  const long long r1 = min(rows, r0 + kBiasPartRows);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (vec) {  // host-checked: width % 8 == 0 and a 16-byte aligned base, so every row piece is aligned
    const uint16_t* p = dy + r0 * width + col;
#pragma unroll 4
    for (long long r = r0; r < r1; ++r, p += width) {
      const uint4 v = ld_cs_v4(p);
      const uint32_t x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += __uint_as_float(x[e] << 16);
        acc[2 * e + 1] += __uint_as_float(x[e] & 0xffff0000u);
      }
    }
  } else {
    for (long long r = r0; r < r1; ++r)
      for (int e = 0; e < 8 && col + e < width; ++e)
        acc[e] += __uint_as_float(static_cast<uint32_t>(dy[r * width + col + e]) << 16);
  }
  float* out = partial + static_cast<long long>(blockIdx.y) * width + col;
  for (int e = 0; e < 8 && col + e < width; ++e) out[e] = acc[e];
}

template <typename OutT>
__global__ void bias_grad_finish_kernel(const float* partial, OutT* out, int parts, int width,
                                        int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= width) return;
  float total = 0.f;
  for (int i = 0; i < parts; ++i) total += partial[static_cast<long long>(i) * width + col];
  if constexpr (sizeof(OutT) == 4) {
    if (accumulate) total += out[col];
    out[col] = total;
  } else {
    if (accumulate) total += __uint_as_float(static_cast<uint32_t>(out[col]) << 16);
    out[col] = __bfloat16_as_ushort(__float2bfloat16_rn(total));
  }
}

long long bias_grad_scratch_floats(long long rows, int width) {
  const long long parts = (rows + kBiasPartRows - 1) / kBiasPartRows;
  return parts * width;
}

int launch_bias_grad(const void* dy, long long rows, int width, void* out, int out_is_f32,
                     int accumulate, float* scratch, cudaStream_t stream) {
  const int parts = static_cast<int>((rows + kBiasPartRows - 1) / kBiasPartRows);
  const int threads = 128;
  dim3 grid1((width + threads * 8 - 1) / (threads * 8), parts);
  const bool vec = width % 8 == 0 && reinterpret_cast<uintptr_t>(dy) % 16 == 0;
  bias_grad_partial_kernel<<<grid1, threads, 0, stream>>>(static_cast<const uint16_t*>(dy), scratch,
                                                          rows, width, vec);
  FGA_LAUNCHED();
  dim3 grid2((width + threads - 1) / threads);
  if (out_is_f32)
    bias_grad_finish_kernel<float><<<grid2, threads, 0, stream>>>(scratch, static_cast<float*>(out),
                                                                  parts, width, accumulate);
  else
    bias_grad_finish_kernel<uint16_t><<<grid2, threads, 0, stream>>>(
        scratch, static_cast<uint16_t*>(out), parts, width, accumulate);
  FGA_LAUNCHED();
  return kSuccess;
}

// ---------------------------------------------------------------------------------------------
// Bias gradient without any allocation, for callers that must not (or cannot) allocate device
// memory when they call: code running under a memory budget that is already fully planned, an
// allocator-free plugin host, or a call site where a cudaMalloc would serialize the device. The
// FP32 partial sums live in a fixed array that is part of this library's device image; every GPU
// that loads the library holds these 4 MiB until the process exits.
//
// The array is shared by every call on a device and keeps whatever the previous call left in it.
// Nothing has to be cleared: pass 1 writes every partial sum that pass 2 reads. Two calls that
// overlap on the GPU (different streams, or graphs replayed concurrently) race on the array.
// ---------------------------------------------------------------------------------------------
constexpr long long kStaticScratchFloats = 1ll << 20;  // 256-row parts x width <= 1 Mi floats (4 MiB)
static __device__ __align__(256) float g_bias_scratch[kStaticScratchFloats];

long long bias_grad_static_capacity_floats() { return kStaticScratchFloats; }

// Device address of the array for the current device. In host code the symbol is only a stand-in,
// never a device pointer, so the address is looked up once per device with that device current.
// The cache is read and written with atomics: two host threads may make a device's first call at
// the same time, and both then store the same address. (It does not survive cudaDeviceReset; a
// process that resets a device must not call this entry point on it afterwards.)
static int static_scratch_address(float** out) {
  constexpr int kMaxDevices = 64;
  static float* cached[kMaxDevices];  // null = not looked up yet on that device
  int dev = 0;
  FGA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return set_error(kUnsupported, "device index %d out of range", dev);
  float* address = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
  if (address == nullptr) {
    FGA_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_bias_scratch));
    if (address == nullptr) return set_error(kCudaError, "the static scratch array has no device address");
    __atomic_store_n(&cached[dev], address, __ATOMIC_RELEASE);
  }
  *out = address;
  return kSuccess;
}

int launch_bias_grad_static(const void* dy, long long rows, int width, void* out, int out_is_f32,
                            int accumulate, cudaStream_t stream) {
  const long long needed = bias_grad_scratch_floats(rows, width);
  if (needed > kStaticScratchFloats)
    return set_error(kInvalidArgument,
                     "fga_bias_grad_static: %lld rows x %d columns need %lld scratch floats, the built-in "
                     "array holds %lld; use fga_bias_grad with caller-provided scratch",
                     rows, width, needed, kStaticScratchFloats);
  float* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != kSuccess) return rc;
  return launch_bias_grad(dy, rows, width, out, out_is_f32, accumulate, scratch, stream);
}

// ---------------------------------------------------------------------------------------------
// MXFP8 quantizer: E4M3 payload + one E8M0 scale per 32 elements along K.
// Scale policy (fused_gemm_a2a_kernels.py:1200-1219): e = ceil(log2(amax / 448)) from the FP32
// exponent/mantissa of amax (448 = 1.75 * 2^8), clamped to [-126, 127]; zero group -> e = 0;
// group with +-Inf -> scale byte 255 (E8M0 NaN) and multiplier 0, so Inf becomes a NaN payload and
// finite values 0. NaN elements do not raise amax (max.f32 drops NaN) and stay NaN.
// Scale bytes are stored in the tcgen05 128-row x 4-group swizzled layout
// (fused_gemm_a2a_kernels.py:1195-1197). Padding rows/columns are written (payload 0, scale 127).
// ---------------------------------------------------------------------------------------------
// Row-major source: one warp per (row, 256-column chunk); 4 lanes share a 32-group.
__global__ void mx_quant_rows_kernel(const uint16_t* a, uint8_t* q, uint8_t* sf, long long rows,
                                     int k, long long rp, int kp, long long stride_row) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = (kp + 255) / 256;
  const bool vec_ok = (stride_row % 8 == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0);
  for (long long u = warp; u < rp * chunks; u += warps) {
    const long long row = u / chunks;
    const int col = static_cast<int>(u % chunks) * 256 + lane * 8;
    const bool active = col < kp;  // shuffles below stay warp-wide; only the stores are masked
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (active && row < rows) {
      if (vec_ok && col + 8 <= k) {
        const uint4 x = *reinterpret_cast<const uint4*>(a + row * stride_row + col);
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[2 * e] = __uint_as_float(w[e] << 16);
          v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
      } else {
        for (int j = 0; j < 8; ++j)
          if (col + j < k) v[j] = __uint_as_float(static_cast<uint32_t>(a[row * stride_row + col + j]) << 16);
      }
    }
    float peak = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) peak = fmaxf(peak, fabsf(v[j]));
    peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 1));
    peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 2));
    int e;
    float inv;
    mx_scale(peak, e, inv);
    uint2 out;
    out.x = to_e4m3x2(v[0] * inv, v[1] * inv) | (static_cast<uint32_t>(to_e4m3x2(v[2] * inv, v[3] * inv)) << 16);
    out.y = to_e4m3x2(v[4] * inv, v[5] * inv) | (static_cast<uint32_t>(to_e4m3x2(v[6] * inv, v[7] * inv)) << 16);
    if (!active) continue;
    *reinterpret_cast<uint2*>(q + row * kp + col) = out;
    if ((lane & 3) == 0) sf[mx_scale_offset(row, col / 32, kp / 32)] = static_cast<uint8_t>(e + 127);
  }
}

// Transposed source (element (row, c) at a[row + c * stride_k]): quantize along the strided axis.
// A block transposes a 64-row x 128-column tile through shared memory (FP32, odd pitch).
__global__ void mx_quant_cols_kernel(const uint16_t* a, uint8_t* q, uint8_t* sf, long long rows,
                                     int k, long long rp, int kp, long long stride_k) {
  __shared__ float tile[128][65];
  const long long row0 = static_cast<long long>(blockIdx.x) * 64;
  const int col0 = blockIdx.y * 128;
  const int tid = threadIdx.x;  // 256 threads
  // Load: memory rows are columns c of the logical matrix; 64 consecutive logical rows are
  // contiguous (128 bytes), 8 lanes x 16 bytes each.
  const bool vec_ok = (stride_k % 8 == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0);
  for (int i = 0; i < 4; ++i) {
    const int c = (tid >> 3) + 32 * i;
    const int r8 = (tid & 7) * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (col0 + c < k) {
      const uint16_t* p = a + (col0 + c) * stride_k + row0 + r8;
      if (vec_ok && row0 + r8 + 8 <= rows) {
        const uint4 x = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[2 * e] = __uint_as_float(w[e] << 16);
          v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
      } else {
        for (int j = 0; j < 8; ++j)
          if (row0 + r8 + j < rows) v[j] = __uint_as_float(static_cast<uint32_t>(p[j]) << 16);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[c][r8 + j] = v[j];
  }
  __syncthreads();
  const int r = tid & 63, g = tid >> 6;  // one (row, 32-group) per thread
  const long long row = row0 + r;
  if (row >= rp || col0 + g * 32 >= kp) return;
  float v[32];
  float peak = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    v[j] = tile[g * 32 + j][r];
    peak = fmaxf(peak, fabsf(v[j]));
  }
  int e;
  float inv;
  mx_scale(peak, e, inv);
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j)
    w[j] = to_e4m3x2(v[4 * j] * inv, v[4 * j + 1] * inv) |
           (static_cast<uint32_t>(to_e4m3x2(v[4 * j + 2] * inv, v[4 * j + 3] * inv)) << 16);
  uint4* dst = reinterpret_cast<uint4*>(q + row * kp + col0 + g * 32);
  dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  sf[mx_scale_offset(row, (col0 >> 5) + g, kp / 32)] = static_cast<uint8_t>(e + 127);
}

int launch_mx_quantize(const void* a, long long rows, int k, long long stride_row,
                       long long stride_k, void* q, void* sf, long long rp, int kp,
                       cudaStream_t stream) {
  if (stride_k == 1) {
    const long long units = rp * ((kp + 255) / 256);
    long long blocks = (units + 7) / 8;  // 8 warps per block
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    mx_quant_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint16_t*>(a), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), rows,
        k, rp, kp, stride_row);
  } else {
    dim3 grid(static_cast<unsigned>(rp / 64), kp / 128);
    mx_quant_cols_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(a),
                                                   static_cast<uint8_t*>(q),
                                                   static_cast<uint8_t*>(sf), rows, k, rp, kp,
                                                   stride_k);
  }
  FGA_LAUNCHED();
  return kSuccess;
}

}  // namespace fga
