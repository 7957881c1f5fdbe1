// Host runtime of libfga: error reporting, TMA descriptor encoding, symmetric (peer-mapped)
// memory, and the extern "C" entry points that are not GEMM launches.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cudaTypedefs.h>
#include "../../include/fga.h"
#include "aux_kernels.cuh"
#include "common.cuh"

namespace fga {

static thread_local char g_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return set_error(kCudaError, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

static unsigned long long g_launches = 0;
void count_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices];  // 0 = not queried yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 tmap_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

int encode_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                   uint64_t rows, uint64_t cols, uint64_t row_pitch_elems, uint32_t box_rows,
                   uint32_t box_cols, bool swizzle128) {
  auto enc = tmap_encoder();
  if (enc == nullptr) return set_error(kCudaError, "cuTensorMapEncodeTiled is not available");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (row_pitch_elems * elem_bytes) % 16 != 0)
    return set_error(kInvalidArgument, "TMA operands need 16-byte aligned bases and row pitches");
  if (swizzle128 && box_cols * elem_bytes != 128)
    return set_error(kInvalidArgument, "128-byte swizzle needs a 128-byte box row");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_pitch_elems * elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(kCudaError, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu)",
                     static_cast<int>(r), static_cast<unsigned long long>(rows),
                     static_cast<unsigned long long>(cols));
  return kSuccess;
}

}  // namespace fga

using namespace fga;

extern "C" {

int fga_version(void) { return 1; }
const char* fga_last_error(void) { return g_error; }
int fga_sm_count(void) { return sm_count(); }
uint64_t fga_launch_count(void) { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

int fga_symm_alloc(size_t bytes, void** ptr) {
  FGA_REQUIRE(ptr != nullptr && bytes > 0, "fga_symm_alloc: need a size and an output pointer");
  FGA_CUDA(cudaMalloc(ptr, bytes));
  cudaError_t e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(*ptr);
    *ptr = nullptr;
    return cuda_fail(e, "cudaMemset");
  }
  FGA_CUDA(cudaDeviceSynchronize());
  return kSuccess;
}

int fga_symm_export(void* ptr, unsigned char handle[FGA_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == FGA_IPC_HANDLE_BYTES, "IPC handle size");
  FGA_REQUIRE(ptr != nullptr && handle != nullptr, "fga_symm_export: null argument");
  cudaIpcMemHandle_t h;
  FGA_CUDA(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle, &h, sizeof(h));
  return kSuccess;
}

int fga_symm_open(const unsigned char handle[FGA_IPC_HANDLE_BYTES], void** peer_ptr) {
  FGA_REQUIRE(handle != nullptr && peer_ptr != nullptr, "fga_symm_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  FGA_CUDA(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return kSuccess;
}

int fga_symm_close(void* peer_ptr) {
  FGA_REQUIRE(peer_ptr != nullptr, "fga_symm_close: null pointer");
  FGA_CUDA(cudaIpcCloseMemHandle(peer_ptr));
  return kSuccess;
}

int fga_symm_free(void* ptr) {
  FGA_REQUIRE(ptr != nullptr, "fga_symm_free: null pointer");
  FGA_CUDA(cudaFree(ptr));
  return kSuccess;
}

int fga_barrier(int64_t* flags, const int64_t* peer_flags, int rank, int p, int bump,
                int32_t* counters, int count, int32_t* epoch_out, int32_t* status,
                uint64_t timeout_ns, void* stream) {
  FGA_REQUIRE(flags && peer_flags && status, "fga_barrier: null flags, peer table or status");
  FGA_REQUIRE(p >= 1 && p <= 32 && rank >= 0 && rank < p,
              "The single-warp device barrier supports CP sizes from 1 to 32 (p=%d rank=%d)", p, rank);
  FGA_REQUIRE(!bump || count == 0 || counters != nullptr, "fga_barrier: bump needs counters");
  return launch_barrier(reinterpret_cast<long long*>(flags),
                        reinterpret_cast<const long long*>(peer_flags), rank, p, bump, counters,
                        bump ? count : 0, epoch_out, status, timeout_ns,
                        static_cast<cudaStream_t>(stream));
}

int fga_copy_rank_rows(const void* const* in, void* const* out, int segments, int peers,
                       int64_t rows_in, int64_t rows_out, int width, const void* bias,
                       int head_dim, int head_offset, void* stream) {
  FGA_REQUIRE(in && out && segments >= 1 && segments <= 4, "fga_copy_rank_rows: 1..4 segments");
  FGA_REQUIRE(peers >= 1 && peers <= 65535 && rows_in >= 1 && rows_out >= 1 && width >= 1,
              "fga_copy_rank_rows: positive row counts, width and peer count");
  for (int i = 0; i < segments; ++i)
    FGA_REQUIRE(in[i] && out[i], "fga_copy_rank_rows: null matrix %d", i);
  FGA_REQUIRE(bias == nullptr || (head_dim >= 1 && width % head_dim == 0 && head_offset >= 0),
              "Bias must cover the interleaved heads being copied");
  return launch_copy_rank_rows(in, out, segments, peers, rows_in, rows_out, width, bias, head_dim,
                               head_offset, static_cast<cudaStream_t>(stream));
}

int64_t fga_bias_grad_scratch_floats(int64_t rows, int width) {
  return bias_grad_scratch_floats(rows, width);
}

int fga_bias_grad(const void* dy, int64_t rows, int width, void* out, int out_is_f32,
                  int accumulate, float* scratch, void* stream) {
  FGA_REQUIRE(dy && out && scratch && rows >= 1 && width >= 1,
              "Bias reduction requires contiguous BF16 rows and a BF16/FP32 output vector");
  FGA_REQUIRE((rows + 255) / 256 <= 65535, "fga_bias_grad: too many rows (%lld)",
              static_cast<long long>(rows));
  return launch_bias_grad(dy, rows, width, out, out_is_f32, accumulate, scratch,
                          static_cast<cudaStream_t>(stream));
}

int64_t fga_bias_grad_static_capacity_floats(void) { return bias_grad_static_capacity_floats(); }

int fga_bias_grad_static(const void* dy, int64_t rows, int width, void* out, int out_is_f32,
                         int accumulate, void* stream) {
  FGA_REQUIRE(dy && out && rows >= 1 && width >= 1,
              "Bias reduction requires contiguous BF16 rows and a BF16/FP32 output vector");
  return launch_bias_grad_static(dy, rows, width, out, out_is_f32, accumulate,
                                 static_cast<cudaStream_t>(stream));
}

int fga_mx_quantize(const void* a, int64_t rows, int k, int64_t stride_row, int64_t stride_k,
                    void* q, void* sf, int64_t rows_padded, int k_padded, void* stream) {
  FGA_REQUIRE(a && q && sf && rows >= 1 && k >= 1, "MXFP8 quantization requires a BF16 matrix");
  FGA_REQUIRE(stride_row == 1 || stride_k == 1,
              "MXFP8 quantization requires 16-byte aligned rows or columns");
  FGA_REQUIRE(rows_padded >= rows && rows_padded % 128 == 0 && k_padded >= k && k_padded % 128 == 0,
              "fga_mx_quantize: padded extents must cover the matrix in multiples of 128");
  FGA_REQUIRE(rows_padded / 64 <= 2147483647LL && k_padded / 128 <= 65535,
              "fga_mx_quantize: matrix too large");
  return launch_mx_quantize(a, rows, k, stride_row, stride_k, q, sf, rows_padded, k_padded,
                            static_cast<cudaStream_t>(stream));
}

}  // extern "C"
