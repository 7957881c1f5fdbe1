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
  int n = __atomic_load_n(&cached[dev], __ATOMIC_RELAXED);  // forward and autograd threads both launch
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    __atomic_store_n(&cached[dev], n, __ATOMIC_RELAXED);
  }
  return n;
}

static PFN_cuTensorMapEncodeTiled_v12000 tmap_encoder() {
  // Initialised once, thread-safely (function-local static).
  static const PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
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

// ---- virtual-memory-management allocations -----------------------------------------------------
// Driver entry points are looked up through the runtime, so the library does not link libcuda.
struct VmmApi {
  PFN_cuMemGetAllocationGranularity_v10020 granularity = nullptr;
  PFN_cuMemCreate_v10020 create = nullptr;
  PFN_cuMemRelease_v10020 release = nullptr;
  PFN_cuMemAddressReserve_v10020 reserve = nullptr;
  PFN_cuMemAddressFree_v10020 address_free = nullptr;
  PFN_cuMemMap_v10020 map = nullptr;
  PFN_cuMemUnmap_v10020 unmap = nullptr;
  PFN_cuMemSetAccess_v10020 set_access = nullptr;
  PFN_cuMemExportToShareableHandle_v10020 export_handle = nullptr;
  PFN_cuMemImportFromShareableHandle_v10020 import_handle = nullptr;
  bool complete = false;
};

template <typename Fn>
static bool driver_entry(const char* name, Fn& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return false;
  fn = reinterpret_cast<Fn>(p);
  return fn != nullptr;
}

static const VmmApi& vmm_api() {
  // Initialised once, thread-safely (function-local static); incomplete when any entry is missing.
  static const VmmApi api = [] {
    VmmApi a;
    a.complete = driver_entry("cuMemGetAllocationGranularity", a.granularity) &&
                 driver_entry("cuMemCreate", a.create) && driver_entry("cuMemRelease", a.release) &&
                 driver_entry("cuMemAddressReserve", a.reserve) &&
                 driver_entry("cuMemAddressFree", a.address_free) && driver_entry("cuMemMap", a.map) &&
                 driver_entry("cuMemUnmap", a.unmap) && driver_entry("cuMemSetAccess", a.set_access) &&
                 driver_entry("cuMemExportToShareableHandle", a.export_handle) &&
                 driver_entry("cuMemImportFromShareableHandle", a.import_handle);
    return a;
  }();
  return api;
}

static int vmm_fail(CUresult r, const char* what) {
  return set_error(kCudaError, "%s failed with CUresult %d", what, static_cast<int>(r));
}

static CUmemAllocationProp vmm_properties(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

// Reserve an address range for `handle`, map it and give the current device read/write access.
// On failure nothing stays reserved or mapped.
static int vmm_map(const VmmApi& api, CUmemGenericAllocationHandle handle, size_t size, size_t granularity,
                   int device, void** out) {
  CUdeviceptr va = 0;
  CUresult r = api.reserve(&va, size, granularity, 0, 0);
  if (r != CUDA_SUCCESS) return vmm_fail(r, "cuMemAddressReserve");
  r = api.map(va, size, 0, handle, 0);
  if (r != CUDA_SUCCESS) {
    api.address_free(va, size);
    return vmm_fail(r, "cuMemMap");
  }
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = api.set_access(va, size, &access, 1);
  if (r != CUDA_SUCCESS) {
    api.unmap(va, size);
    api.address_free(va, size);
    return vmm_fail(r, "cuMemSetAccess");
  }
  *out = reinterpret_cast<void*>(va);
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

int64_t fga_symm_vmm_size(size_t bytes) {
  const VmmApi& api = vmm_api();
  int device = 0;
  if (bytes == 0 || !api.complete || cudaGetDevice(&device) != cudaSuccess) {
    set_error(kUnsupported, "fga_symm_vmm_size: no size, or the driver's virtual memory management API is not available");
    return -1;
  }
  const CUmemAllocationProp prop = vmm_properties(device);
  size_t granularity = 0;
  if (api.granularity(&granularity, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || granularity == 0) {
    set_error(kCudaError, "cuMemGetAllocationGranularity failed");
    return -1;
  }
  return static_cast<int64_t>((bytes + granularity - 1) / granularity * granularity);
}

int fga_symm_alloc_vmm(size_t bytes, void** ptr, int* fd) {
  FGA_REQUIRE(ptr != nullptr && fd != nullptr && bytes > 0, "fga_symm_alloc_vmm: need a size and two output pointers");
  const VmmApi& api = vmm_api();
  if (!api.complete) return set_error(kUnsupported, "the driver's virtual memory management API is not available");
  int device = 0;
  FGA_CUDA(cudaFree(nullptr));  // make sure the runtime has a context on the current device
  FGA_CUDA(cudaGetDevice(&device));
  const CUmemAllocationProp prop = vmm_properties(device);
  size_t granularity = 0;
  CUresult r = api.granularity(&granularity, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || granularity == 0) return vmm_fail(r, "cuMemGetAllocationGranularity");
  const size_t size = (bytes + granularity - 1) / granularity * granularity;
  CUmemGenericAllocationHandle handle = 0;
  r = api.create(&handle, size, &prop, 0);
  if (r != CUDA_SUCCESS) return vmm_fail(r, "cuMemCreate");
  void* mapped = nullptr;
  int rc = vmm_map(api, handle, size, granularity, device, &mapped);
  int exported = -1;
  if (rc == kSuccess) {
    r = api.export_handle(&exported, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) rc = vmm_fail(r, "cuMemExportToShareableHandle");
  }
  // The mapping (and every importer's) keeps the physical memory alive; the creation handle is not
  // needed any longer.
  api.release(handle);
  if (rc == kSuccess) {
    cudaError_t e = cudaMemset(mapped, 0, size);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) rc = cuda_fail(e, "cudaMemset");
  }
  if (rc != kSuccess) {
    if (mapped != nullptr) {
      api.unmap(reinterpret_cast<CUdeviceptr>(mapped), size);
      api.address_free(reinterpret_cast<CUdeviceptr>(mapped), size);
    }
    return rc;
  }
  *ptr = mapped;
  *fd = exported;
  return kSuccess;
}

int fga_symm_open_vmm(int fd, size_t bytes, void** peer_ptr) {
  FGA_REQUIRE(fd >= 0 && bytes > 0 && peer_ptr != nullptr, "fga_symm_open_vmm: need a descriptor, a size and an output pointer");
  const VmmApi& api = vmm_api();
  if (!api.complete) return set_error(kUnsupported, "the driver's virtual memory management API is not available");
  int device = 0;
  FGA_CUDA(cudaGetDevice(&device));
  const CUmemAllocationProp prop = vmm_properties(device);
  size_t granularity = 0;
  CUresult r = api.granularity(&granularity, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || granularity == 0) return vmm_fail(r, "cuMemGetAllocationGranularity");
  FGA_REQUIRE(bytes % granularity == 0, "fga_symm_open_vmm: the size must be the owner's fga_symm_vmm_size()");
  CUmemGenericAllocationHandle handle = 0;
  r = api.import_handle(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return vmm_fail(r, "cuMemImportFromShareableHandle");
  const int rc = vmm_map(api, handle, bytes, granularity, device, peer_ptr);
  api.release(handle);  // the mapping holds its own reference
  return rc;
}

int fga_symm_release_vmm(void* ptr, size_t bytes) {
  FGA_REQUIRE(ptr != nullptr && bytes > 0, "fga_symm_release_vmm: null pointer or no size");
  const VmmApi& api = vmm_api();
  if (!api.complete) return set_error(kUnsupported, "the driver's virtual memory management API is not available");
  CUresult r = api.unmap(reinterpret_cast<CUdeviceptr>(ptr), bytes);
  if (r != CUDA_SUCCESS) return vmm_fail(r, "cuMemUnmap");
  r = api.address_free(reinterpret_cast<CUdeviceptr>(ptr), bytes);
  if (r != CUDA_SUCCESS) return vmm_fail(r, "cuMemAddressFree");
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
  FGA_REQUIRE((rows + 255) / 256 <= 65535, "fga_bias_grad_static: too many rows (%lld)",
              static_cast<long long>(rows));
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
