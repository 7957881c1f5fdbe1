// Shared host/device definitions of libfga: status codes, error reporting, launch parameters.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace fga {

// Device status word (int[4] in global memory, owned by the caller):
//   [0] error code (0 = ok), [1] where (role / wait id), [2] detail (tile, counter value ...),
//   [3] reserved. Written once by the first failing wait (atomicCAS on [0]); never cleared by a
//   kernel. Every other bounded wait polls [0] on its slow path and gives up when it is set.
enum DeviceError : int {
  kOk = 0,
  kErrBarrierTimeout = 1,   // group barrier: a peer never published its epoch
  kErrCounterTimeout = 2,   // recv GEMM: a row block never collected all arrivals
  kErrPipelineTimeout = 3,  // an mbarrier of the TMA/MMA/epilogue pipeline never flipped
  kErrQuantTimeout = 4,     // receive-side quantizer: a row block never arrived
};

// Host return codes of every extern "C" entry point.
enum HostError : int {
  kSuccess = 0,
  kInvalidArgument = -1,
  kCudaError = -2,
  kUnsupported = -3,
};

int set_error(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define FGA_CUDA(expr)                                        \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::fga::cuda_fail(_e, #expr); \
  } while (0)

// After every kernel launch: surface launch errors and count the launch (fga_launch_count).
void count_launch();
#define FGA_LAUNCHED()                   \
  do {                                   \
    FGA_CUDA(cudaGetLastError());        \
    ::fga::count_launch();               \
  } while (0)

#define FGA_REQUIRE(cond, ...)                                                \
  do {                                                                        \
    if (!(cond)) return ::fga::set_error(::fga::kInvalidArgument, __VA_ARGS__); \
  } while (0)

// Encode a 2-D row-major tensor map [rows, cols] of `elem_bytes` elements with a
// [box_rows, box_cols] box and 128-byte swizzle (box_cols * elem_bytes must be 128).
int encode_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                   uint64_t rows, uint64_t cols, uint64_t row_pitch_elems, uint32_t box_rows,
                   uint32_t box_cols, bool swizzle128 = true);

int sm_count();

}  // namespace fga
