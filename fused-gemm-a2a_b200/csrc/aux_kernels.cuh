// Launchers of the auxiliary kernels (see aux_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace fga {

int launch_barrier(long long* flags, const long long* peer_flags, int rank, int p, int bump,
                   int* counters, int count, int* epoch_out, int* status,
                   unsigned long long timeout_ns, cudaStream_t stream);

int launch_copy_rank_rows(const void* const* in, void* const* out, int segments, int peers,
                          long long rows_in, long long rows_out, int width, const void* bias,
                          int head_dim, int head_off, cudaStream_t stream);

long long bias_grad_scratch_floats(long long rows, int width);
int launch_bias_grad(const void* dy, long long rows, int width, void* out, int out_is_f32,
                     int accumulate, float* scratch, cudaStream_t stream);
long long bias_grad_static_capacity_floats();
int launch_bias_grad_static(const void* dy, long long rows, int width, void* out, int out_is_f32,
                            int accumulate, cudaStream_t stream);

int launch_mx_quantize(const void* a, long long rows, int k, long long stride_row,
                       long long stride_k, void* q, void* sf, long long rp, int kp,
                       cudaStream_t stream);

}  // namespace fga
