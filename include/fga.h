/* libfga - C ABI of the B200 (sm_100a) fused projection-GEMM + Ulysses all-to-all path.
 *
 * The reference project (niyunsheng/fused-gemm-a2a) has no FFI: its boundary is the Python module
 * surface of fused_gemm_a2a.py / fused_gemm_a2a_kernels.py, which JIT-compiles CuTe-DSL and Triton
 * kernels. This header is the boundary a binding of that surface calls instead. Each entry point
 * names the reference interface it replaces (file:line in the reference tree).
 *
 * Conventions
 *   - plain C: raw device pointers, sizes, a cudaStream_t passed as void*; no torch types.
 *   - every function returns 0 on success, a negative FgaResult otherwise; fga_last_error()
 *     returns the message of the calling thread's last failure. Nothing throws.
 *   - launch functions enqueue on `stream`, never synchronize, never allocate, and are legal
 *     under CUDA stream capture (except where noted). The current device must be the one the
 *     pointers live on.
 *   - `status` is a caller-owned int[4] in device memory, zeroed once by the caller. A kernel
 *     whose bounded wait expires writes {code, where, detail, 0} (FgaDeviceError) and returns;
 *     the context stays usable. Kernels never clear it, and the error is sticky: while status[0]
 *     is non-zero, fga_barrier and the fused GEMMs return at once without touching any peer's
 *     memory (the peer that did not answer may have exited and unmapped it). The host reads the
 *     word, tears the group down or repairs it, and zeroes the word before it launches again.
 *   - all matrices are row-major; BF16 is passed as 16-bit words.
 *   - pointer alignment: matrix operands, outputs, biases and pusher sources must be 16-byte aligned
 *     (TMA and 16-byte vector accesses); a launcher that would need an aligned pointer and does not
 *     get one returns FGA_INVALID_ARGUMENT, or takes a scalar path where one exists
 *     (fga_copy_rank_rows, fga_bias_grad). No kernel is ever launched on a misaligned operand.
 *   - tuning variables are read from the environment by the launcher, on the host, at every call:
 *     FGA_STAGES, FGA_GROUP_M_PUSH, FGA_GROUP_M_RECV, FGA_GROUP_M_LOCAL (raster group sizes),
 *     FGA_PUSHER_WARPS, FGA_PUSH_LEAD, FGA_WGRAD_SPLITS (fga_gemm_local with FP32 output: shares of the
 *     reduction axis per tile, a number or "auto"), FGA_MX_TILE_N (128: block-scaled GEMMs use 128-column
 *     tiles with two accumulator stages everywhere instead of 256-column tiles with one). Unset means the defaults that were measured; none
 *     of them changes results beyond FP32 summation order. A launch captured into a CUDA graph keeps
 *     the values it was captured with: changing a variable afterwards does not affect replays.
 */
#ifndef FGA_H_
#define FGA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum FgaResult {
  FGA_SUCCESS = 0,
  FGA_INVALID_ARGUMENT = -1,
  FGA_CUDA_ERROR = -2,
  FGA_UNSUPPORTED = -3
} FgaResult;

typedef enum FgaDeviceError {
  FGA_DEV_OK = 0,
  FGA_DEV_BARRIER_TIMEOUT = 1,  /* a peer never published its barrier epoch */
  FGA_DEV_COUNTER_TIMEOUT = 2,  /* a receive row block never collected all arrivals */
  FGA_DEV_PIPELINE_TIMEOUT = 3, /* an in-kernel TMA/MMA/epilogue barrier never flipped */
  FGA_DEV_QUANT_TIMEOUT = 4     /* receive-side quantizer never saw its row block */
} FgaDeviceError;

#define FGA_IPC_HANDLE_BYTES 64

int fga_version(void);
const char* fga_last_error(void);
/* Number of SMs of the current device (grid sizing, also used by the host layer). */
int fga_sm_count(void);
/* Kernels this library has launched in this process so far (all entry points, all threads). */
uint64_t fga_launch_count(void);

/* ---- symmetric memory ---------------------------------------------------------------------
 * Replaces torch symmetric memory with the NVSHMEM backend, used by the reference only to
 * allocate and rendezvous peer-mapped buffers (fused_gemm_a2a.py:100, 118-127). One allocation
 * per buffer set; the 64-byte handle is exchanged once over the CP group by the host layer. */
int fga_symm_alloc(size_t bytes, void** ptr);                        /* cudaMalloc + zero fill */
int fga_symm_export(void* ptr, unsigned char handle[FGA_IPC_HANDLE_BYTES]);
int fga_symm_open(const unsigned char handle[FGA_IPC_HANDLE_BYTES], void** peer_ptr);
int fga_symm_close(void* peer_ptr);
int fga_symm_free(void* ptr);

/* The same buffers from the driver's virtual memory management API instead of cudaMalloc + CUDA IPC
 * (what the Python layer uses unless FGA_SYMM=ipc or a rank of the group cannot). The physical memory is reference counted
 * by every mapping, the owner's and each importer's, so a rank that exits does not pull the memory
 * out from under peers that are still storing into it. The shareable handle is a POSIX file
 * descriptor, which the host layer passes to the peers over a Unix-domain socket.
 *   fga_symm_vmm_size(bytes)          bytes rounded up to the allocation granularity (-1 on error);
 *                                      every rank maps this size.
 *   fga_symm_alloc_vmm(bytes, &p, &fd) zero-filled memory of fga_symm_vmm_size(bytes) mapped at p for the
 *                                      current device, and a descriptor for the peers (close it after
 *                                      the exchange).
 *   fga_symm_open_vmm(fd, size, &p)    map a peer's allocation of `size` = its fga_symm_vmm_size();
 *                                      the descriptor may be closed afterwards.
 *   fga_symm_release_vmm(p, size)      unmap either kind of mapping; the memory is freed with its
 *                                      last mapping. */
int64_t fga_symm_vmm_size(size_t bytes);
int fga_symm_alloc_vmm(size_t bytes, void** ptr, int* fd);
int fga_symm_open_vmm(int fd, size_t bytes, void** peer_ptr);
int fga_symm_release_vmm(void* ptr, size_t bytes);

/* ---- group barrier ------------------------------------------------------------------------
 * Replaces barrier / _barrier_kernel (fused_gemm_a2a_kernels.py:204-234; host wrapper
 * fused_gemm_a2a.py:129-135). flags: this rank's int64[P]; peer_flags: device int64[P] holding
 * every rank's flags address. bump != 0 zeroes counters[0:count] before publishing and increments
 * epoch_out[0] afterwards. */
int fga_barrier(int64_t* flags, const int64_t* peer_flags, int rank, int p, int bump,
                int32_t* counters, int count, int32_t* epoch_out, int32_t* status,
                uint64_t timeout_ns, void* stream);

/* ---- fused GEMMs --------------------------------------------------------------------------
 * Replace _Comm.gemm / UlyssesGemm (fused_gemm_a2a.py:162-234; fused_gemm_a2a_kernels.py:400-929).
 * b is [n, k] when b_is_kn == 0 and [k, n] otherwise. */

/* push: heads[seg] on peer dest receives rows [rank*head_rows, rank*head_rows + a_rows) of
 * a[m, k] * b^T (+ bias in FP32 when bias != NULL), one 128-column head tile at a time.
 * Rows of a beyond m read as zero. peer_heads[s]: device int64[P] of the peers' buffer bases for
 * segment s (s < segments; segments is 1, 3 or 4). n = segments * n_segment.
 * Reference: mode 'push' with _tile_mapping and _epilogue_push_simt
 * (fused_gemm_a2a_kernels.py:617-635, 900-913, 975-1050). */
int fga_gemm_push(const void* a, int m, int k, int a_rows, const void* b, int b_is_kn,
                  const void* bias, int segments, int n_segment, const int64_t* const* peer_heads,
                  int64_t head_rows, int rank, int p, int32_t* status, uint64_t timeout_ns,
                  void* stream);

/* recv: pusher warps copy srcs[t][d*src_rows + row, :] (t < num_in) into peer d's receive buffer
 * in [head][q|k|v|g][128] column order, rows >= src_rows as zeros, and bump peer d's counter of
 * that 128-row block; the GEMM c[recv_rows, n] = recv[recv_rows, k] * b^T consumes a row block
 * once its counter reaches p * num_in * split. roles: bit 0 GEMM, bit 1 pushers (both = 3).
 * progress (may be NULL): pacing of the pushers, used only with FGA_PUSH_LEAD > 0 and roles == 3. A
 * caller-owned device int32 that the launcher zeroes on the stream in front of the kernel and in
 * which the GEMM publishes 1 + the row tile it has reached; the pushers then stay a bounded number
 * of raster groups ahead of it. epoch is reserved and ignored (pass NULL or any device word).
 * Reference: mode 'recv' with _push_jobs / _push_one
 * (fused_gemm_a2a_kernels.py:291-380, 764-772, 798-804). */
int fga_gemm_recv(const void* recv, int recv_rows, int k, const void* b, int b_is_kn, int n,
                  void* c, const int64_t* peer_recv, const int64_t* peer_counters,
                  int32_t* counters, const void* const* srcs, int num_in, int src_rows, int split,
                  int rank, int p, int roles, const int64_t* epoch, int32_t* progress, int32_t* status,
                  uint64_t timeout_ns, void* stream);

/* Grouped-query attention: q_per_kv query heads share one key/value head. The weight rows of the QKV
 * projection (= output columns of the push, = receive-buffer columns of its dgrad) are grouped per
 * key/value head, [q_g0 .. q_g(r-1); k_g; v_g; (gate_g0 .. gate_g(r-1))] with r = q_per_kv, each head
 * 128 rows; rank d owns the kv_heads / p consecutive groups d*kv_heads/p ... With q_per_kv == 1 this is
 * the per-head order of fga_gemm_push / fga_gemm_recv with 3 or 4 segments. The reference rejects
 * these shapes in its fused modules (fused_gemm_a2a.py:592-593) and supports them only in its unfused
 * baseline (benchmark/reference.py:151-163), which is what the results are checked against.
 *   push: peer_heads holds 3 (4 with gate) tables: q, k, v(, gate). The q and gate buffers are
 *         [p*head_rows, kv_heads/p * q_per_kv * 128], the k and v buffers [p*head_rows, kv_heads/p * 128].
 *         a [m, k] * b^T with b [kv_heads*(q_per_kv*(1+gate)+2)*128, k]; bias indexed by weight row.
 *   recv: srcs holds the head-side gradients in the same order and with those widths
 *         ([p*src_rows, width]); recv is [recv_rows, K] with K = kv_heads*(q_per_kv*(1+gate)+2)*128 in
 *         weight-row order; c [recv_rows, n] = recv * b with b [K, n]. */
int fga_gemm_push_gqa(const void* a, int m, int k, int a_rows, const void* b, const void* bias, int kv_heads,
                      int q_per_kv, int gate, const int64_t* const* peer_heads, int64_t head_rows, int rank,
                      int p, int32_t* status, uint64_t timeout_ns, void* stream);
int fga_gemm_recv_gqa(const void* recv, int recv_rows, const void* b, int n, void* c, const int64_t* peer_recv,
                      const int64_t* peer_counters, int32_t* counters, const void* const* srcs, int kv_heads,
                      int q_per_kv, int gate, int src_rows, int split, int rank, int p, int roles,
                      int32_t* progress, int32_t* status, uint64_t timeout_ns, void* stream);

/* local: c[m, n] (=|+=) a * b^T with a as [m, k] (a_is_km == 0) or [k, m] (a_is_km != 0, read
 * transposed) and b as [n, k] or [k, n]. out_f32 selects FP32 output; accumulate (FP32 only) adds
 * into c. Rows of the reduction axis beyond k read as zero. With a_is_km = b_is_kn = 1 this is
 * the weight gradient dW = dY^T X with optional accumulation into main_grad.
 * Reference: _weight_grad (fused_gemm_a2a.py:249-275) and the 'local' mode with
 * _epilogue_accumulate (fused_gemm_a2a_kernels.py:914-918, 932-972). */
int fga_gemm_local(const void* a, int a_is_km, const void* b, int b_is_kn, int m, int n, int k,
                   int64_t lda, int64_t ldb, void* c, int64_t ldc, int out_f32, int accumulate,
                   int32_t* status, uint64_t timeout_ns, void* stream);

/* ---- MXFP8 variants -----------------------------------------------------------------------
 * Same three modes with E4M3 operands and one E8M0 scale per 32 elements of the reduction axis,
 * block-scaled tcgen05 MMAs, FP32 accumulation. Operands are what fga_mx_quantize writes: payload
 * [rows_padded, kp] (rows padded to 256, kp to a multiple of 128) and scale bytes in the tcgen05
 * 128-row x 4-group layout. Only BF16 ever crosses the links.
 * Reference: UlyssesGemm with mxfp8 (fused_gemm_a2a_kernels.py:445-502, 557-579, 834-866),
 * mxfp8_wgrad (1398-1421) and the receive-side quantizer _mx_quantize_received (1295-1343). */

/* c[m, n] (=|+=) dequant(aq) * dequant(bq)^T over kp. */
int fga_gemm_local_mx(const void* aq, const void* sfa, int64_t a_rows_padded, const void* bq,
                      const void* sfb, int64_t b_rows_padded, int m, int n, int kp, void* c, int64_t ldc,
                      int out_f32, int accumulate, int32_t* status, uint64_t timeout_ns, void* stream);

/* push with quantized activations aq [a_rows_padded, kp] and weights bq [b_rows_padded, kp]. */
int fga_gemm_push_mx(const void* aq, const void* sfa, int64_t a_rows_padded, int kp, int a_rows,
                     const void* bq, const void* sfb, int64_t b_rows_padded, const void* bias, int segments,
                     int n_segment, const int64_t* const* peer_heads, int64_t head_rows, int rank, int p,
                     int32_t* status, uint64_t timeout_ns, void* stream);

/* recv: the pushers move BF16 into the peers' receive buffers as in fga_gemm_recv; two more warps
 * per CTA quantize every arrived 128-row block of `recv` into mx_recv [recv_rows, k] / mx_scale
 * (8 rows per job, 16 completions per block on the same counter) and the GEMM reads those. */
int fga_gemm_recv_mx(const void* recv, void* mx_recv, void* mx_scale, int recv_rows, int k, const void* bq,
                     const void* sfb, int64_t b_rows_padded, int b_kp, int n, void* c,
                     const int64_t* peer_recv, const int64_t* peer_counters, int32_t* counters,
                     const void* const* srcs, int num_in, int src_rows, int split, int rank, int p,
                     int roles, const int64_t* epoch, int32_t* progress, int32_t* status,
                     uint64_t timeout_ns, void* stream);

/* Grouped-query attention with MXFP8 operands: fga_gemm_push_mx / fga_gemm_recv_mx with the grouped
 * column layout of fga_gemm_push_gqa / fga_gemm_recv_gqa (same buffers, tables and source widths). No
 * counterpart in the reference, whose fused modules reject these shapes. */
int fga_gemm_push_gqa_mx(const void* aq, const void* sfa, int64_t a_rows_padded, int kp, int a_rows, const void* bq,
                         const void* sfb, int64_t b_rows_padded, const void* bias, int kv_heads, int q_per_kv,
                         int gate, const int64_t* const* peer_heads, int64_t head_rows, int rank, int p,
                         int32_t* status, uint64_t timeout_ns, void* stream);
int fga_gemm_recv_gqa_mx(const void* recv, void* mx_recv, void* mx_scale, int recv_rows, const void* bq,
                         const void* sfb, int64_t b_rows_padded, int b_kp, int n, void* c, const int64_t* peer_recv,
                         const int64_t* peer_counters, int32_t* counters, const void* const* srcs, int kv_heads,
                         int q_per_kv, int gate, int src_rows, int split, int rank, int p, int roles,
                         int32_t* progress, int32_t* status, uint64_t timeout_ns, void* stream);

/* ---- auxiliary kernels -------------------------------------------------------------------- */

/* Replaces resize_rank_rows (fused_gemm_a2a_kernels.py:1145-1188). in/out: `segments` BF16
 * matrices [peers*rows_in, width] -> [peers*rows_out, width]. bias may be NULL. */
int fga_copy_rank_rows(const void* const* in, void* const* out, int segments, int peers,
                       int64_t rows_in, int64_t rows_out, int width, const void* bias,
                       int head_dim, int head_offset, void* stream);

/* Replaces reduce_bias_grad (fused_gemm_a2a_kernels.py:1086-1103). scratch: FP32 buffer of
 * fga_bias_grad_scratch_floats(rows, width) elements in device memory. */
int64_t fga_bias_grad_scratch_floats(int64_t rows, int width);
int fga_bias_grad(const void* dy, int64_t rows, int width, void* out, int out_is_f32,
                  int accumulate, float* scratch, void* stream);

/* No counterpart in the reference. The same reduction as fga_bias_grad for callers that cannot
 * hand over scratch memory because they must not allocate at the call site (a fully planned
 * memory budget, a host that forbids cudaMalloc in its hot path): the FP32 partial sums go to a
 * 4 MiB array that is part of the library's device image, so this call allocates nothing, and
 * neither does anything it calls. Limit: ceil(rows / 256) * width must not exceed
 * fga_bias_grad_static_capacity_floats() (1 Mi floats); larger problems are rejected with
 * FGA_INVALID_ARGUMENT. The first call on each device looks up the array's device address; make
 * that first call before any stream capture begins. All calls on a device share the array, which
 * keeps the previous call's partial sums; calls that overlap on the GPU race with each other. */
int64_t fga_bias_grad_static_capacity_floats(void);
int fga_bias_grad_static(const void* dy, int64_t rows, int width, void* out, int out_is_f32,
                         int accumulate, void* stream);

/* Replaces mxfp8_quantize / _mx_quant_kernel (fused_gemm_a2a_kernels.py:1222-1292, 1358-1376).
 * a: BF16 [rows, k] with element strides (stride_row, stride_k), one of them 1. q: E4M3
 * [rows_padded, k_padded]; sf: rows_padded*k_padded/32 E8M0 bytes in the tcgen05 128x4 layout. */
int fga_mx_quantize(const void* a, int64_t rows, int k, int64_t stride_row, int64_t stride_k,
                    void* q, void* sf, int64_t rows_padded, int k_padded, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FGA_H_ */
