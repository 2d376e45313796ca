/*
 * b200gru -- C ABI of the B200 (sm_100a) persistent GRU scan library.
 *
 * One shared library, plain pointers and sizes, no framework types.  Every
 * entry point replaces one Python wrapper of LarocheC/gru-triton (package
 * gru_qat); the citation beside each declaration names the file:line of the
 * reference interface it stands in for.
 *
 * Conventions shared by all entry points
 *  - all tensors are fp32 device pointers, row-major, last dimension contiguous
 *    and tightly packed: gi[T,B,3H] (gates r,z,n stacked along the last axis,
 *    input bias already added), h0[B,H], bh[3H], out[T,B,H];
 *  - q_in / q_out describe the frozen per-tensor symmetric fake-quant of the
 *    hidden state (NULL or enabled == 0 -> off);
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, the
 *    library never synchronises and never allocates: scratch memory comes from
 *    the caller (`workspace`, size from b200gru_workspace_bytes, 256-byte aligned);
 *  - return value 0 = success, otherwise a b200gru_status (see b200gru_strerror).
 */
#ifndef B200GRU_H
#define B200GRU_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  B200GRU_OK = 0,
  B200GRU_INVALID_ARGUMENT = 1,   /* NULL pointer, non-positive size, bad shape relation   */
  B200GRU_UNSUPPORTED = 2,        /* shape outside what this build can run                  */
  B200GRU_LAUNCH_FAILURE = 3,     /* cudaGetLastError() != cudaSuccess after a launch       */
  B200GRU_WORKSPACE_TOO_SMALL = 4, /* workspace_bytes < b200gru_workspace_bytes(...)        */
  B200GRU_SCRATCH_EXCEEDED = 5    /* problem too large for the built-in scratch of a _noalloc call */
} b200gru_status;

typedef enum {
  B200GRU_DENSE = 0,
  B200GRU_DIAGONAL = 1,
  B200GRU_MONARCH = 2,    /* one block-diagonal factor per gate */
  B200GRU_BUTTERFLY = 3
} b200gru_kind;

/* (scale, qmin, qmax) of gru_qat's h_in_quant / h_out_quant tuples
 * (src/gru_qat/gru_layer.py:30-48; semantics src/gru_qat/triton_kernels/scan.py:1450-1457):
 * fq(x) = clamp(rint(x / scale), qmin, qmax) * scale, round-half-to-even. */
typedef struct {
  float scale;
  int qmin;
  int qmax;
  int enabled;
} b200gru_quant;

/* Problem shape.  nblocks: MONARCH = number of diagonal blocks (block size H/nblocks);
 * BUTTERFLY = number of stacked butterfly factors.  log2_hpad: BUTTERFLY only, twiddles
 * are [3, nblocks, log2_hpad, hpad/2, 2, 2] with hpad = 1 << log2_hpad >= H. */
typedef struct {
  int kind;
  int T, B, H;
  int nblocks;
  int log2_hpad;
} b200gru_shape;

/* Bytes of caller-provided scratch needed by the forward (backward == 0), by a backward that
 * recomputes the gate activations (backward == 1), or by a backward that is handed the
 * forward's `save` buffer (backward == 2) of `shape`.  0 is a valid answer.  Returns (size_t)-1
 * for an invalid shape.  Replaces the torch.zeros/torch.empty scratch allocations
 * of the reference wrappers (scan.py:710-717, scan_monarch.py:848-856,
 * scan_butterfly.py:429-432, 1033-1040). */
size_t b200gru_workspace_bytes(const b200gru_shape* shape, int backward);

/* Bytes of the optional `save` buffer (gate activations r, z, n and the n-gate
 * hidden pre-activation, [4,T,B,H] fp32) that the forward can emit and the backward
 * can consume to skip its recompute pass.  No reference counterpart: the reference
 * recomputes the gates inside its backward kernels (scan.py:389-432). */
size_t b200gru_save_bytes(const b200gru_shape* shape);

/* Generic forward: out[T,B,H] from gi, h0, W, bh.  `save` may be NULL.
 * Replaces gru_scan_forward_persistent (scan.py:213-293), gru_scan_forward
 * (scan.py:1688-1765), gru_scan_diagonal_forward_triton (scan_diagonal.py:226-282),
 * gru_scan_monarch_forward_triton (scan_monarch.py:320-406) and
 * gru_scan_butterfly_forward_triton (scan_butterfly.py:369-459). */
int b200gru_scan_forward(const b200gru_shape* shape,
                         const float* gi, const float* h0, const float* W, const float* bh,
                         const b200gru_quant* q_in, const b200gru_quant* q_out,
                         float* out, float* save,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Generic backward: (dgi[T,B,3H], dh0[B,H], dW like W, dbh[3H]) from the forward's
 * inputs, its `out`, and dout[T,B,H].  Every output element is written (no
 * pre-zeroing needed).  `save` is the forward's save buffer or NULL (then the
 * gates are recomputed).  Replaces gru_scan_backward_persistent (scan.py:646-752),
 * gru_scan_backward_triton (scan.py:1355-1447), gru_scan_diagonal_backward_triton
 * (scan_diagonal.py:490-561), gru_scan_monarch_backward_triton
 * (scan_monarch.py:776-884) and gru_scan_butterfly_backward_triton
 * (scan_butterfly.py:971-1075), including their trailing partial.sum(0). */
int b200gru_scan_backward(const b200gru_shape* shape,
                          const float* gi, const float* h0, const float* W, const float* bh,
                          const float* out, const float* dout, const float* save,
                          const b200gru_quant* q_in, const b200gru_quant* q_out,
                          float* dgi, float* dh0, float* dW, float* dbh,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Per-kind conveniences with the argument order of the reference functions.
 * W is Wh_cat[3H,H] (dense), Wh_diag[3,H], Wh_struct[3,nblocks,H/nblocks,H/nblocks]
 * or twiddles[3,nblocks,log2_hpad,hpad/2,2,2]. */

/* gru_scan_forward_persistent, scan.py:213 */
int b200gru_dense_forward(const float* gi, const float* h0, const float* Wh_cat, const float* bh_cat,
                          int T, int B, int H, const b200gru_quant* q_in, const b200gru_quant* q_out,
                          float* out, float* save, void* workspace, size_t workspace_bytes, void* stream);
/* gru_scan_backward_persistent, scan.py:646 */
int b200gru_dense_backward(const float* gi, const float* h0, const float* Wh_cat, const float* bh_cat,
                           const float* out, const float* dout, const float* save,
                           int T, int B, int H, const b200gru_quant* q_in, const b200gru_quant* q_out,
                           float* dgi, float* dh0, float* dWh, float* dbh,
                           void* workspace, size_t workspace_bytes, void* stream);
/* gru_scan_diagonal_forward_triton, scan_diagonal.py:226 */
int b200gru_diagonal_forward(const float* gi, const float* h0, const float* Wh_diag, const float* bh_cat,
                             int T, int B, int H, const b200gru_quant* q_in, const b200gru_quant* q_out,
                             float* out, void* stream);
/* gru_scan_diagonal_backward_triton, scan_diagonal.py:490 */
int b200gru_diagonal_backward(const float* gi, const float* h0, const float* Wh_diag, const float* bh_cat,
                              const float* out, const float* dout,
                              int T, int B, int H, const b200gru_quant* q_in, const b200gru_quant* q_out,
                              float* dgi, float* dh0, float* dWh_diag, float* dbh,
                              void* workspace, size_t workspace_bytes, void* stream);
/* gru_scan_monarch_forward_triton, scan_monarch.py:320 */
int b200gru_monarch_forward(const float* gi, const float* h0, const float* Wh_struct, const float* bh_cat,
                            int T, int B, int H, int nblocks,
                            const b200gru_quant* q_in, const b200gru_quant* q_out,
                            float* out, float* save, void* workspace, size_t workspace_bytes, void* stream);
/* gru_scan_monarch_backward_triton, scan_monarch.py:776 */
int b200gru_monarch_backward(const float* gi, const float* h0, const float* Wh_struct, const float* bh_cat,
                             const float* out, const float* dout, const float* save,
                             int T, int B, int H, int nblocks,
                             const b200gru_quant* q_in, const b200gru_quant* q_out,
                             float* dgi, float* dh0, float* dWh_struct, float* dbh,
                             void* workspace, size_t workspace_bytes, void* stream);
/* gru_scan_butterfly_forward_triton, scan_butterfly.py:369 */
int b200gru_butterfly_forward(const float* gi, const float* h0, const float* twiddles, const float* bh_cat,
                              int T, int B, int H, int nblocks, int log2_hpad,
                              const b200gru_quant* q_in, const b200gru_quant* q_out,
                              float* out, float* save, void* workspace, size_t workspace_bytes, void* stream);
/* gru_scan_butterfly_backward_triton, scan_butterfly.py:971 */
int b200gru_butterfly_backward(const float* gi, const float* h0, const float* twiddles, const float* bh_cat,
                               const float* out, const float* dout, const float* save,
                               int T, int B, int H, int nblocks, int log2_hpad,
                               const b200gru_quant* q_in, const b200gru_quant* q_out,
                               float* dgi, float* dh0, float* dtwiddles, float* dbh,
                               void* workspace, size_t workspace_bytes, void* stream);

/* ---- dense layers with int8 weights ------------------------------------------------------------
 * Weight preparation: per-output-row symmetric fake-quant of W[rows, cols]
 * (s_r = max(max_k |W[r,k]|, 1e-8) / qmax, q = clamp(rint(W / s_r), -qmax, qmax), qmax = 2^(bits-1) - 1,
 * 2 <= bits <= 8, cols % 4 == 0): emits the int8 codes, the row scales and (Wq may be NULL) the
 * fake-quantised values q * s_r.  Replaces the per-gate FakeQuantizePerChannel(axis=0) calls of
 * GRUCellQuant.quantize_weights / quantize_input_weights (src/gru_qat/gru_cell.py:239-299;
 * src/gru_qat/quantizers.py:118-134, 177-189) for weights stacked r,z,n along the rows. */
int b200gru_quantize_rows(const float* W, int rows, int cols, int bits, signed char* codes, float* scales,
                          float* Wq, void* stream);
/* Its gradient, dW from dWq, as autograd derives it from fake_quant_ste with a dynamic scale
 * (src/gru_qat/ste.py:65-95): the clamp mask on dWq plus the term that reaches the row's largest
 * element through s_r. */
int b200gru_quantize_rows_backward(const float* W, const float* dWq, int rows, int cols, int bits, float* dW,
                                   void* stream);

/* Dense scan whose hidden weights come from b200gru_quantize_rows: Wq (fp32 values), codes and
 * scales of Wh_cat[3H,H].  Same results as b200gru_dense_forward / _backward on Wq (same workspace
 * sizes, b200gru_workspace_bytes with kind DENSE); at GEMM-sized batch the products run on the
 * integer codes (int8 x int8 -> int32 in the forward when the hidden state is quantised too).
 * dWq is the gradient with respect to Wq; feed it to b200gru_quantize_rows_backward.  Stands in
 * for gru_scan_persistent on the weights of GRUCellQuant.quantize_weights() (README.md:65-74,
 * src/gru_qat/gru_cell.py:239-271 of the reference). */
int b200gru_dense_q8_forward(const float* gi, const float* h0, const float* Wq, const signed char* codes,
                             const float* scales, const float* bh_cat, int T, int B, int H,
                             const b200gru_quant* q_in, const b200gru_quant* q_out, float* out, float* save,
                             void* workspace, size_t workspace_bytes, void* stream);
int b200gru_dense_q8_backward(const float* gi, const float* h0, const float* Wq, const signed char* codes,
                              const float* scales, const float* bh_cat, const float* out, const float* dout,
                              const float* save, int T, int B, int H, const b200gru_quant* q_in,
                              const b200gru_quant* q_out, float* dgi, float* dh0, float* dWq, float* dbh,
                              void* workspace, size_t workspace_bytes, void* stream);

/* ---- tensor-core GEMM core (tcgen05 / tensor memory) ------------------------------------------
 * The products of the path that are real GEMMs -- the input projection gi = x . Wi^T + bi
 * (F.linear, src/gru_qat/gru_layer.py:251-253, src/gru_qat/gru_cell.py:410-435), the per-step
 * h . Wh^T and dgh . Wh at GEMM-sized batch (tl.dot, src/gru_qat/triton_kernels/scan.py:153-155,
 * 521-569) and the weight gradients dgh^T . h (scan.py:573-616) -- run on one kernel:
 *
 *   C[s][M,N] = alpha * row_scale[m] * col_scale[n] * sum_q A_{pair_a[q]} . B_{pair_b[q]}^T + bias[n]
 *
 * Operands are bf16 (dtype 0, fp32 accumulation), int8 (dtype 1, exact int32 accumulation) or
 * fp16 (dtype 2, fp32 accumulation) and come as 1..3 planes: an fp32 operand is split into bf16
 * terms hi + mid + lo by b200gru_split_bf16 (three planes are exact) or into two row-scaled fp16
 * terms by b200gru_split_f16 (22 significant bits; three cross products instead of six), an
 * operand on an int8 grid is one exact plane of codes.  pair_a / pair_b list the plane cross
 * products to accumulate.
 *   a_mn_major == 0: A is [planes][M][lda] (K contiguous);  1: A is [planes][K][lda] (M contiguous)
 *   b_mn_major == 0: B is [planes][N][ldb] (K contiguous);  1: B is [planes][K][ldb] (N contiguous)
 * (int8 operands: K contiguous only).  Strides in elements; bases 16-byte aligned; byte strides
 * multiples of 16; N and ldc multiples of 4.  split_k > 1 writes split_k partial matrices
 * `split_stride` floats apart (sum them in order); it must be the value b200gru_tc_gemm_splits
 * returns for the wanted count.  row_scale / col_scale / bias may be NULL.
 * The tensor core's fp32 accumulator truncates, so the sum is built in chunks: chunk_kblocks
 * k-blocks (64 bf16 / 128 int8 elements of K each) are accumulated in tensor memory, then added
 * to a register total with round-to-nearest.  0 picks at most 32 accumulation steps per chunk
 * (int8: one chunk, the int32 sum is exact). */
typedef struct {
  int dtype;
  int M, N, K;
  const void* A;
  const void* B;
  int a_planes, b_planes;
  int a_mn_major, b_mn_major;
  long long lda, ldb, a_plane_stride, b_plane_stride;
  int npairs;
  int pair_a[9], pair_b[9];
  int split_k;
  int tile_n;             /* 0 = library's choice, else 64, 128 or 256 */
  int chunk_kblocks;      /* 0 = library's choice; see below */
  int accumulate;         /* != 0: add the result to what C already holds */
  float alpha;
  const float* row_scale;
  const float* col_scale;
  const float* bias;
  float* C;
  long long ldc, split_stride;
} b200gru_gemm_args;

int b200gru_tc_gemm(const b200gru_gemm_args* args, void* stream);
int b200gru_tc_gemm_splits(const b200gru_gemm_args* args, int wanted);

/* dst[p][i] (bf16, planes `plane_stride` elements apart) = p-th bf16 term of
 * src[i] * col_scale[i % ncols] (col_scale may be NULL): hi = RN(x), mid = RN(x - hi),
 * lo = RN(x - hi - mid).  n % 4 == 0.  Operand preparation for b200gru_tc_gemm; the reference
 * feeds fp32 tensors to tl.dot / cuBLAS directly. */
int b200gru_split_bf16(const float* src, void* dst, size_t n, size_t plane_stride, int planes,
                       const float* col_scale, int ncols, void* stream);

/* dst[0 | 1][r][c] (fp16, planes `plane_stride` elements apart) = leading / trailing fp16 term of
 * src[r][c] * 2^k_r, with 2^k_r chosen per row so that the row's largest element lands in
 * [2^14, 2^15); inv_scale[r] = 2^-k_r is the row_scale (A operand) or col_scale (B operand) of the
 * product.  cols % 4 == 0.  Operand preparation like b200gru_split_bf16. */
int b200gru_split_f16(const float* src, void* dst, int rows, int cols, size_t plane_stride, float* inv_scale,
                      void* stream);

/* dst[c] = sum over r of src[r][c] for a contiguous src[rows][cols], in a fixed summation order
 * (two-level: row slices, then the slices in order).  The bias gradient of the input projection
 * (autograd of F.linear at src/gru_qat/gru_layer.py:251-253) and the sum of split-K partials. */
size_t b200gru_column_sums_workspace_bytes(size_t rows, int cols);
int b200gru_column_sums(const float* src, size_t rows, int cols, float* dst, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Diagonal backward for callers that cannot allocate device memory.  It has no counterpart in
 * the reference (whose wrappers always allocate their scratch with torch).  Same inputs, outputs
 * and results as b200gru_diagonal_backward, but no workspace argument: the partial sums go into a
 * buffer of B200GRU_NOALLOC_SCRATCH_BYTES built into the library (held on every GPU the process
 * uses, for the life of the process).  Meant for hosts that run under someone else's memory
 * budget or on a path where cudaMalloc is forbidden; the call itself performs no allocation.
 *  - Limit: ceil(B/4) * 6 * H * 4 bytes must fit the buffer (e.g. B=256, H=1024 needs 1.5 MiB);
 *    larger problems return B200GRU_SCRATCH_EXCEEDED and launch nothing.
 *  - The first call on each device looks up the buffer's device address; make that first call
 *    outside any stream capture.
 *  - All calls share the one buffer per device.  Nothing needs clearing between calls, but two
 *    calls that overlap on the GPU (different streams) race on it: serialise them. */
#define B200GRU_NOALLOC_SCRATCH_BYTES (4u << 20)
int b200gru_diagonal_backward_noalloc(const float* gi, const float* h0, const float* Wh_diag,
                                      const float* bh_cat, const float* out, const float* dout,
                                      int T, int B, int H, const b200gru_quant* q_in,
                                      const b200gru_quant* q_out, float* dgi, float* dh0,
                                      float* dWh_diag, float* dbh, void* stream);

/* Number of kernels the library has launched in this process since it was loaded
 * (all streams).  Used by the benchmark to report its launch count; no reference
 * counterpart. */
unsigned long long b200gru_launch_count(void);

/* Health of the in-kernel waits on the current device.  The dense / block-diagonal kernels
 * exchange data between the CTAs of a cluster and wait for it with a bounded number of polls;
 * a wait that gives up sets a device flag and lets the kernel finish (its results are then
 * invalid).  This call SYNCHRONISES the device and returns that flag (0 = healthy, 1 = a wait
 * gave up, -1 = CUDA error); reset != 0 clears it.  Meant for tests and post-mortems, not for
 * the hot path.  No reference counterpart: the reference's spin-wait is unbounded
 * (scan.py:202-205). */
int b200gru_device_status(int reset);

/* ---- calibration on the device --------------------------------------------------------------
 * Forward scan with the two hidden-state quantisers in observing ("min_max") mode, the state
 * GRULayer.calibrate() puts them in (src/gru_qat/gru_layer.py:308-339, src/gru_qat/calibration.py:
 * 30-135): at every step quant_h_in sees h_{t-1} and quant_h_out sees h_raw_t; each call
 * fake-quantises with the dynamic symmetric scale max(|min|, |max|, 1e-8) / qmax of its own
 * argument and folds (min, max) into the running range -- set by the first call, blended with
 * `momentum` (0.99 in the reference, src/gru_qat/quantizers.py:136-156) afterwards.  The reference
 * runs this through its Python per-step cell; here the ranges, scales and running statistics stay
 * in device memory and nothing synchronises with the host.
 * in_min/in_max, out_min/out_max: one float each in device memory, the running ranges of the two
 * quantisers (read when *_initialized != 0, always written).  out[T,B,H] receives the quantised
 * states.  Every hidden kind; no frozen quantiser is involved, so there are no q_in / q_out. */
size_t b200gru_calibration_workspace_bytes(const b200gru_shape* shape);
int b200gru_calibration_scan(const b200gru_shape* shape, const float* gi, const float* h0, const float* W,
                             const float* bh, int qmax, double momentum, float* in_min, float* in_max,
                             int in_initialized, float* out_min, float* out_max, int out_initialized,
                             float* out, void* workspace, size_t workspace_bytes, void* stream);

/* ---- test hooks (no reference counterpart; not for production callers) ------------------------
 * b200gru_test_select_kernels: the library keeps two kernels for some problems and picks by
 * shape; a non-zero argument makes the butterfly launches use the register / global-twiddle
 * kernels, resp. the diagonal forward use its register-ring kernel, on every shape, so that the
 * tests can hold both to the same parity bar.  Process-wide; (0, 0) restores the normal dispatch.
 * b200gru_test_wait_timeout: launches one tiny kernel whose bounded wait must run out (it waits
 * about a millisecond for bytes nothing sends), which sets the flag b200gru_device_status
 * reports; the kernel returns normally and the device stays usable. */
void b200gru_test_select_kernels(int butterfly_register_kernels, int diagonal_register_ring);
int b200gru_test_wait_timeout(void* stream);

/* Human-readable text for a b200gru_status; plus the text of the last CUDA error
 * seen by a launch in this thread (empty string if none). */
const char* b200gru_strerror(int status);
const char* b200gru_last_cuda_error(void);

/* Library version: major*10000 + minor*100 + patch. */
int b200gru_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200GRU_H */
