// Host interface of the tensor-core dense scan (tc_scan.cu) and of the weight preparation kernels.
#pragma once

#include "common.cuh"

namespace b200gru {
namespace tc {

// Hidden weights Wh_cat[3H,H] in one of two forms: fp32 values (W), or int8 codes with one scale
// per output row (codes, row_scale: W[r,k] = codes[r,k] * row_scale[r]).
struct TcWeights {
  const float* W;
  const signed char* codes;
  const float* row_scale;
};

// Shape rule of the tensor-core path (the workspace query and the launch must agree).
bool tc_dense_path(int B, int H);
size_t tc_dense_fwd_scratch_bytes(int T, int B, int H, bool w_codes);
size_t tc_dense_bwd_scratch_bytes(int T, int B, int H, bool w_codes);

int launch_tc_dense_forward(const float* gi, const float* h0, const TcWeights& w, const float* bh, float* out,
                            float* save, void* scratch, int T, int B, int H, Quant qin, Quant qout, cudaStream_t st);
// dW is the gradient with respect to the weight VALUES (for codes: codes * row_scale).
int launch_tc_dense_backward(const float* h0, const TcWeights& w, const float* out, const float* S, const float* dout,
                             float* dgi, float* dh0, float* dW, float* dbh, void* scratch, int T, int B, int H,
                             Quant qin, Quant qout, cudaStream_t st);

// Weight gradient of the dense scan as one tensor-core product over all T*B rows (used after the
// cluster kernels' serial backward): dW[3H,H] = dgh^T . fq_in(h_prev), S = r activations [T*B][H].
bool tc_weight_grads_applies(int T, int B, int H);
size_t tc_weight_grads_scratch_bytes(int T, int B, int H, bool h_codes);
int launch_tc_weight_grads(const float* dgi, const float* S, const float* h0, const float* out, Quant qin, float* dW,
                           void* scratch, int T, int B, int H, cudaStream_t st);

// Per-output-row symmetric fake-quant of a weight matrix W[rows, cols] (dynamic scale
// s_r = max(max|row|, 1e-8) / qmax, qmax = 2^(bits-1) - 1): codes (int8), scales and, optionally,
// the fake-quantised fp32 values codes * s.  cols % 4 == 0, 2 <= bits <= 8.
int launch_quantize_rows(const float* W, int rows, int cols, int bits, signed char* codes, float* scales, float* Wq,
                         cudaStream_t st);
// Straight-through gradient of the same operation, including the path through the dynamic scale:
//   dW[r,k] = dWq[r,k] + [k == argmax_k |W[r,k]|] * sign(W[r,k]) / qmax * sum_k' dWq[r,k'] * (q[r,k'] - W[r,k'] / s_r)
int launch_quantize_rows_backward(const float* W, const float* dWq, int rows, int cols, int bits, float* dW,
                                  cudaStream_t st);

// dst[c] = sum over r of src[r][c] (fixed summation order); scratch of column_sums_scratch_bytes.
size_t column_sums_scratch_bytes(size_t rows, int cols);
int launch_column_sums(const float* src, size_t rows, int cols, float* dst, float* scratch, cudaStream_t st);

}  // namespace tc
}  // namespace b200gru
