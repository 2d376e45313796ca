// Weight preparation: per-output-row symmetric fake-quant of a weight matrix, emitting the int8
// codes and row scales the tensor-core products consume, and its straight-through gradient.
//
// Reference semantics (src/gru_qat/quantizers.py:118-134, 177-189 with axis = 0, dynamic mode;
// applied per gate in src/gru_qat/gru_cell.py:239-299; arithmetic src/gru_qat/ste.py:65-95):
//   s_r = max(max_k |W[r,k]|, 1e-8) / qmax,   q = clamp(rint(W / s_r), -qmax, qmax),   Wq = q * s_r
// with a true fp32 division and round-half-to-even.  The scale is part of the autograd graph there
// (it is computed from W), so the gradient has a second term that lands on the row's largest
// element:  dW[r,k] = mask * dWq[r,k] + [k = argmax|W[r,:]|] * sign(W[r,k]) / qmax * G_r,
//           G_r = sum_k dWq[r,k] * (q[r,k] - mask * W[r,k] / s_r).
// One CTA per row; all reductions run in a fixed order.

#include "tc_scan.cuh"

namespace b200gru {
namespace tc {

namespace {

constexpr int WP_THREADS = 256;

struct RowMax {
  float v;
  int k;
};

// Largest |W[r,k]| of the row and its first index, identical in every thread.
__device__ RowMax row_absmax(const float* __restrict__ row, int cols) {
  __shared__ float sv[WP_THREADS];
  __shared__ int sk[WP_THREADS];
  float best = -1.0f;
  int bk = 0;
  for (int k = threadIdx.x; k < cols; k += WP_THREADS) {
    const float a = fabsf(row[k]);
    if (a > best) { best = a; bk = k; }
  }
  sv[threadIdx.x] = best; sk[threadIdx.x] = bk;
  __syncthreads();
  for (int off = WP_THREADS / 2; off > 0; off >>= 1) {
    if (threadIdx.x < off) {
      const float o = sv[threadIdx.x + off];
      const int ok = sk[threadIdx.x + off];
      if (o > sv[threadIdx.x] || (o == sv[threadIdx.x] && ok < sk[threadIdx.x])) { sv[threadIdx.x] = o; sk[threadIdx.x] = ok; }
    }
    __syncthreads();
  }
  RowMax r;
  r.v = sv[0]; r.k = sk[0];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(WP_THREADS)
quantize_rows_kernel(const float* __restrict__ W, int cols, float qmax, signed char* __restrict__ codes,
                     float* __restrict__ scales, float* __restrict__ Wq) {
  const size_t base = (size_t)blockIdx.x * cols;
  const RowMax m = row_absmax(W + base, cols);
  const float s = __fdiv_rn(fmaxf(m.v, 1e-8f), qmax);
  if (threadIdx.x == 0) scales[blockIdx.x] = s;
  for (int k = threadIdx.x * 4; k < cols; k += WP_THREADS * 4) {
    const float4 w = *reinterpret_cast<const float4*>(W + base + k);
    const float x[4] = {w.x, w.y, w.z, w.w};
    float q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) q[e] = fminf(fmaxf(rintf(__fdiv_rn(x[e], s)), -qmax), qmax);
    *reinterpret_cast<char4*>(codes + base + k) =
        make_char4((signed char)(int)q[0], (signed char)(int)q[1], (signed char)(int)q[2], (signed char)(int)q[3]);
    if (Wq != nullptr)
      *reinterpret_cast<float4*>(Wq + base + k) = make_float4(q[0] * s, q[1] * s, q[2] * s, q[3] * s);
  }
}

__global__ void __launch_bounds__(WP_THREADS)
quantize_rows_bwd_kernel(const float* __restrict__ W, const float* __restrict__ dWq, int cols, float qmax,
                         float* __restrict__ dW) {
  __shared__ float red[WP_THREADS];
  const size_t base = (size_t)blockIdx.x * cols;
  const RowMax m = row_absmax(W + base, cols);
  const float s = __fdiv_rn(fmaxf(m.v, 1e-8f), qmax);
  float g_acc = 0.f;
  for (int k = threadIdx.x * 4; k < cols; k += WP_THREADS * 4) {
    const float4 w = *reinterpret_cast<const float4*>(W + base + k);
    const float4 g = *reinterpret_cast<const float4*>(dWq + base + k);
    const float x[4] = {w.x, w.y, w.z, w.w}, gv[4] = {g.x, g.y, g.z, g.w};
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float v = __fdiv_rn(x[e], s);
      const float r = rintf(v);
      const float mask = (r >= -qmax && r <= qmax) ? 1.0f : 0.0f;
      const float q = fminf(fmaxf(r, -qmax), qmax);
      o[e] = gv[e] * mask;
      g_acc += gv[e] * (q - mask * v);
    }
    *reinterpret_cast<float4*>(dW + base + k) = make_float4(o[0], o[1], o[2], o[3]);
  }
  red[threadIdx.x] = g_acc;
  __syncthreads();
  for (int off = WP_THREADS / 2; off > 0; off >>= 1) {
    if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0 && m.v > 1e-8f) {
    const float sign = W[base + m.k] < 0.f ? -1.0f : 1.0f;
    dW[base + m.k] += sign * red[0] / qmax;          // same thread block wrote dW[base + m.k] above
  }
}

bool ok_args(const void* a, const void* b, int rows, int cols, int bits) {
  return a != nullptr && b != nullptr && rows > 0 && cols > 0 && (cols & 3) == 0 && bits >= 2 && bits <= 8 &&
         (reinterpret_cast<uintptr_t>(a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(b) & 15u) == 0;
}

}  // namespace

int launch_quantize_rows(const float* W, int rows, int cols, int bits, signed char* codes, float* scales, float* Wq,
                         cudaStream_t st) {
  if (!ok_args(W, codes, rows, cols, bits) || scales == nullptr) return B200GRU_INVALID_ARGUMENT;
  if (Wq != nullptr && (reinterpret_cast<uintptr_t>(Wq) & 15u)) return B200GRU_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(codes) & 3u)) return B200GRU_INVALID_ARGUMENT;
  const float qmax = (float)((1 << (bits - 1)) - 1);
  quantize_rows_kernel<<<rows, WP_THREADS, 0, st>>>(W, cols, qmax, codes, scales, Wq);
  note_launch();
  return check_launch("quantize_rows_kernel");
}

int launch_quantize_rows_backward(const float* W, const float* dWq, int rows, int cols, int bits, float* dW,
                                  cudaStream_t st) {
  if (!ok_args(W, dWq, rows, cols, bits) || dW == nullptr || (reinterpret_cast<uintptr_t>(dW) & 15u))
    return B200GRU_INVALID_ARGUMENT;
  const float qmax = (float)((1 << (bits - 1)) - 1);
  quantize_rows_bwd_kernel<<<rows, WP_THREADS, 0, st>>>(W, dWq, cols, qmax, dW);
  note_launch();
  return check_launch("quantize_rows_bwd_kernel");
}

}  // namespace tc
}  // namespace b200gru
