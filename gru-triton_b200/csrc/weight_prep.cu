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

// ---- column sums (bias gradient of the input projection) -----------------------------------------
// partial[s][c] = sum of src[r][c] over the rows of slice s; a CTA takes 64 columns of one slice,
// four row groups of 64 threads each, combined in a fixed order.  The slices are added in order
// afterwards: no atomics.
__global__ void __launch_bounds__(256)
column_sums_kernel(const float* __restrict__ src, size_t rows, int cols, size_t rows_per_slice,
                   float* __restrict__ partial) {
  __shared__ float red[4][64];
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * 64 + (threadIdx.x & 63);
  const int grp = threadIdx.x >> 6;
  const size_t r0 = (size_t)blockIdx.y * rows_per_slice;
  const size_t r1 = r0 + rows_per_slice < rows ? r0 + rows_per_slice : rows;
  float s = 0.f;
  if (c < cols)
    for (size_t r = r0 + grp; r < r1; r += 4) s += __ldcs(src + r * cols + c);
  red[grp][threadIdx.x & 63] = s;
  __syncthreads();
  if (grp == 0 && c < cols)
    partial[(size_t)blockIdx.y * cols + c] = ((red[0][threadIdx.x] + red[1][threadIdx.x]) + red[2][threadIdx.x]) + red[3][threadIdx.x];
}

// The same for cols % 4 == 0: a CTA takes 256 columns (float4 per thread), four row groups, four
// independent partial sums per thread so that the loads overlap.
__global__ void __launch_bounds__(256)
column_sums4_kernel(const float* __restrict__ src, size_t rows, int cols, size_t rows_per_slice,
                    float* __restrict__ partial) {
  __shared__ float4 red[4][64];
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.x * 64 + (threadIdx.x & 63)) * 4;
  const int grp = threadIdx.x >> 6;
  const size_t r0 = (size_t)blockIdx.y * rows_per_slice;
  const size_t r1 = r0 + rows_per_slice < rows ? r0 + rows_per_slice : rows;
  float4 s[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < cols) {
    size_t r = r0 + grp;
    for (; r + 12 < r1; r += 16) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(src + (r + 4 * u) * cols + c));
        s[u].x += v.x; s[u].y += v.y; s[u].z += v.z; s[u].w += v.w;
      }
    }
    for (; r < r1; r += 4) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(src + r * cols + c));
      s[0].x += v.x; s[0].y += v.y; s[0].z += v.z; s[0].w += v.w;
    }
  }
  float4 t;
  t.x = (s[0].x + s[1].x) + (s[2].x + s[3].x); t.y = (s[0].y + s[1].y) + (s[2].y + s[3].y);
  t.z = (s[0].z + s[1].z) + (s[2].z + s[3].z); t.w = (s[0].w + s[1].w) + (s[2].w + s[3].w);
  red[grp][threadIdx.x & 63] = t;
  __syncthreads();
  if (grp == 0 && c < cols) {
    const int i = threadIdx.x;
    float4 o;
    o.x = ((red[0][i].x + red[1][i].x) + red[2][i].x) + red[3][i].x;
    o.y = ((red[0][i].y + red[1][i].y) + red[2][i].y) + red[3][i].y;
    o.z = ((red[0][i].z + red[1][i].z) + red[2][i].z) + red[3][i].z;
    o.w = ((red[0][i].w + red[1][i].w) + red[2][i].w) + red[3][i].w;
    *reinterpret_cast<float4*>(partial + (size_t)blockIdx.y * cols + c) = o;
  }
}

static int column_slices(size_t rows, int cols) {
  const int col_tiles = cdiv(cols, (cols % 4 == 0) ? 256 : 64);
  int s = cdiv(2 * 148, col_tiles);
  const size_t by_rows = (rows + 63) / 64;
  if ((size_t)s > by_rows) s = (int)by_rows;
  return s < 1 ? 1 : s;
}

size_t column_sums_scratch_bytes(size_t rows, int cols) {
  return align_up((size_t)column_slices(rows, cols) * cols * sizeof(float), 256);
}

int launch_column_sums(const float* src, size_t rows, int cols, float* dst, float* scratch, cudaStream_t st) {
  if (src == nullptr || dst == nullptr || scratch == nullptr || cols <= 0) return B200GRU_INVALID_ARGUMENT;
  if (rows == 0) {
    cudaMemsetAsync(dst, 0, (size_t)cols * sizeof(float), st);
    return check_launch("column sums");
  }
  if (rows <= 16) {                               // a handful of partial results: one pass, fixed order
    launch_reduce_partials(src, (int)rows, (size_t)cols, (size_t)cols, dst, st);
    return check_launch("reduce_partials");
  }
  const int slices = column_slices(rows, cols);
  const size_t rps = (rows + slices - 1) / slices;
  const int used = (int)((rows + rps - 1) / rps);
  if (cols % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0)
    launch_pdl(column_sums4_kernel, dim3(cdiv(cols, 256), used), dim3(256), 0, st, src, rows, cols, rps, scratch);
  else
    launch_pdl(column_sums_kernel, dim3(cdiv(cols, 64), used), dim3(256), 0, st, src, rows, cols, rps, scratch);
  note_launch();
  launch_reduce_partials(scratch, used, (size_t)cols, (size_t)cols, dst, st);
  return check_launch("column_sums_kernel");
}

}  // namespace tc
}  // namespace b200gru
