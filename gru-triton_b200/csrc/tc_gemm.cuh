// Host interface of the tensor-core GEMM core (tc_gemm.cu).
#pragma once

#include "common.cuh"

namespace b200gru {
namespace tc {

constexpr int TC_MAX_PAIRS = 9;
constexpr int TC_MAX_STAGES = 8;
constexpr int TC_SMEM_BUDGET = 208 * 1024;    // bytes of the operand ring

enum { TC_KIND_BF16 = 0, TC_KIND_I8 = 1, TC_KIND_F16 = 2 };

// C[split][M,N] (fp32, row stride ldc) = alpha * row_scale[m] * col_scale[n] * sum_q A_{pa[q]} . B_{pb[q]}^T + bias[n]
// over the K slice of each split.  Operand element type: bf16 (kind 0), int8 (kind 1) or fp16 (kind 2).
//   a_mn == 0: A is [planes][M][lda], K contiguous.   a_mn == 1: A is [planes][K][lda], M contiguous.
//   b_mn == 0: B is [planes][N][ldb], K contiguous.   b_mn == 1: B is [planes][K][ldb], N contiguous.
// Strides are in elements; bases 16-byte aligned, byte strides multiples of 16; N % 4 == 0.
// scale / bias pointers may be NULL.  split_k > 1: C holds split_k partial matrices `split_stride`
// floats apart, split_k must equal tc_gemm_splits(g, wanted).
struct TcGemm {
  int kind;
  int M, N, K;
  const void* A;
  const void* B;
  int a_planes, b_planes;
  int a_mn, b_mn;
  long long lda, ldb, a_plane_stride, b_plane_stride;
  int npairs;
  int pa[TC_MAX_PAIRS], pb[TC_MAX_PAIRS];
  int split_k;
  int tile_n;                  // 0 = choose; else 64 / 128 / 256
  int chunk_kb;                // 0 = choose; k-blocks accumulated in tensor memory between drains
  int accumulate;              // != 0: add the result to what C already holds
  float alpha;
  const float* row_scale;
  const float* col_scale;
  const float* bias;
  float* C;
  long long ldc, split_stride;
};

// K elements per k-block of this problem (the unit split_k divides).
int tc_gemm_kblock(const TcGemm& g);
// Number of K slices actually used when `want` are asked for (no slice is empty).
int tc_gemm_splits(const TcGemm& g, int want);
int tc_gemm_tile_n(const TcGemm& g);
int launch_tc_gemm(const TcGemm& g, cudaStream_t st);

// Launches the bounded-wait probe (a wait that must run out); sets the tensor-core health word.
int launch_wait_timeout_probe(cudaStream_t st);

// dst[pl][i] (bf16, planes `plane_stride` elements apart) = pl-th term of src[i] * col_scale[i % ncols];
// n % 4 == 0; col_scale may be NULL.
int launch_split_planes(const float* src, void* dst, size_t n, size_t plane_stride, int planes,
                        const float* col_scale, int ncols, cudaStream_t st);

// dst[0 | 1][r][c] (fp16, planes `plane_stride` elements apart) = leading / trailing half of
// src[r][c] * 2^k_r with the power of two chosen per row; inv_scale[r] = 2^-k_r.  cols % 4 == 0.
int launch_split_rows_f16(const float* src, void* dst, int rows, int cols, size_t plane_stride, float* inv_scale,
                          cudaStream_t st);

}  // namespace tc
}  // namespace b200gru
