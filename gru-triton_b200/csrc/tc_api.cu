// C ABI of the tensor-core GEMM core: argument translation only.

#include <cstring>

#include "tc_gemm.cuh"

using namespace b200gru;

namespace {

bool to_internal(const b200gru_gemm_args* a, tc::TcGemm* g) {
  if (a == nullptr) return false;
  if (a->npairs < 1 || a->npairs > tc::TC_MAX_PAIRS) return false;
  memset(g, 0, sizeof(*g));
  if (a->dtype < 0 || a->dtype > 2) return false;
  g->kind = a->dtype == 1 ? tc::TC_KIND_I8 : (a->dtype == 2 ? tc::TC_KIND_F16 : tc::TC_KIND_BF16);
  g->M = a->M; g->N = a->N; g->K = a->K;
  g->A = a->A; g->B = a->B;
  g->a_planes = a->a_planes; g->b_planes = a->b_planes;
  g->a_mn = a->a_mn_major ? 1 : 0; g->b_mn = a->b_mn_major ? 1 : 0;
  g->lda = a->lda; g->ldb = a->ldb;
  g->a_plane_stride = a->a_plane_stride; g->b_plane_stride = a->b_plane_stride;
  g->npairs = a->npairs;
  for (int q = 0; q < a->npairs; ++q) { g->pa[q] = a->pair_a[q]; g->pb[q] = a->pair_b[q]; }
  g->split_k = a->split_k < 1 ? 1 : a->split_k;
  g->tile_n = a->tile_n;
  g->chunk_kb = a->chunk_kblocks;
  g->accumulate = a->accumulate;
  g->alpha = a->alpha; g->row_scale = a->row_scale; g->col_scale = a->col_scale; g->bias = a->bias;
  g->C = a->C; g->ldc = a->ldc; g->split_stride = a->split_stride;
  return true;
}

}  // namespace

extern "C" {

int b200gru_tc_gemm(const b200gru_gemm_args* args, void* stream) {
  tc::TcGemm g;
  if (!to_internal(args, &g)) return B200GRU_INVALID_ARGUMENT;
  return tc::launch_tc_gemm(g, static_cast<cudaStream_t>(stream));
}

int b200gru_tc_gemm_splits(const b200gru_gemm_args* args, int wanted) {
  tc::TcGemm g;
  if (!to_internal(args, &g) || g.K <= 0) return 0;
  return tc::tc_gemm_splits(g, wanted);
}

int b200gru_split_bf16(const float* src, void* dst, size_t n, size_t plane_stride, int planes,
                       const float* col_scale, int ncols, void* stream) {
  return tc::launch_split_planes(src, dst, n, plane_stride, planes, col_scale, ncols,
                                 static_cast<cudaStream_t>(stream));
}

int b200gru_split_f16(const float* src, void* dst, int rows, int cols, size_t plane_stride, float* inv_scale,
                      void* stream) {
  return tc::launch_split_rows_f16(src, dst, rows, cols, plane_stride, inv_scale, static_cast<cudaStream_t>(stream));
}

int b200gru_test_wait_timeout(void* stream) {
  return tc::launch_wait_timeout_probe(static_cast<cudaStream_t>(stream));
}

}  // extern "C"
