// Interfaces between the butterfly scan kernels and the C ABI.
#pragma once

#include "common.cuh"

namespace b200gru {

constexpr int BFLY_THREADS = 256;
constexpr int BFLY_MAX_PASSES = 48;

// A run of consecutive stages [l0, l0 + nst) whose strides touch only bits [lb, lb + r).
// pb[s] = (log-stride of stage l0 + s) - lb, the stage's bit inside the pass.
struct BflyPass {
  short l0, nst, lb, r;
  short pb[4];
};

struct BflyArgs {
  const float* gi;
  const float* h0;        // rows [0, h0_rows)
  const float* h0_tail;   // rows [h0_rows, B): previous hidden states taken from `out` (gate recompute)
  const float* tw;        // [3][nstages][Hpad/2][2][2]
  const float* twp;       // staged kernels: the same twiddles in pass order (bfly2_permute_twiddles), or NULL
  const float* bh;
  float* out;             // may be NULL (gate recompute)
  float* save;            // [4][T][B][H] or NULL
  const float* S;         // backward: activations
  const float* dout;
  const float* out_c;     // backward: forward output
  const float* dgi_c;     // twiddle gradients: dgi as input
  float* dgi;
  float* dh0;
  int T, B, H, Hpad, logn, nstages;
  int h0_rows;
  int npasses;
  int tw_in_smem;
  int tw_mode;            // staged kernels: 0 twiddles read from global, 1 resident in smem, 2 streamed per pass
  int RSZ;                // staged kernels: swizzled row stride of the running vectors
  BflyPass passes[BFLY_MAX_PASSES];
  Quant qin, qout;
};

int build_bfly_passes(int logn, int nblocks, BflyPass* passes, int max_passes);
int bfly_launch_forward(BflyArgs a, cudaStream_t st);
// butterfly_scan2.cu: staged variants; return -1 when they do not apply to the problem
int bfly2_permute_twiddles(const BflyArgs& a, float* twp, cudaStream_t st);
int bfly2_launch_forward(BflyArgs a, int want_bt, cudaStream_t st);
int bfly2_launch_backward(BflyArgs a, int want_bt, cudaStream_t st);
size_t bfly2_wgrad_scratch_bytes(int T, int B, int H, int Hpad, int nstages);   // 0: does not apply
int bfly2_launch_wgrad(BflyArgs a, float* partial, float* dtw, cudaStream_t st);
int bfly_read_status(int reset);
int bfly_launch_backward(BflyArgs a, cudaStream_t st);
size_t bfly_wgrad_scratch_bytes(int T, int B, int H, int Hpad, int nstages);
int bfly_launch_wgrad(BflyArgs a, float* partial, float* dtw, cudaStream_t st);

// block_gemm.cu: bias gradient (shared by dense, block-diagonal and butterfly)
size_t bias_grads_scratch_bytes(int T, int B, int H);
int launch_bias_grads(const float* dgi, const float* S, float* partial, float* dbh, int T, int B, int H,
                      cudaStream_t st);

}  // namespace b200gru
