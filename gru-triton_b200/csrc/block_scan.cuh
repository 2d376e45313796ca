// Interfaces between the dense / block-diagonal scan kernels and the C ABI.
#pragma once

#include "common.cuh"

namespace b200gru {

constexpr int BLOCK_SCAN_THREADS = 256;

// Arguments of the serial scan kernels.  W(g, n, o, k) = W[g*w_gate_stride + n*w_block_stride + o*Hb + k]
// covers both layouts: dense Wh_cat[3H,H] (nb = 1, gate stride H*H) and block-diagonal
// Wh_struct[3,nb,Hb,Hb] (gate stride nb*Hb*Hb, block stride Hb*Hb).
struct BlockScanArgs {
  const float* gi;
  const float* h0;
  const float* W;
  const float* Wt;     // forward only: W transposed to [nb][Hb(k)][3][WtR(o), zero padded], used when a slice misses smem
  const float* bh;
  float* out;          // forward: written; backward: read (const in effect)
  float* save;         // forward: optional [4][T][B][H] (r, z, n, gh_n)
  const float* S;      // backward: the same four activations
  const float* dout;
  float* dgi;
  float* dh0;
  int* status;         // device word set to 1 if a bounded wait inside a kernel gave up
  int T, B, H;
  int nb, Hb;
  long long w_gate_stride, w_block_stride;
  // launch configuration (filled by launch_block_scan)
  int C, Hc, Hc4, HbP, Hb4, RS, NH, WtR, w_in_smem;
  Quant qin, qout;
};

// C: cluster size; BT: batch rows per cluster; Hc: units per CTA (Hc4: rounded to 4);
// HbP = C*Hc >= Hb (Hb4: rounded to 4); RS: forward weight row stride in shared memory;
// IPW: forward 4-unit items per warp; TW/NH/GPT: backward vector width, contraction halves,
// owned elements per thread.
struct BlockScanConfig {
  int C, BT, Hc, Hc4, HbP, Hb4, RS, IPW, TW, NH, GPT, w_in_smem;
  size_t smem;
};

// Row length of the transposed weight copy for a block of width Hb (upper bound over all
// cluster sizes; the forward reads 4 units at a time and may run past the last owned unit).
inline int transposed_row_bound(int Hb) { return Hb + 72; }     // C * round_up(ceil(Hb / C), 4) + 4 + 4, C <= 16

bool choose_block_config(bool fwd, int B, int Hb, int nb, BlockScanConfig* out);
int launch_block_scan(bool fwd, const BlockScanConfig& c, BlockScanArgs args, int nb, cudaStream_t st);

// block_gemm.cu -- the parallel (off-chain) parts of the dense / block-diagonal backward.
//   transpose_weights : W(g,n,o,k) -> Wt[n][k][g][o]
//   recompute_gates   : S = {r, z, n, gh_n}[T,B,H] from (gi, h0, out, W, bh) for every t at once
//   weight_grads      : dW(g,n,o,k) = sum_{t,b} dgh[t,b,g,n*Hb+o] * fq_in(h_{t-1})[b,n*Hb+k]
//                       dbh[g*H+u]  = sum_{t,b} dgh[t,b,g,u]
//     with dgh_r = dgi_r, dgh_z = dgi_z, dgh_n = dgi_n * r.
struct BlockGemmArgs {
  const float* gi;
  const float* h0;
  const float* out;
  const float* W;
  const float* bh;
  const float* dgi;
  float* S;            // recompute_gates: written; weight_grads: read
  float* dW;
  float* dbh;
  float* partial;      // scratch for split reductions
  int T, B, H, nb, Hb;
  long long w_gate_stride, w_block_stride;
  Quant qin;
  int out_on_qin_grid;   // weight_grads: `out` was produced by an output quantiser identical to qin
};

int launch_transpose_weights(const float* W, float* Wt, int nb, int Hb, int WtR, long long w_gate_stride,
                             long long w_block_stride, cudaStream_t st);
int launch_recompute_gates(const BlockGemmArgs& a, cudaStream_t st);
size_t weight_grads_scratch_bytes(int T, int B, int H, int nb, int Hb);
int launch_weight_grads(const BlockGemmArgs& a, cudaStream_t st);

}  // namespace b200gru
