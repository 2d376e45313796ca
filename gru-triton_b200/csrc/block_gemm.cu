// Off-chain (fully parallel) parts of the dense / block-diagonal scan.
//
// In the backward pass every h_t is already known, so two of the three matrix
// products do not sit on the serial dependence chain and run as ordinary tiled
// FP32 GEMMs over all T*B rows at once:
//
//   recompute_gates : gh = fq_in(h_{t-1}) @ W^T (+ bias) for every (t, b), fused with
//                     the gate nonlinearities -> S = {r, z, n, gh_n}
//                     (reference: in-kernel recompute, scan.py:389-432)
//   weight_grads    : dW = dgh^T @ fq_in(h_{t-1}) summed over all (t, b), dbh = sum dgh
//                     (reference: per-step load-add-store of a dWh partial, scan.py:573-616,
//                      then partial.sum(0), scan.py:750-751)
//
// FP32 FMA keeps the 1e-5 / 1e-4 parity budget; reductions are split over row
// ranges into partial buffers and summed in a fixed order (bitwise reproducible).

#include "block_scan.cuh"
#include "butterfly_scan.cuh"

namespace b200gru {

namespace {

// previous hidden state of flattened row tb = t*B + b, column c
__device__ __forceinline__ float h_prev_at(const float* __restrict__ h0, const float* __restrict__ out,
                                           int tb, int B, int H, int c) {
  return (tb < B) ? h0[(size_t)tb * H + c] : out[(size_t)(tb - B) * H + c];
}

}  // namespace

// ---------------------------------------------------------------------------
// W(g,n,o,k) -> Wt[((n*Hb + k)*3 + g)*WtR + o], zero for o in [Hb, WtR)
// ---------------------------------------------------------------------------
__global__ void transpose_weights_kernel(const float* __restrict__ W, float* __restrict__ Wt, int nb,
                                         int Hb, int WtR, long long gs, long long bs) {
  __shared__ float tile[32][33];
  const int gn = blockIdx.z;                 // g * nb + n
  const int g = gn / nb, n = gn - g * nb;
  const int o0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
  const float* src = W + (size_t)g * gs + (size_t)n * bs;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int o = o0 + r, k = k0 + threadIdx.x;
    tile[r][threadIdx.x] = (o < Hb && k < Hb) ? src[(size_t)o * Hb + k] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, o = o0 + threadIdx.x;
    if (k < Hb && o < WtR) Wt[(((size_t)n * Hb + k) * 3 + g) * WtR + o] = tile[threadIdx.x][r];
  }
}

int launch_transpose_weights(const float* W, float* Wt, int nb, int Hb, int WtR, long long gs, long long bs,
                             cudaStream_t st) {
  dim3 grid(cdiv(Hb, 32), cdiv(WtR, 32), 3 * nb), block(32, 8);
  transpose_weights_kernel<<<grid, block, 0, st>>>(W, Wt, nb, Hb, WtR, gs, bs);
  note_launch();
  return check_launch("transpose_weights_kernel");
}

// ---------------------------------------------------------------------------
// recompute_gates
// ---------------------------------------------------------------------------
constexpr int RG_ROWS = 64;    // rows (t,b) per CTA
constexpr int RG_KT = 32;      // k chunk

__global__ void __launch_bounds__(256)
recompute_gates_kernel(const BlockGemmArgs a) {
  __shared__ float As[RG_ROWS][RG_KT + 1];     // fq_in(h_prev)[row][k]
  __shared__ float Bs[RG_KT][96 + 1];          // W[k][g*32 + j]
  const int Hb = a.Hb, H = a.H, B = a.B;
  const int TB = a.T * B;
  const int ntile_u = cdiv(Hb, 32);
  const int n = blockIdx.x / ntile_u;
  const int ut = blockIdx.x - n * ntile_u;
  const int row0 = blockIdx.y * RG_ROWS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* Wn = a.W + (size_t)n * a.w_block_stride;

  float acc[3][8];
#pragma unroll
  for (int g = 0; g < 3; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;

  for (int k0 = 0; k0 < Hb; k0 += RG_KT) {
    for (int idx = tid; idx < RG_ROWS * RG_KT; idx += 256) {
      const int r = idx / RG_KT, k = idx - r * RG_KT;
      const int tb = row0 + r;
      float v = 0.f;
      if (tb < TB && k0 + k < Hb) {
        v = h_prev_at(a.h0, a.out, tb, B, H, n * Hb + k0 + k);
        if (a.qin.enabled) v = fake_quant<true>(v, a.qin);
      }
      As[r][k] = v;
    }
    for (int idx = tid; idx < 96 * RG_KT; idx += 256) {
      const int k = idx % RG_KT, gj = idx / RG_KT;
      const int g = gj / 32, j = gj - g * 32;
      const int o = ut * 32 + j;
      float v = 0.f;
      if (o < Hb && k0 + k < Hb) v = Wn[(size_t)g * a.w_gate_stride + (size_t)o * Hb + k0 + k];
      Bs[k][gj] = v;
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < RG_KT; ++k) {
      const float w0 = Bs[k][lane], w1 = Bs[k][32 + lane], w2 = Bs[k][64 + lane];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float h = As[warp * 8 + i][k];
        acc[0][i] = fmaf(w0, h, acc[0][i]);
        acc[1][i] = fmaf(w1, h, acc[1][i]);
        acc[2][i] = fmaf(w2, h, acc[2][i]);
      }
    }
    __syncthreads();
  }

  const int o = ut * 32 + lane;
  if (o >= Hb) return;
  const int u = n * Hb + o;
  const float br = a.bh[u], bz = a.bh[H + u], bn = a.bh[2 * H + u];
  const size_t comp = (size_t)TB * H;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int tb = row0 + warp * 8 + i;
    if (tb >= TB) continue;
    const float* g = a.gi + (size_t)tb * 3 * H + u;
    const float ghn = acc[2][i] + bn;
    const float r = sigmoidf_acc(g[0] + (acc[0][i] + br));
    const float z = sigmoidf_acc(g[H] + (acc[1][i] + bz));
    const float nn = tanhf(g[2 * H] + r * ghn);
    const size_t off = (size_t)tb * H + u;
    a.S[off] = r;
    a.S[comp + off] = z;
    a.S[2 * comp + off] = nn;
    a.S[3 * comp + off] = ghn;
  }
}

int launch_recompute_gates(const BlockGemmArgs& a, cudaStream_t st) {
  dim3 grid(cdiv(a.Hb, 32) * a.nb, cdiv(a.T * a.B, RG_ROWS));
  recompute_gates_kernel<<<grid, 256, 0, st>>>(a);
  note_launch();
  return check_launch("recompute_gates_kernel");
}

// ---------------------------------------------------------------------------
// weight_grads
// ---------------------------------------------------------------------------
constexpr int WG_O = 64;       // output units per CTA (x 3 gates)
constexpr int WG_K = 64;       // input units per CTA (two per lane)
constexpr int WG_R = 16;       // rows (t,b) per shared-memory chunk

// CTA tile: dW[g, 64 o, 64 k] for one row range.  Warp w owns 8 output units, lane l owns
// input units 2l, 2l+1: 48 accumulators per thread, 7 shared loads per 48 FMAs.  The next
// chunk's operands are fetched into registers (fake-quant / r-scaling applied) while the
// current chunk is consumed from shared memory.
__global__ void __launch_bounds__(256)
weight_grads_kernel(const BlockGemmArgs a, float* __restrict__ dst, int rows_per_split) {
  __shared__ __align__(16) float Ds[WG_R][3 * WG_O];     // dgh[row][g*64 + o]
  __shared__ __align__(16) float Hs[WG_R][WG_K];         // fq_in(h_prev)[row][k]
  const int Hb = a.Hb, H = a.H, B = a.B;
  const int TB = a.T * B;
  const int nkt = cdiv(Hb, WG_K), not_ = cdiv(Hb, WG_O);
  int bx = blockIdx.x;
  const int kt = bx % nkt; bx /= nkt;
  const int ot = bx % not_;
  const int n = bx / not_;
  const int split = blockIdx.y;
  const int r_begin = split * rows_per_split;
  const int r_end = min(TB, r_begin + rows_per_split);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  constexpr int ND = WG_R * 3 * WG_O / 256;               // 12 dgh values per thread per chunk
  constexpr int NH_ = WG_R * WG_K / 256;                  // 4 h values per thread per chunk
  float dreg[ND], hreg[NH_];

  auto fetch = [&](int r0) {
#pragma unroll
    for (int m = 0; m < ND; ++m) {
      const int idx = tid + m * 256;
      const int r = idx / (3 * WG_O), go = idx - r * (3 * WG_O);
      const int g = go / WG_O, o = go - g * WG_O;
      const int tb = r0 + r, uo = ot * WG_O + o;
      float v = 0.f;
      if (tb < r_end && uo < Hb) {
        const int u = n * Hb + uo;
        v = __ldg(a.dgi + (size_t)tb * 3 * H + (size_t)g * H + u);
        if (g == 2) v = v * __ldg(a.S + (size_t)tb * H + u);         // dgh_n = dgi_n * r
      }
      dreg[m] = v;
    }
#pragma unroll
    for (int m = 0; m < NH_; ++m) {
      const int idx = tid + m * 256;
      const int r = idx / WG_K, k = idx - r * WG_K;
      const int tb = r0 + r, uk = kt * WG_K + k;
      float v = 0.f;
      if (tb < r_end && uk < Hb) {
        v = h_prev_at(a.h0, a.out, tb, B, H, n * Hb + uk);
        if (a.qin.enabled) v = fake_quant<true>(v, a.qin);
      }
      hreg[m] = v;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int m = 0; m < ND; ++m) (&Ds[0][0])[tid + m * 256] = dreg[m];
#pragma unroll
    for (int m = 0; m < NH_; ++m) (&Hs[0][0])[tid + m * 256] = hreg[m];
  };

  float2 acc[3][2][4];                                  // [gate][k of the pair][unit pair]: packed FP32 FMA
#pragma unroll
  for (int g = 0; g < 3; ++g)
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[g][kk][i] = make_float2(0.f, 0.f);

  fetch(r_begin);
  for (int r0 = r_begin; r0 < r_end; r0 += WG_R) {
    stash();
    __syncthreads();
    if (r0 + WG_R < r_end) fetch(r0 + WG_R);
#pragma unroll 4
    for (int r = 0; r < WG_R; ++r) {
      const float2 h = *reinterpret_cast<const float2*>(&Hs[r][2 * lane]);
      const float2 h0 = make_float2(h.x, h.x), h1 = make_float2(h.y, h.y);
#pragma unroll
      for (int g = 0; g < 3; ++g) {
        const float4 d0 = *reinterpret_cast<const float4*>(&Ds[r][g * WG_O + warp * 8]);
        const float4 d1 = *reinterpret_cast<const float4*>(&Ds[r][g * WG_O + warp * 8 + 4]);
        const float2 d[4] = {make_float2(d0.x, d0.y), make_float2(d0.z, d0.w), make_float2(d1.x, d1.y),
                             make_float2(d1.z, d1.w)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[g][0][i] = __ffma2_rn(d[i], h0, acc[g][0][i]);
          acc[g][1][i] = __ffma2_rn(d[i], h1, acc[g][1][i]);
        }
      }
    }
    __syncthreads();
  }

  const int k = kt * WG_K + 2 * lane;
  if (k >= Hb) return;
  const size_t dw_elems = (size_t)3 * a.nb * Hb * Hb;      // dense: 3*H*H as well
  float* base = dst + (size_t)split * dw_elems + (size_t)n * a.w_block_stride;
#pragma unroll
  for (int g = 0; g < 3; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int o = ot * WG_O + warp * 8 + i;
      if (o < Hb) {
        float* p = base + (size_t)g * a.w_gate_stride + (size_t)o * Hb + k;
        const float2 v0 = acc[g][0][i >> 1], v1 = acc[g][1][i >> 1];
        p[0] = (i & 1) ? v0.y : v0.x;
        if (k + 1 < Hb) p[1] = (i & 1) ? v1.y : v1.x;
      }
    }
}

// dbh: column sums of dgh over a range of rows; partial[split][3H]
__global__ void __launch_bounds__(256)
bias_grads_kernel(const float* __restrict__ dgi, const float* __restrict__ S, float* __restrict__ dst,
                  int TB, int H, int rows_per_split) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;                  // in [0, 3H)
  const int r_begin = blockIdx.y * rows_per_split;
  const int r_end = min(TB, r_begin + rows_per_split);
  float s = 0.f;
  if (col < 3 * H) {
    const bool is_n = col >= 2 * H;
    for (int tb = r_begin + warp; tb < r_end; tb += 8) {
      float v = dgi[(size_t)tb * 3 * H + col];
      if (is_n) v = v * S[(size_t)tb * H + (col - 2 * H)];
      s += v;
    }
  }
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && col < 3 * H) {
    float t = red[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += red[w][lane];
    dst[(size_t)blockIdx.y * 3 * H + col] = t;
  }
}

static void wg_splits(int T, int B, int nb, int Hb, int* nsplit, int* rows_per_split) {
  const int TB = T * B;
  const long long tiles = (long long)nb * cdiv(Hb, WG_O) * cdiv(Hb, WG_K);
  long long s = (2 * 148 + tiles - 1) / tiles;
  const long long max_by_rows = (TB + 8 * WG_R - 1) / (8 * WG_R);
  if (s > max_by_rows) s = max_by_rows;
  if (s > 32) s = 32;
  if (s < 1) s = 1;
  int rps = cdiv(cdiv(TB, (int)s), WG_R) * WG_R;
  *nsplit = cdiv(TB, rps);
  *rows_per_split = rps;
}

static void bg_splits(int T, int B, int* nsplit, int* rows_per_split) {
  const int TB = T * B;
  int s = cdiv(TB, 256);
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  const int rps = cdiv(TB, s);
  *nsplit = cdiv(TB, rps);
  *rows_per_split = rps;
}

size_t bias_grads_scratch_bytes(int T, int B, int H) {
  int nsb, rpsb;
  bg_splits(T, B, &nsb, &rpsb);
  return align_up((size_t)nsb * 3 * H * sizeof(float), 256);
}

int launch_bias_grads(const float* dgi, const float* S, float* partial, float* dbh, int T, int B, int H,
                      cudaStream_t st) {
  int nsb, rpsb;
  bg_splits(T, B, &nsb, &rpsb);
  dim3 gridb(cdiv(3 * H, 32), nsb);
  bias_grads_kernel<<<gridb, 256, 0, st>>>(dgi, S, partial, T * B, H, rpsb);
  note_launch();
  int rc = check_launch("bias_grads_kernel");
  if (rc) return rc;
  launch_reduce_partials(partial, nsb, (size_t)3 * H, (size_t)3 * H, dbh, st);
  return check_launch("reduce_partials");
}

size_t weight_grads_scratch_bytes(int T, int B, int H, int nb, int Hb) {
  int ns, rps, nsb, rpsb;
  wg_splits(T, B, nb, Hb, &ns, &rps);
  bg_splits(T, B, &nsb, &rpsb);
  size_t f = 0;
  if (ns > 1) f += (size_t)ns * 3 * nb * Hb * Hb;
  f += (size_t)nsb * 3 * H;
  return align_up(f * sizeof(float), 256);
}

int launch_weight_grads(const BlockGemmArgs& a, cudaStream_t st) {
  int ns, rps, nsb, rpsb;
  wg_splits(a.T, a.B, a.nb, a.Hb, &ns, &rps);
  bg_splits(a.T, a.B, &nsb, &rpsb);
  const size_t dw_elems = (size_t)3 * a.nb * a.Hb * a.Hb;
  float* part_w = a.partial;
  float* part_b = a.partial + (ns > 1 ? (size_t)ns * dw_elems : 0);

  dim3 grid(cdiv(a.Hb, WG_K) * cdiv(a.Hb, WG_O) * a.nb, ns);
  weight_grads_kernel<<<grid, 256, 0, st>>>(a, ns > 1 ? part_w : a.dW, rps);
  note_launch();
  int rc = check_launch("weight_grads_kernel");
  if (rc) return rc;
  if (ns > 1) launch_reduce_partials(part_w, ns, dw_elems, dw_elems, a.dW, st);

  return launch_bias_grads(a.dgi, a.S, part_b, a.dbh, a.T, a.B, a.H, st);
}

}  // namespace b200gru
