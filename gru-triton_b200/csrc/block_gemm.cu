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
// weight gradients: for each block n, C[m][k] = sum_tb A[tb][m] * Bm[tb][k] with
//   m = g*Hb + o  (3*Hb rows),  A[tb][m] = dgh[tb][g][n*Hb + o],  Bm[tb][k] = fq_in(h_prev)[tb][n*Hb + k].
// Both operands are contiguous along the output dimensions, so this is an outer-product SGEMM:
// CTA tile (16*TM) x (16*TN), 16 x 16 threads, each thread TM x TN accumulators held as packed
// FP32 pairs; per tb a thread reads TM/4 + TN/4 float4 from shared memory for TM*TN/2 packed FMAs.
// The next 16 rows are fetched into registers (r-scaling of the n gate and the input fake-quant
// applied on the way) while the current 16 are consumed; one barrier per 16 rows.
// Rows are split over blockIdx.y into partial buffers that a second kernel sums in a fixed order.
// ---------------------------------------------------------------------------
constexpr int WG_BK = 16;      // rows (t,b) per shared-memory stage

template <int TM, int TN, bool VEC>
__global__ void __launch_bounds__(256, 2)
weight_grads_kernel(const BlockGemmArgs a, float* __restrict__ dst, int rows_per_split, int ntm, int ntn) {
  constexpr int BM = 16 * TM, BN = 16 * TN;
  constexpr int NA = TM / 4, NB = TN / 4;                 // float4 groups per thread per stage
  __shared__ __align__(16) float As[2][WG_BK][BM];
  __shared__ __align__(16) float Bs[2][WG_BK][BN];
  const int Hb = a.Hb, H = a.H, B = a.B;
  const int TB = a.T * B;
  const int M = 3 * Hb;
  int bx = blockIdx.x;
  const int nt = bx % ntn; bx /= ntn;
  const int mt = bx % ntm;
  const int n = bx / ntm;
  const int m0 = mt * BM, k0 = nt * BN;
  const int r_begin = blockIdx.y * rows_per_split;
  const int r_end = min(TB, r_begin + rows_per_split);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  float4 areg[NA], breg[NB];

  auto fetch = [&](int r0) {
#pragma unroll
    for (int j = 0; j < NA; ++j) {
      const int idx = tid + j * 256;
      const int r = idx / (BM / 4), c = (idx - r * (BM / 4)) * 4;
      const int tb = r0 + r, m = m0 + c;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tb < r_end) {
        if (VEC) {
          if (m < M) {                                   // Hb % 4 == 0: the four share gate and validity
            const int g = m / Hb, u = n * Hb + (m - g * Hb);
            v = __ldg(reinterpret_cast<const float4*>(a.dgi + (size_t)tb * 3 * H + (size_t)g * H + u));
            if (g == 2) {                                // dgh_n = dgi_n * r
              const float4 rr = __ldg(reinterpret_cast<const float4*>(a.S + (size_t)tb * H + u));
              v.x = v.x * rr.x; v.y = v.y * rr.y; v.z = v.z * rr.z; v.w = v.w * rr.w;
            }
          }
        } else {
          float e[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            e[q] = 0.f;
            const int mq = m + q;
            if (mq < M) {
              const int g = mq / Hb, u = n * Hb + (mq - g * Hb);
              e[q] = __ldg(a.dgi + (size_t)tb * 3 * H + (size_t)g * H + u);
              if (g == 2) e[q] = e[q] * __ldg(a.S + (size_t)tb * H + u);
            }
          }
          v = make_float4(e[0], e[1], e[2], e[3]);
        }
      }
      areg[j] = v;
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int idx = tid + j * 256;
      const int r = idx / (BN / 4), c = (idx - r * (BN / 4)) * 4;
      const int tb = r0 + r, k = k0 + c;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tb < r_end) {
        const float* hp = (tb < B) ? a.h0 + (size_t)tb * H : a.out + (size_t)(tb - B) * H;   // h_{t-1}
        hp += n * Hb;
        if (VEC) {
          if (k < Hb) v = __ldg(reinterpret_cast<const float4*>(hp + k));
        } else {
          if (k < Hb) v.x = __ldg(hp + k);
          if (k + 1 < Hb) v.y = __ldg(hp + k + 1);
          if (k + 2 < Hb) v.z = __ldg(hp + k + 2);
          if (k + 3 < Hb) v.w = __ldg(hp + k + 3);
        }
        // h_t (t >= 0) is already on the output grid: when both quantisers are the same grid,
        // fq_in leaves it unchanged, so only rows taken from h0 need the rounding
        if (a.qin.enabled && !(a.out_on_qin_grid && tb >= B)) {
          v.x = fake_quant<true>(v.x, a.qin); v.y = fake_quant<true>(v.y, a.qin);
          v.z = fake_quant<true>(v.z, a.qin); v.w = fake_quant<true>(v.w, a.qin);
        }
      }
      breg[j] = v;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int j = 0; j < NA; ++j) reinterpret_cast<float4*>(&As[buf][0][0])[tid + j * 256] = areg[j];
#pragma unroll
    for (int j = 0; j < NB; ++j) reinterpret_cast<float4*>(&Bs[buf][0][0])[tid + j * 256] = breg[j];
  };

  float2 acc[TM][TN / 2];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN / 2; ++j) acc[i][j] = make_float2(0.f, 0.f);

  fetch(r_begin);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int r0 = r_begin; r0 < r_end; r0 += WG_BK) {
    const bool more = r0 + WG_BK < r_end;
    if (more) fetch(r0 + WG_BK);
#pragma unroll 4
    for (int kk = 0; kk < WG_BK; ++kk) {
      float av[TM], bv[TN];
#pragma unroll
      for (int j = 0; j < NA; ++j) {
        const float4 t = *reinterpret_cast<const float4*>(&As[buf][kk][j * 64 + ty * 4]);
        av[4 * j] = t.x; av[4 * j + 1] = t.y; av[4 * j + 2] = t.z; av[4 * j + 3] = t.w;
      }
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const float4 t = *reinterpret_cast<const float4*>(&Bs[buf][kk][j * 64 + tx * 4]);
        bv[4 * j] = t.x; bv[4 * j + 1] = t.y; bv[4 * j + 2] = t.z; bv[4 * j + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const float2 aa = make_float2(av[i], av[i]);
#pragma unroll
        for (int j = 0; j < TN / 2; ++j)
          acc[i][j] = __ffma2_rn(aa, make_float2(bv[2 * j], bv[2 * j + 1]), acc[i][j]);
      }
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }

  float* base = dst + (size_t)blockIdx.y * ((size_t)3 * a.nb * Hb * Hb) + (size_t)n * a.w_block_stride;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (m >= M) continue;
    const int g = m / Hb, o = m - g * Hb;
    float* row = base + (size_t)g * a.w_gate_stride + (size_t)o * Hb;
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int k = k0 + j * 64 + tx * 4;
      const float2 v0 = acc[i][2 * j], v1 = acc[i][2 * j + 1];
      if (VEC) {
        if (k < Hb) *reinterpret_cast<float4*>(row + k) = make_float4(v0.x, v0.y, v1.x, v1.y);
      } else {
        if (k < Hb) row[k] = v0.x;
        if (k + 1 < Hb) row[k + 1] = v0.y;
        if (k + 2 < Hb) row[k + 2] = v1.x;
        if (k + 3 < Hb) row[k + 3] = v1.y;
      }
    }
  }
}

// dbh: column sums of dgh over a range of rows; partial[split][3H]
__global__ void __launch_bounds__(256)
bias_grads_kernel(const float* __restrict__ dgi, const float* __restrict__ S, float* __restrict__ dst,
                  int TB, int H, int rows_per_split) {
  __shared__ float red[8][32];
  pdl_launch_dependents();
  pdl_wait();
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

// Tile shape and row split of the weight-gradient GEMM: big tiles when a block is at least 128
// wide, and enough row ranges for about two CTAs per SM.
struct WgPlan { int tm, tn, ntm, ntn, nsplit, rows_per_split; };

static WgPlan wg_plan(int T, int B, int nb, int Hb) {
  WgPlan p;
  const int TB = T * B;
  p.tm = (3 * Hb >= 128) ? 8 : 4;
  p.tn = (Hb >= 128) ? 8 : 4;
  p.ntm = cdiv(3 * Hb, 16 * p.tm);
  p.ntn = cdiv(Hb, 16 * p.tn);
  const long long tiles = (long long)nb * p.ntm * p.ntn;
  // two CTAs fit an SM: pick the split count whose CTA total fills whole waves of 2 * 148 best
  // (ties go to fewer splits: less partial traffic)
  const long long slots = 2 * 148;
  long long max_s = cdiv(TB, 8 * WG_BK);
  if (max_s > 32) max_s = 32;
  if (max_s < 1) max_s = 1;
  long long s = 1;
  double best = 0.0;
  for (long long c = 1; c <= max_s; ++c) {
    const long long ctas = tiles * c;
    const double eff = (double)ctas / (double)(((ctas + slots - 1) / slots) * slots);
    if (eff > best + 0.03) { best = eff; s = c; }
  }
  const int rps = cdiv(cdiv(TB, (int)s), WG_BK) * WG_BK;
  p.nsplit = cdiv(TB, rps);
  p.rows_per_split = rps;
  return p;
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
  launch_pdl(bias_grads_kernel, gridb, dim3(256), 0, st, dgi, S, partial, T * B, H, rpsb);
  note_launch();
  int rc = check_launch("bias_grads_kernel");
  if (rc) return rc;
  launch_reduce_partials(partial, nsb, (size_t)3 * H, (size_t)3 * H, dbh, st);
  return check_launch("reduce_partials");
}

size_t weight_grads_scratch_bytes(int T, int B, int H, int nb, int Hb) {
  int nsb, rpsb;
  const int ns = wg_plan(T, B, nb, Hb).nsplit;
  bg_splits(T, B, &nsb, &rpsb);
  size_t f = 0;
  if (ns > 1) f += (size_t)ns * 3 * nb * Hb * Hb;
  f += (size_t)nsb * 3 * H;
  return align_up(f * sizeof(float), 256);
}

int launch_weight_grads(const BlockGemmArgs& a, cudaStream_t st) {
  int nsb, rpsb;
  const WgPlan p = wg_plan(a.T, a.B, a.nb, a.Hb);
  const int ns = p.nsplit;
  bg_splits(a.T, a.B, &nsb, &rpsb);
  const size_t dw_elems = (size_t)3 * a.nb * a.Hb * a.Hb;
  float* part_w = a.partial;
  float* part_b = a.partial + (ns > 1 ? (size_t)ns * dw_elems : 0);
  float* dst = ns > 1 ? part_w : a.dW;

  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  const bool vec = a.Hb % 4 == 0 && a.H % 4 == 0 && a.w_gate_stride % 4 == 0 && a.w_block_stride % 4 == 0 &&
                   al16(a.dgi) && al16(a.S) && al16(a.h0) && al16(a.out) && al16(dst);
  dim3 grid(p.ntm * p.ntn * a.nb, ns);
#define B200GRU_WG(TM_, TN_)                                                                              \
  do {                                                                                                    \
    if (vec) weight_grads_kernel<TM_, TN_, true><<<grid, 256, 0, st>>>(a, dst, p.rows_per_split, p.ntm, p.ntn);  \
    else weight_grads_kernel<TM_, TN_, false><<<grid, 256, 0, st>>>(a, dst, p.rows_per_split, p.ntm, p.ntn);     \
  } while (0)
  if (p.tm == 8 && p.tn == 8) B200GRU_WG(8, 8);
  else if (p.tm == 8) B200GRU_WG(8, 4);
  else B200GRU_WG(4, 4);
#undef B200GRU_WG
  note_launch();
  int rc = check_launch("weight_grads_kernel");
  if (rc) return rc;
  if (ns > 1) launch_reduce_partials(part_w, ns, dw_elems, dw_elems, a.dW, st);

  return launch_bias_grads(a.dgi, a.S, part_b, a.dbh, a.T, a.B, a.H, st);
}

}  // namespace b200gru
