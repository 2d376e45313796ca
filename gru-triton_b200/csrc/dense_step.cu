// Dense scan at GEMM-sized batch: one launch per time step.
//
// The cluster kernels of block_scan.cu keep a CTA's weight slice in shared memory and pay a
// fixed latency per step; once the slice no longer fits (H = 1024: 786 KB per CTA of a 16-CTA
// cluster) they stream weights through L1/L2 every step.  With a large batch the step itself is
// a compute-bound product, so here every step is one tiled FP32 SGEMM with the gate math fused
// into its epilogue; the stream order between launches is the recurrence.
//
//   forward  step t : gh[b, (g,u)] = sum_k hq_{t-1}[b,k] * W[(g,u),k]   -> gates -> out[t], save,
//                     and fq_in(h_t) written TRANSPOSED ([H][Bp]) as the next step's A operand
//   backward step t : via[b,k] = sum_(g,u) dgh_t[b,(g,u)] * W[(g,u),k]  -> dh_{t-1} -> gate grads
//                     of step t-1 -> dgi[t-1], and dgh_{t-1} written transposed ([3H][Bp])
//
// Both products are outer-product SGEMMs (operands contiguous along the output dimensions, 16 x 16
// threads, packed FP32 FMA accumulators, operands staged through registers into a double-buffered
// shared-memory tile).  Sums run over k in ascending order inside one thread: deterministic.
// Reference: the same recurrence as scan.py:389-432 (forward) and scan.py:450-616 (backward),
// where a spin barrier across batch tiles plays the role of the launch boundary.

#include <cooperative_groups.h>

#include "block_scan.cuh"

namespace cg = cooperative_groups;

namespace b200gru {

namespace {

constexpr int DS_BK = 16;

struct StepArgs {
  const float* gi;
  const float* h0;
  const float* W;        // backward: Wh_cat [3H][H]
  const float* Wt;       // forward: transposed copy [k][g][WtR]
  const float* bh;
  float* out;            // forward: written; backward: read
  float* save;           // forward, optional
  const float* S;        // backward
  const float* dout;
  float* dgi;
  float* dh0;
  const float* opT_in;   // forward: fq_in(h_{t-1})^T [H][Bp]; backward: dgh_t^T [3H][Bp]
  float* opT_out;
  float* direct;         // backward: dh * z of the current step, [B][H]
  int t, T, B, Bp, H, WtR;
  Quant qin, qout;
};

__device__ __forceinline__ float4 ld4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// fq_in(h0)^T with zero padding of the batch to Bp: the A operand of forward step 0
__global__ void __launch_bounds__(256)
step_h0_transpose_kernel(const float* __restrict__ h0, float* __restrict__ hqT, int B, int Bp, int H, Quant qin) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.x * 32, b0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int b = b0 + r, k = k0 + tx;
    float v = 0.f;
    if (b < B && k < H) {
      v = h0[(size_t)b * H + k];
      if (qin.enabled) v = fake_quant<true>(v, qin);
    }
    tile[r][tx] = v;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int k = k0 + r, b = b0 + tx;
    if (k < H && b < Bp) hqT[(size_t)k * Bp + b] = tile[tx][r];
  }
}

// ---------------------------------------------------------------------------
// forward step: CTA tile = (16*TM rows) x (32 units x 3 gates)
// ---------------------------------------------------------------------------
template <int TM>
__global__ void __launch_bounds__(256, 2)
dense_step_fwd_kernel(const StepArgs a) {
  constexpr int BM = 16 * TM, BN = 96;
  constexpr int NA = TM / 4;
  __shared__ __align__(16) float As[2][DS_BK][BM];
  __shared__ __align__(16) float Bs[2][DS_BK][BN];
  const int H = a.H, B = a.B, Bp = a.Bp;
  const int m0 = blockIdx.x * BM, u0 = blockIdx.y * 32;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  float4 areg[NA], breg[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int j = 0; j < NA; ++j) {
      const int idx = tid + j * 256;
      const int r = idx / (BM / 4), c = (idx - r * (BM / 4)) * 4;
      const int m = m0 + c;
      areg[j] = (m < Bp) ? ld4(a.opT_in + (size_t)(k0 + r) * Bp + m) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int idx = tid + j * 256;
      breg[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (idx < DS_BK * 24) {
        const int r = idx / 24, q = idx - r * 24;
        const int g = q >> 3, j4 = (q & 7) * 4;
        breg[j] = ld4(a.Wt + (size_t)(k0 + r) * 3 * a.WtR + (size_t)g * a.WtR + u0 + j4);
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int j = 0; j < NA; ++j) reinterpret_cast<float4*>(&As[buf][0][0])[tid + j * 256] = areg[j];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int idx = tid + j * 256;
      if (idx < DS_BK * 24) reinterpret_cast<float4*>(&Bs[buf][0][0])[idx] = breg[j];
    }
  };

  float2 acc[TM][3];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int g = 0; g < 3; ++g) acc[i][g] = make_float2(0.f, 0.f);

  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < H; k0 += DS_BK) {
    const bool more = k0 + DS_BK < H;
    if (more) fetch(k0 + DS_BK);
#pragma unroll 4
    for (int kk = 0; kk < DS_BK; ++kk) {
      float av[TM];
#pragma unroll
      for (int j = 0; j < NA; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][j * 64 + ty * 4]);
        av[4 * j] = v.x; av[4 * j + 1] = v.y; av[4 * j + 2] = v.z; av[4 * j + 3] = v.w;
      }
      float2 bv[3];
#pragma unroll
      for (int g = 0; g < 3; ++g) bv[g] = *reinterpret_cast<const float2*>(&Bs[buf][kk][g * 32 + 2 * tx]);
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const float2 aa = make_float2(av[i], av[i]);
#pragma unroll
        for (int g = 0; g < 3; ++g) acc[i][g] = __ffma2_rn(aa, bv[g], acc[i][g]);
      }
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }

  // ---- gates for (row, unit pair) and the transposed operand of the next step
  const int u = u0 + 2 * tx;
  const float2 br = *reinterpret_cast<const float2*>(a.bh + u);
  const float2 bz = *reinterpret_cast<const float2*>(a.bh + H + u);
  const float2 bn = *reinterpret_cast<const float2*>(a.bh + 2 * H + u);
  const size_t out_step = (size_t)B * H, comp = (size_t)a.T * out_step;
#pragma unroll
  for (int j = 0; j < NA; ++j) {
    const int mb = m0 + j * 64 + ty * 4;
    float hq0[4], hq1[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int b = mb + i;
      hq0[i] = 0.f; hq1[i] = 0.f;
      if (b < B) {
        const float* g = a.gi + ((size_t)a.t * B + b) * 3 * H + u;
        const float2 gr = __ldcs(reinterpret_cast<const float2*>(g));
        const float2 gz = __ldcs(reinterpret_cast<const float2*>(g + H));
        const float2 gn = __ldcs(reinterpret_cast<const float2*>(g + 2 * H));
        const float* hp = (a.t == 0) ? a.h0 + (size_t)b * H + u : a.out + (size_t)(a.t - 1) * out_step + (size_t)b * H + u;
        const float2 hv = *reinterpret_cast<const float2*>(hp);
        const float2 sr = acc[4 * j + i][0], sz = acc[4 * j + i][1], sn = acc[4 * j + i][2];
        const float ghn0 = sn.x + bn.x, ghn1 = sn.y + bn.y;
        const GateOut g0 = gru_gates(gr.x, gz.x, gn.x, sr.x + br.x, sz.x + bz.x, ghn0, hv.x);
        const GateOut g1 = gru_gates(gr.y, gz.y, gn.y, sr.y + br.y, sz.y + bz.y, ghn1, hv.y);
        const float h0n = a.qout.enabled ? fake_quant<true>(g0.h_raw, a.qout) : g0.h_raw;
        const float h1n = a.qout.enabled ? fake_quant<true>(g1.h_raw, a.qout) : g1.h_raw;
        const size_t o = (size_t)a.t * out_step + (size_t)b * H + u;
        *reinterpret_cast<float2*>(a.out + o) = make_float2(h0n, h1n);
        if (a.save != nullptr) {
          __stcs(reinterpret_cast<float2*>(a.save + o), make_float2(g0.r, g1.r));
          __stcs(reinterpret_cast<float2*>(a.save + comp + o), make_float2(g0.z, g1.z));
          __stcs(reinterpret_cast<float2*>(a.save + 2 * comp + o), make_float2(g0.n, g1.n));
          __stcs(reinterpret_cast<float2*>(a.save + 3 * comp + o), make_float2(ghn0, ghn1));
        }
        hq0[i] = a.qin.enabled ? fake_quant<true>(h0n, a.qin) : h0n;
        hq1[i] = a.qin.enabled ? fake_quant<true>(h1n, a.qin) : h1n;
      }
    }
    if (mb < Bp && a.t + 1 < a.T) {
      *reinterpret_cast<float4*>(a.opT_out + (size_t)u * Bp + mb) = make_float4(hq0[0], hq0[1], hq0[2], hq0[3]);
      *reinterpret_cast<float4*>(a.opT_out + (size_t)(u + 1) * Bp + mb) = make_float4(hq1[0], hq1[1], hq1[2], hq1[3]);
    }
  }
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------

// Gate gradients of step tt for row b, units u..u+3, given dh = dout[tt] + carry.  Writes dgi[tt],
// the direct term dh*z and, transposed, dgh (dgh_n = dgi_n * r) for the next product.
__device__ __forceinline__ void bwd_emit(const StepArgs& a, int tt, int b, int u, const float (&carry)[4],
                                         float (&dgr)[4], float (&dgz)[4], float (&dghn)[4]) {
  const int H = a.H, B = a.B;
  const size_t out_step = (size_t)B * H, comp = (size_t)a.T * out_step;
  const size_t o = (size_t)tt * out_step + (size_t)b * H + u;
  const float4 d4 = __ldcs(reinterpret_cast<const float4*>(a.dout + o));
  const float4 r4 = __ldcs(reinterpret_cast<const float4*>(a.S + o));
  const float4 z4 = __ldcs(reinterpret_cast<const float4*>(a.S + comp + o));
  const float4 n4 = __ldcs(reinterpret_cast<const float4*>(a.S + 2 * comp + o));
  const float4 g4 = __ldcs(reinterpret_cast<const float4*>(a.S + 3 * comp + o));
  const float4 h4 = *reinterpret_cast<const float4*>(tt > 0 ? a.out + o - out_step : a.h0 + (size_t)b * H + u);
  const float dv[4] = {d4.x, d4.y, d4.z, d4.w}, rv[4] = {r4.x, r4.y, r4.z, r4.w}, zv[4] = {z4.x, z4.y, z4.z, z4.w};
  const float nv[4] = {n4.x, n4.y, n4.z, n4.w}, gv[4] = {g4.x, g4.y, g4.z, g4.w}, hv[4] = {h4.x, h4.y, h4.z, h4.w};
  float dgn[4], dir[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float dh = dv[c] + carry[c];
    if (a.qout.enabled) {
      const float h_raw = (1.0f - zv[c]) * nv[c] + zv[c] * hv[c];
      dh = dh * ste_mask<true>(h_raw, a.qout);
    }
    const GateGrad gg = gru_gate_grads(dh, rv[c], zv[c], nv[c], gv[c], hv[c]);
    dgr[c] = gg.dgr; dgz[c] = gg.dgz; dgn[c] = gg.dgn; dghn[c] = gg.dghn; dir[c] = gg.dh_direct;
  }
  float* d = a.dgi + ((size_t)tt * B + b) * 3 * H + u;
  __stcs(reinterpret_cast<float4*>(d), make_float4(dgr[0], dgr[1], dgr[2], dgr[3]));
  __stcs(reinterpret_cast<float4*>(d + H), make_float4(dgz[0], dgz[1], dgz[2], dgz[3]));
  __stcs(reinterpret_cast<float4*>(d + 2 * H), make_float4(dgn[0], dgn[1], dgn[2], dgn[3]));
  *reinterpret_cast<float4*>(a.direct + (size_t)b * H + u) = make_float4(dir[0], dir[1], dir[2], dir[3]);
}

// last time step: dh = dout[T-1]; one thread per (4 rows, 4 units)
__global__ void __launch_bounds__(256)
dense_step_bwd_first_kernel(const StepArgs a) {
  const int H4 = a.H >> 2, Bp4 = a.Bp >> 2;
  const int idx = blockIdx.x * 256 + threadIdx.x;
  if (idx >= H4 * Bp4) return;
  const int bq = idx % Bp4, uq = idx / Bp4;                // consecutive threads -> consecutive rows
  const int b0 = bq * 4, u = uq * 4;
  float tr[3][4][4];                                       // [gate][unit][row]
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float dgr[4] = {0.f, 0.f, 0.f, 0.f}, dgz[4] = {0.f, 0.f, 0.f, 0.f}, dghn[4] = {0.f, 0.f, 0.f, 0.f};
    if (b0 + i < a.B) {
      const float carry[4] = {0.f, 0.f, 0.f, 0.f};
      bwd_emit(a, a.T - 1, b0 + i, u, carry, dgr, dgz, dghn);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) { tr[0][c][i] = dgr[c]; tr[1][c][i] = dgz[c]; tr[2][c][i] = dghn[c]; }
  }
#pragma unroll
  for (int g = 0; g < 3; ++g)
#pragma unroll
    for (int c = 0; c < 4; ++c)
      *reinterpret_cast<float4*>(a.opT_out + ((size_t)g * a.H + u + c) * a.Bp + b0) =
          make_float4(tr[g][c][0], tr[g][c][1], tr[g][c][2], tr[g][c][3]);
}

// backward step t: CTA tile = (16*TM rows) x (16*TN positions k).
// KSPLIT = 2 (64 x 64 tiles only): the two CTAs of a cluster (blockIdx.z) each take half of the
// contraction range; CTA 1 then writes its accumulators into CTA 0's operand buffers (DSMEM stores
// between two cluster barriers), CTA 0 adds them and runs the epilogue.  This doubles the number of
// CTAs when the batch shard is too small to give every SM two tiles.
template <int TM, int TN, int KSPLIT>
__global__ void __launch_bounds__(256, 2)
dense_step_bwd_kernel(const StepArgs a) {
  constexpr int BM = 16 * TM, BN = 16 * TN;
  constexpr int NA = TM / 4, NB = TN / 4;
  static_assert(KSPLIT == 1 || TM * TN * 256 <= 2 * DS_BK * (BM + BN), "accumulators must fit the operand buffers");
  __shared__ __align__(16) float tiles[2 * DS_BK * (BM + BN)];
  float (*As)[DS_BK][BM] = reinterpret_cast<float (*)[DS_BK][BM]>(tiles);
  float (*Bs)[DS_BK][BN] = reinterpret_cast<float (*)[DS_BK][BN]>(tiles + 2 * DS_BK * BM);
  const int H = a.H, B = a.B, Bp = a.Bp;
  const int Kall = 3 * a.H;
  const int kbeg = (KSPLIT == 1) ? 0 : (int)blockIdx.z * (Kall / KSPLIT);
  const int K = (KSPLIT == 1) ? Kall : kbeg + Kall / KSPLIT;      // end of this CTA's range
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  float4 areg[NA], breg[NB];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int j = 0; j < NA; ++j) {
      const int idx = tid + j * 256;
      const int r = idx / (BM / 4), c = (idx - r * (BM / 4)) * 4;
      const int m = m0 + c;
      areg[j] = (m < Bp) ? ld4(a.opT_in + (size_t)(k0 + r) * Bp + m) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int idx = tid + j * 256;
      const int r = idx / (BN / 4), c = (idx - r * (BN / 4)) * 4;
      const int n = n0 + c;
      breg[j] = (n < H) ? ld4(a.W + (size_t)(k0 + r) * H + n) : make_float4(0.f, 0.f, 0.f, 0.f);
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

  fetch(kbeg);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = kbeg; k0 < K; k0 += DS_BK) {
    const bool more = k0 + DS_BK < K;
    if (more) fetch(k0 + DS_BK);
#pragma unroll 4
    for (int kk = 0; kk < DS_BK; ++kk) {
      float av[TM], bv[TN];
#pragma unroll
      for (int j = 0; j < NA; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][j * 64 + ty * 4]);
        av[4 * j] = v.x; av[4 * j + 1] = v.y; av[4 * j + 2] = v.z; av[4 * j + 3] = v.w;
      }
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][j * 64 + tx * 4]);
        bv[4 * j] = v.x; bv[4 * j + 1] = v.y; bv[4 * j + 2] = v.z; bv[4 * j + 3] = v.w;
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

  if (KSPLIT == 2) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();                                        // both CTAs are done with their operand buffers
    float4* mine = reinterpret_cast<float4*>(tiles) + tid * (TM * TN / 4);
    if (blockIdx.z == 1) {
      float4* dst = cluster.map_shared_rank(mine, 0);
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN / 4; ++j)
          dst[i * (TN / 4) + j] = make_float4(acc[i][2 * j].x, acc[i][2 * j].y, acc[i][2 * j + 1].x, acc[i][2 * j + 1].y);
    }
    cluster.sync();                                        // the partial sums have landed in CTA 0
    if (blockIdx.z == 1) return;
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN / 4; ++j) {
        const float4 v = mine[i * (TN / 4) + j];
        acc[i][2 * j].x += v.x; acc[i][2 * j].y += v.y; acc[i][2 * j + 1].x += v.z; acc[i][2 * j + 1].y += v.w;
      }
  }

  // ---- dh_{t-1} = direct_t + mask_in(h_{t-1}) * via, then the gate gradients of step t-1
  const int t = a.t;
  const size_t out_step = (size_t)B * H;
#pragma unroll
  for (int jn = 0; jn < NB; ++jn) {
    const int u = n0 + jn * 64 + tx * 4;
    if (u >= H) continue;
#pragma unroll
    for (int jm = 0; jm < NA; ++jm) {
      const int mb = m0 + jm * 64 + ty * 4;
      float tr[3][4][4];                                   // [gate][unit][row]
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int b = mb + i;
        float dgr[4] = {0.f, 0.f, 0.f, 0.f}, dgz[4] = {0.f, 0.f, 0.f, 0.f}, dghn[4] = {0.f, 0.f, 0.f, 0.f};
        if (b < B) {
          const float2 s01 = acc[4 * jm + i][2 * jn], s23 = acc[4 * jm + i][2 * jn + 1];
          const float sv[4] = {s01.x, s01.y, s23.x, s23.y};
          const float4 dir4 = *reinterpret_cast<const float4*>(a.direct + (size_t)b * H + u);
          const float dirv[4] = {dir4.x, dir4.y, dir4.z, dir4.w};
          const float4 hp4 = *reinterpret_cast<const float4*>(
              t > 0 ? a.out + (size_t)(t - 1) * out_step + (size_t)b * H + u : a.h0 + (size_t)b * H + u);
          const float hpv[4] = {hp4.x, hp4.y, hp4.z, hp4.w};
          float carry[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float mk = a.qin.enabled ? ste_mask<true>(hpv[c], a.qin) : 1.0f;
            carry[c] = dirv[c] + sv[c] * mk;
          }
          if (t == 0) {
            *reinterpret_cast<float4*>(a.dh0 + (size_t)b * H + u) = make_float4(carry[0], carry[1], carry[2], carry[3]);
          } else {
            bwd_emit(a, t - 1, b, u, carry, dgr, dgz, dghn);
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) { tr[0][c][i] = dgr[c]; tr[1][c][i] = dgz[c]; tr[2][c][i] = dghn[c]; }
      }
      if (t > 0 && mb < Bp) {
#pragma unroll
        for (int g = 0; g < 3; ++g)
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<float4*>(a.opT_out + ((size_t)g * H + u + c) * Bp + mb) =
                make_float4(tr[g][c][0], tr[g][c][1], tr[g][c][2], tr[g][c][3]);
      }
    }
  }
}

inline int padded_batch(int B) { return (B + 3) & ~3; }

}  // namespace

// The per-step path serves dense problems whose weight slice misses the shared memory of a
// 16-CTA cluster, at a batch large enough to fill the GPU with tiles (measured break-even against
// the streaming cluster kernel at H = 1024: about 128 rows).  Shape-only, so that the workspace
// query and the launch agree.
bool dense_step_path(int B, int H) {
  const size_t slice = (size_t)3 * ((H + 15) / 16) * H * sizeof(float);
  return slice > (size_t)200 * 1024 && B >= 128 && H % 32 == 0;
}

size_t dense_step_fwd_scratch_bytes(int B, int H) {
  return align_up((size_t)2 * H * padded_batch(B) * sizeof(float), 256);
}

size_t dense_step_bwd_scratch_bytes(int B, int H) {
  return align_up(((size_t)2 * 3 * H * padded_batch(B) + (size_t)B * H) * sizeof(float), 256);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Wt: transposed weight copy [k][g][WtR]; scratch: dense_step_fwd_scratch_bytes
int launch_dense_step_forward(const float* gi, const float* h0, const float* Wt, int WtR, const float* bh, float* out,
                              float* save, float* scratch, int T, int B, int H, Quant qin, Quant qout,
                              cudaStream_t st) {
  if (!aligned16(gi) || !aligned16(h0) || !aligned16(bh) || !aligned16(out) || !aligned16(save) ||
      !aligned16(Wt) || !aligned16(scratch))
    return B200GRU_INVALID_ARGUMENT;
  StepArgs a;
  memset(&a, 0, sizeof(a));
  a.gi = gi; a.h0 = h0; a.Wt = Wt; a.bh = bh; a.out = out; a.save = save;
  a.T = T; a.B = B; a.Bp = padded_batch(B); a.H = H; a.WtR = WtR; a.qin = qin; a.qout = qout;
  float* opT[2] = {scratch, scratch + (size_t)H * a.Bp};

  dim3 tg(cdiv(H, 32), cdiv(a.Bp, 32));
  step_h0_transpose_kernel<<<tg, 256, 0, st>>>(h0, opT[0], B, a.Bp, H, qin);
  note_launch();
  int rc = check_launch("step_h0_transpose_kernel");
  if (rc) return rc;

  // 128-row tiles as soon as they cover most SMs (measured at B = 512, H = 1024: 89 us per step
  // against 105 us with twice as many 64-row tiles)
  const bool big = (long long)cdiv(B, 128) * (H / 32) >= 120;
  for (int t = 0; t < T; ++t) {
    a.t = t; a.opT_in = opT[t & 1]; a.opT_out = opT[(t + 1) & 1];
    if (big) dense_step_fwd_kernel<8><<<dim3(cdiv(B, 128), H / 32), 256, 0, st>>>(a);
    else dense_step_fwd_kernel<4><<<dim3(cdiv(B, 64), H / 32), 256, 0, st>>>(a);
    note_launch();
  }
  return check_launch("dense_step_fwd_kernel");
}

// scratch: dense_step_bwd_scratch_bytes
int launch_dense_step_backward(const float* h0, const float* W, const float* out, const float* S, const float* dout,
                               float* dgi, float* dh0, float* scratch, int T, int B, int H, Quant qin, Quant qout,
                               cudaStream_t st) {
  if (!aligned16(h0) || !aligned16(W) || !aligned16(out) || !aligned16(S) || !aligned16(dout) || !aligned16(dgi) ||
      !aligned16(dh0) || !aligned16(scratch))
    return B200GRU_INVALID_ARGUMENT;
  StepArgs a;
  memset(&a, 0, sizeof(a));
  a.h0 = h0; a.W = W; a.out = const_cast<float*>(out); a.S = S; a.dout = dout; a.dgi = dgi; a.dh0 = dh0;
  a.T = T; a.B = B; a.Bp = padded_batch(B); a.H = H; a.qin = qin; a.qout = qout;
  float* opT[2] = {scratch, scratch + (size_t)3 * H * a.Bp};
  a.direct = scratch + (size_t)2 * 3 * H * a.Bp;

  a.t = T - 1; a.opT_out = opT[0];
  const int n = (H / 4) * (a.Bp / 4);
  dense_step_bwd_first_kernel<<<cdiv(n, 256), 256, 0, st>>>(a);
  note_launch();
  int rc = check_launch("dense_step_bwd_first_kernel");
  if (rc) return rc;

  const long long t128 = (long long)cdiv(B, 128) * cdiv(H, 128);
  const long long t8464 = (long long)cdiv(B, 128) * cdiv(H, 64);
  const long long t6464 = (long long)cdiv(B, 64) * cdiv(H, 64);
  int flip = 0;
  for (int t = T - 1; t >= 0; --t) {
    a.t = t; a.opT_in = opT[flip]; a.opT_out = opT[flip ^ 1];
    if (t128 >= 120) dense_step_bwd_kernel<8, 8, 1><<<dim3(cdiv(B, 128), cdiv(H, 128)), 256, 0, st>>>(a);
    else if (t8464 >= 120) dense_step_bwd_kernel<8, 4, 1><<<dim3(cdiv(B, 128), cdiv(H, 64)), 256, 0, st>>>(a);
    else if (t6464 >= 2 * 148) dense_step_bwd_kernel<4, 4, 1><<<dim3(cdiv(B, 64), cdiv(H, 64)), 256, 0, st>>>(a);
    else {
      // too few tiles for two CTAs per SM: pairs of CTAs split the contraction
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(cdiv(B, 64), cdiv(H, 64), 2);
      cfg.blockDim = dim3(256, 1, 1);
      cfg.dynamicSmemBytes = 0;
      cfg.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 2;
      cfg.attrs = at; cfg.numAttrs = 1;
      cudaLaunchKernelEx(&cfg, dense_step_bwd_kernel<4, 4, 2>, a);
    }
    note_launch();
    flip ^= 1;
  }
  return check_launch("dense_step_bwd_kernel");
}

}  // namespace b200gru
