// Dense and block-diagonal ("monarch") hidden weights: the serial part of the scan.
//
// Both kinds are `nb` independent GRUs of width Hb (dense: nb = 1, Hb = H) sharing
// gi / out.  Sequences are independent too, so the work splits into
// (hidden block n) x (batch tile of BT rows) problems with no traffic between
// them.  One thread-block CLUSTER of C CTAs owns one such problem for all T steps:
//
//   * CTA `rank` owns hidden units [rank*Hc, (rank+1)*Hc) of the block and keeps
//     its slice of the weights resident in shared memory for the whole launch
//     (forward: W[g, o in slice, all k], k-major;  backward: W[g, all o, k in slice]).
//     When the slice does not fit (large H) the same loops read it through L1/L2.
//   * every step the CTA needs the whole h_{t-1} (forward) or dgh_t (backward)
//     vector of the block: each CTA publishes its own slice into the shared memory
//     of all C peers (DSMEM stores), then one hardware cluster barrier ends the step.
//     The recurrence never round-trips through HBM or L2; `out[t]` / `dgi[t]` are
//     written once, for the caller.
//   * the contraction itself is FP32 FMA: a warp owns 32 output columns x a K slice,
//     partial sums meet in shared memory and are added in a fixed order (bitwise
//     reproducible run to run).  At batch tiles this narrow the step is latency
//     bound, not FLOP bound.
//
// Only the matrix-vector products that sit ON the dependence chain run here.  The
// gate recompute for the backward (one big GEMM over all t, since every h_t is
// known) and the weight-gradient GEMM live in block_gemm.cu.
//
// Step arithmetic follows src/gru_qat/triton_kernels/scan.py:1491-1550 and
// scan_monarch.py:74-127, 955-1053.

#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "block_scan.cuh"

namespace cg = cooperative_groups;

namespace b200gru {

namespace {

constexpr int NT = BLOCK_SCAN_THREADS;   // threads per CTA
constexpr int NW = NT / 32;

template <int BT> struct HVec { float v[BT]; };

template <int BT>
__device__ __forceinline__ void load_rows(const float* p, float (&v)[BT]) {
  if constexpr (BT == 1) {
    v[0] = p[0];
  } else if constexpr (BT == 2) {
    float2 x = *reinterpret_cast<const float2*>(p);
    v[0] = x.x; v[1] = x.y;
  } else {
#pragma unroll
    for (int q = 0; q < BT / 4; ++q) {
      float4 x = *reinterpret_cast<const float4*>(p + 4 * q);
      v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
    }
  }
}

// Publish `nfloats` contiguous floats (16-byte multiple) that this CTA just wrote at
// local shared address `src` to the same address in every peer CTA of the cluster.
__device__ __forceinline__ void publish_to_peers(cg::cluster_group& cluster, float* src, int nfloats,
                                                 int C, int rank) {
  const int nvec = nfloats >> 2;
  const float4* s4 = reinterpret_cast<const float4*>(src);
  for (int idx = threadIdx.x; idx < nvec * (C - 1); idx += NT) {
    const int p = idx / nvec;
    const int e = idx - p * nvec;
    const int peer = p + (p >= rank ? 1 : 0);
    float4* d4 = reinterpret_cast<float4*>(cluster.map_shared_rank(src, peer));
    d4[e] = s4[e];
  }
}

}  // namespace

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <int BT, int GPT>
__global__ void __launch_bounds__(NT, 1)
block_fwd_kernel(const BlockScanArgs a) {
  extern __shared__ __align__(16) float smem[];
  cg::cluster_group cluster = cg::this_cluster();

  const int C = a.C, Hb = a.Hb, Hc = a.Hc, Hcp = a.Hcp, H = a.H;
  const int rank = blockIdx.x % C;
  const int n = blockIdx.x / C;                       // hidden block
  const int b0 = blockIdx.y * BT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int u0 = rank * Hc;                           // first owned unit (inside the block)
  const int nown = max(0, min(Hc, Hb - u0));          // owned units
  const int HbP = a.HbP;                              // Hb rounded so that C*Hc*BT slices stay 16B aligned

  float* hbuf = smem;                                 // [2][HbP][BT]   fq_in(h), k-major
  float* red = hbuf + 2 * HbP * BT;                   // [KS][3][BT][Hcp]
  float* wsm = red + a.KS * 3 * BT * Hcp;             // [Hb][3*Hcp + 1]  (only if w_in_smem)

  // ---- weights: W(g, n, u0 + j, k)  ->  wsm[k][g*Hcp + j]
  const float* wbase;
  int kstride, gstride;
  if (a.w_in_smem) {
    kstride = 3 * Hcp + 1;
    gstride = Hcp;
    const float* Wn = a.W + (size_t)n * a.w_block_stride;
    const int total = 3 * Hcp * Hb;
    for (int idx = tid; idx < total; idx += NT) {
      const int k = idx % Hb;
      const int gj = idx / Hb;
      const int g = gj / Hcp, j = gj - g * Hcp;
      float v = 0.f;
      if (j < nown) v = Wn[(size_t)g * a.w_gate_stride + (size_t)(u0 + j) * Hb + k];
      wsm[k * kstride + g * Hcp + j] = v;
    }
    wbase = wsm;
  } else {
    // transposed global copy: Wt[((n*Hb + k)*3 + g)*Hb + u]
    kstride = 3 * Hb;
    gstride = Hb;
    wbase = a.Wt + (size_t)n * Hb * 3 * Hb + u0;
  }

  // ---- h_{-1}: every CTA loads the whole block row itself
  for (int idx = tid; idx < HbP * BT; idx += NT) {
    const int k = idx / BT, b = idx - k * BT;
    float v = 0.f;
    if (k < Hb && b0 + b < a.B) v = a.h0[(size_t)(b0 + b) * H + n * Hb + k];
    hbuf[idx] = a.qin.enabled ? fake_quant<true>(v, a.qin) : v;
    hbuf[HbP * BT + idx] = 0.f;
  }

  // gate-phase ownership: item q of this thread is (b, j) = divmod(tid + q*NT, Hcp)
  float hown[GPT], gr[GPT], gz[GPT], gn[GPT], bias_r[GPT], bias_z[GPT], bias_n[GPT];
  bool valid[GPT];
  int ib[GPT], ij[GPT];
#pragma unroll
  for (int q = 0; q < GPT; ++q) {
    const int idx = tid + q * NT;
    ib[q] = idx / Hcp;
    ij[q] = idx - ib[q] * Hcp;
    valid[q] = (idx < BT * Hcp) && (ij[q] < nown) && (b0 + ib[q] < a.B);
    hown[q] = 0.f; gr[q] = gz[q] = gn[q] = 0.f; bias_r[q] = bias_z[q] = bias_n[q] = 0.f;
    if (valid[q]) {
      const int u = n * Hb + u0 + ij[q];
      hown[q] = a.h0[(size_t)(b0 + ib[q]) * H + u];
      bias_r[q] = a.bh[u]; bias_z[q] = a.bh[H + u]; bias_n[q] = a.bh[2 * H + u];
      const float* g = a.gi + (size_t)(b0 + ib[q]) * 3 * H + u;
      gr[q] = __ldcs(g); gz[q] = __ldcs(g + H); gn[q] = __ldcs(g + 2 * H);
    }
  }
  if (C > 1) cluster.sync(); else __syncthreads();

  const int nct = Hcp / 32;
  const int nitems = nct * a.KS;
  const int Kper = (Hb + a.KS - 1) / a.KS;
  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;

  for (int t = 0; t < a.T; ++t) {
    const float* hcur = hbuf + (t & 1) * HbP * BT;
    float* hnxt = hbuf + ((t + 1) & 1) * HbP * BT;

    // ---- gh partial sums: warp = (column tile, K slice)
    for (int item = warp; item < nitems; item += NW) {
      const int ct = item % nct, ks = item / nct;
      const int j = ct * 32 + lane;
      const int jr = (j < nown) ? j : 0;
      const int k0 = ks * Kper, k1 = min(Hb, k0 + Kper);
      float acc[3][BT];
#pragma unroll
      for (int g = 0; g < 3; ++g)
#pragma unroll
        for (int b = 0; b < BT; ++b) acc[g][b] = 0.f;
      const float* wp = wbase + jr;
#pragma unroll 4
      for (int k = k0; k < k1; ++k) {
        const float w0 = wp[(size_t)k * kstride];
        const float w1 = wp[(size_t)k * kstride + gstride];
        const float w2 = wp[(size_t)k * kstride + 2 * gstride];
        float hv[BT];
        load_rows<BT>(hcur + k * BT, hv);
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          acc[0][b] = fmaf(w0, hv[b], acc[0][b]);
          acc[1][b] = fmaf(w1, hv[b], acc[1][b]);
          acc[2][b] = fmaf(w2, hv[b], acc[2][b]);
        }
      }
#pragma unroll
      for (int g = 0; g < 3; ++g)
#pragma unroll
        for (int b = 0; b < BT; ++b) red[((ks * 3 + g) * BT + b) * Hcp + j] = acc[g][b];
    }
    __syncthreads();

    // ---- gates for the owned (b, j) items; next step's gi goes in flight first
    float ngr[GPT], ngz[GPT], ngn[GPT];
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      ngr[q] = ngz[q] = ngn[q] = 0.f;
      if (valid[q] && t + 1 < a.T) {
        const float* g = a.gi + (size_t)(t + 1) * gi_step + (size_t)(b0 + ib[q]) * 3 * H + n * Hb + u0 + ij[q];
        ngr[q] = __ldcs(g); ngz[q] = __ldcs(g + H); ngn[q] = __ldcs(g + 2 * H);
      }
    }
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      const int idx = tid + q * NT;
      if (idx < BT * Hcp) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f;
        for (int ks = 0; ks < a.KS; ++ks) {
          s0 += red[((ks * 3 + 0) * BT + ib[q]) * Hcp + ij[q]];
          s1 += red[((ks * 3 + 1) * BT + ib[q]) * Hcp + ij[q]];
          s2 += red[((ks * 3 + 2) * BT + ib[q]) * Hcp + ij[q]];
        }
        float hq = 0.f;
        if (valid[q]) {
          const float ghn = s2 + bias_n[q];
          const GateOut g = gru_gates(gr[q], gz[q], gn[q], s0 + bias_r[q], s1 + bias_z[q], ghn, hown[q]);
          const float hnew = a.qout.enabled ? fake_quant<true>(g.h_raw, a.qout) : g.h_raw;
          hown[q] = hnew;
          const size_t o = (size_t)t * out_step + (size_t)(b0 + ib[q]) * H + n * Hb + u0 + ij[q];
          a.out[o] = hnew;
          if (a.save != nullptr) {
            const size_t comp = (size_t)a.T * out_step;
            __stcs(a.save + o, g.r);
            __stcs(a.save + comp + o, g.z);
            __stcs(a.save + 2 * comp + o, g.n);
            __stcs(a.save + 3 * comp + o, ghn);
          }
          hq = a.qin.enabled ? fake_quant<true>(hnew, a.qin) : hnew;
        }
        if (ij[q] < Hc) hnxt[(u0 + ij[q]) * BT + ib[q]] = hq;
      }
      gr[q] = ngr[q]; gz[q] = ngz[q]; gn[q] = ngn[q];
    }
    if (C > 1) {
      __syncthreads();
      publish_to_peers(cluster, hnxt + u0 * BT, Hc * BT, C, rank);
      cluster.sync();
    } else {
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------
// backward (serial part): dgi[t], dh chain, dh0.  Gate activations come from `S`.
// ---------------------------------------------------------------------------
template <int BT, int GPT>
__global__ void __launch_bounds__(NT, 1)
block_bwd_kernel(const BlockScanArgs a) {
  extern __shared__ __align__(16) float smem[];
  cg::cluster_group cluster = cg::this_cluster();

  const int C = a.C, Hb = a.Hb, Hc = a.Hc, Hcp = a.Hcp, H = a.H;
  const int rank = blockIdx.x % C;
  const int n = blockIdx.x / C;
  const int b0 = blockIdx.y * BT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int u0 = rank * Hc;
  const int nown = max(0, min(Hc, Hb - u0));
  const int HbP = a.HbP;
  const int K3 = 3 * HbP;                              // contraction length: (gate, unit)

  float* xbuf = smem;                                  // [2][3][HbP][BT]  dgh, k-major
  float* red = xbuf + 2 * K3 * BT;                     // [KS][BT][Hcp]
  float* wsm = red + a.KS * BT * Hcp;                  // [3][Hb][Hcp]

  // ---- weights: W(g, n, o, u0 + j) -> wsm[(g*Hb + o)*Hcp + j]
  const float* wbase;
  size_t gstride;      // between gates
  int ostride;         // between output units o
  if (a.w_in_smem) {
    gstride = (size_t)Hb * Hcp;
    ostride = Hcp;
    const float* Wn = a.W + (size_t)n * a.w_block_stride;
    const int total = 3 * Hb * Hcp;
    for (int idx = tid; idx < total; idx += NT) {
      const int j = idx % Hcp;
      const int go = idx / Hcp;
      const int g = go / Hb, o = go - g * Hb;
      float v = 0.f;
      if (j < nown) v = Wn[(size_t)g * a.w_gate_stride + (size_t)o * Hb + u0 + j];
      wsm[idx] = v;
    }
    wbase = wsm;
  } else {
    gstride = (size_t)a.w_gate_stride;
    ostride = Hb;
    wbase = a.W + (size_t)n * a.w_block_stride + u0;
  }
  for (int idx = tid; idx < 2 * K3 * BT; idx += NT) xbuf[idx] = 0.f;

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;

  float dh_acc[GPT];
  float c_do[GPT], c_r[GPT], c_z[GPT], c_n[GPT], c_ghn[GPT], c_hp[GPT];
  bool valid[GPT];
  int ib[GPT], ij[GPT];
  size_t off[GPT];                                     // (b, u) offset inside one [B,H] slab
#pragma unroll
  for (int q = 0; q < GPT; ++q) {
    const int idx = tid + q * NT;
    ib[q] = idx / Hcp;
    ij[q] = idx - ib[q] * Hcp;
    valid[q] = (idx < BT * Hcp) && (ij[q] < nown) && (b0 + ib[q] < a.B);
    off[q] = valid[q] ? (size_t)(b0 + ib[q]) * H + n * Hb + u0 + ij[q] : 0;
    dh_acc[q] = 0.f;
    c_do[q] = c_r[q] = c_z[q] = c_n[q] = c_ghn[q] = c_hp[q] = 0.f;
    if (valid[q]) {
      const int t = a.T - 1;
      const size_t o = (size_t)t * out_step + off[q];
      c_do[q] = __ldcs(a.dout + o);
      c_r[q] = __ldcs(a.S + o);
      c_z[q] = __ldcs(a.S + comp + o);
      c_n[q] = __ldcs(a.S + 2 * comp + o);
      c_ghn[q] = __ldcs(a.S + 3 * comp + o);
      c_hp[q] = (t > 0) ? a.out[o - out_step] : a.h0[off[q]];
    }
  }
  if (C > 1) cluster.sync(); else __syncthreads();

  const int nct = Hcp / 32;
  const int nitems = nct * a.KS;
  const int K = 3 * Hb;
  const int Kper = (K + a.KS - 1) / a.KS;

  for (int t = a.T - 1; t >= 0; --t) {
    const int par = (a.T - 1 - t) & 1;
    float* xcur = xbuf + par * K3 * BT;

    // ---- gate gradients for the owned items; publish dgh
    float dh_direct[GPT], mask_in[GPT];
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      const int idx = tid + q * NT;
      dh_direct[q] = 0.f; mask_in[q] = 1.f;
      if (idx < BT * Hcp) {
        float x0 = 0.f, x1 = 0.f, x2 = 0.f;
        if (valid[q]) {
          float dh = c_do[q] + dh_acc[q];
          if (a.qout.enabled) {
            const float h_raw = (1.0f - c_z[q]) * c_n[q] + c_z[q] * c_hp[q];
            dh = dh * ste_mask<true>(h_raw, a.qout);
          }
          const GateGrad gg = gru_gate_grads(dh, c_r[q], c_z[q], c_n[q], c_ghn[q], c_hp[q]);
          dh_direct[q] = gg.dh_direct;
          if (a.qin.enabled) mask_in[q] = ste_mask<true>(c_hp[q], a.qin);
          float* d = a.dgi + (size_t)t * gi_step + (size_t)(b0 + ib[q]) * 3 * H + n * Hb + u0 + ij[q];
          __stcs(d, gg.dgr); __stcs(d + H, gg.dgz); __stcs(d + 2 * H, gg.dgn);
          x0 = gg.dgr; x1 = gg.dgz; x2 = gg.dghn;
        }
        if (ij[q] < Hc) {
          const int k = u0 + ij[q];
          xcur[(0 * HbP + k) * BT + ib[q]] = x0;
          xcur[(1 * HbP + k) * BT + ib[q]] = x1;
          xcur[(2 * HbP + k) * BT + ib[q]] = x2;
        }
      }
    }
    // ---- operands of step t-1 go in flight now
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      if (valid[q] && t > 0) {
        const size_t o = (size_t)(t - 1) * out_step + off[q];
        c_do[q] = __ldcs(a.dout + o);
        c_r[q] = __ldcs(a.S + o);
        c_z[q] = __ldcs(a.S + comp + o);
        c_n[q] = __ldcs(a.S + 2 * comp + o);
        c_ghn[q] = __ldcs(a.S + 3 * comp + o);
        c_hp[q] = (t > 1) ? a.out[o - out_step] : a.h0[off[q]];
      }
    }
    if (C > 1) {
      __syncthreads();
#pragma unroll
      for (int g = 0; g < 3; ++g)
        publish_to_peers(cluster, xcur + (g * HbP + u0) * BT, Hc * BT, C, rank);
      cluster.sync();
    } else {
      __syncthreads();
    }

    // ---- dh_via[b, u0 + j] = sum_{g,o} dgh[b,g,o] * W(g, o, u0 + j)
    for (int item = warp; item < nitems; item += NW) {
      const int ct = item % nct, ks = item / nct;
      const int j = ct * 32 + lane;
      const int jr = (j < nown) ? j : 0;
      const int k0 = ks * Kper, k1 = min(K, k0 + Kper);
      float acc[BT];
#pragma unroll
      for (int b = 0; b < BT; ++b) acc[b] = 0.f;
      int g = k0 / Hb, o = k0 - g * Hb;
      const float* wp = wbase + jr;
      for (int kk = k0; kk < k1; ++kk) {
        const float w = wp[(size_t)g * gstride + (size_t)o * ostride];
        float xv[BT];
        load_rows<BT>(xcur + (g * HbP + o) * BT, xv);
#pragma unroll
        for (int b = 0; b < BT; ++b) acc[b] = fmaf(w, xv[b], acc[b]);
        if (++o == Hb) { o = 0; ++g; }
      }
#pragma unroll
      for (int b = 0; b < BT; ++b) red[(ks * BT + b) * Hcp + j] = acc[b];
    }
    __syncthreads();

#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      const int idx = tid + q * NT;
      if (idx < BT * Hcp && valid[q]) {
        float s = 0.f;
        for (int ks = 0; ks < a.KS; ++ks) s += red[(ks * BT + ib[q]) * Hcp + ij[q]];
        dh_acc[q] = dh_direct[q] + s * mask_in[q];
      }
    }
    // `red` is rewritten only after the next step's barrier, `xbuf` alternates: no extra sync.
  }

#pragma unroll
  for (int q = 0; q < GPT; ++q)
    if (valid[q]) a.dh0[off[q]] = dh_acc[q];
}

// ---------------------------------------------------------------------------
// host side: configuration and launch
// ---------------------------------------------------------------------------

using KernelFn = void (*)(const BlockScanArgs);

template <int BT>
static KernelFn pick_gpt(bool fwd, int gpt) {
  if (fwd) {
    if (gpt == 1) return block_fwd_kernel<BT, 1>;
    if (gpt == 2) return block_fwd_kernel<BT, 2>;
    return block_fwd_kernel<BT, 4>;
  }
  if (gpt == 1) return block_bwd_kernel<BT, 1>;
  if (gpt == 2) return block_bwd_kernel<BT, 2>;
  return block_bwd_kernel<BT, 4>;
}

static KernelFn pick_kernel(bool fwd, int bt, int gpt) {
  switch (bt) {
    case 1: return pick_gpt<1>(fwd, gpt);
    case 2: return pick_gpt<2>(fwd, gpt);
    case 4: return pick_gpt<4>(fwd, gpt);
    default: return pick_gpt<8>(fwd, gpt);
  }
}

static size_t smem_bytes(bool fwd, int BT, int Hb, int HbP, int Hcp, int KS, bool w_in_smem) {
  size_t f;
  if (fwd) {
    f = (size_t)2 * HbP * BT + (size_t)KS * 3 * BT * Hcp;
    if (w_in_smem) f += (size_t)Hb * (3 * Hcp + 1);
  } else {
    f = (size_t)2 * 3 * HbP * BT + (size_t)KS * BT * Hcp;
    if (w_in_smem) f += (size_t)3 * Hb * Hcp;
  }
  return f * sizeof(float);
}

struct DeviceInfo {
  int sms = 0;
  size_t smem_optin = 0;
  bool ok = false;
};

static DeviceInfo device_info() {
  static std::mutex mu;
  static std::map<int, DeviceInfo> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(dev);
  if (it != cache.end()) return it->second;
  DeviceInfo d;
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) d.sms = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess) d.smem_optin = (size_t)v;
  d.ok = d.sms > 0 && d.smem_optin > 0;
  cache[dev] = d;
  return d;
}

// Once per (device, kernel): allow the full opt-in shared memory and 16-CTA clusters.  The
// attributes are per function, so they are set to the maximum any configuration may need
// instead of per launch (a smaller later value would otherwise undo a larger earlier one).
static cudaError_t prepare_kernel(KernelFn fn) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, cudaError_t> done;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  auto key = std::make_pair(dev, (const void*)fn);
  auto it = done.find(key);
  if (it != done.end()) return it->second;
  const DeviceInfo di = device_info();
  cudaError_t e = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)di.smem_optin);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) cudaGetLastError();
  done[key] = e;
  return e;
}

// How many clusters of this shape the device can hold at once (0 = cannot launch).
static int max_active_clusters(KernelFn fn, int C, size_t smem) {
  static std::mutex mu;
  static std::map<std::tuple<int, const void*, int, size_t>, int> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  auto key = std::make_tuple(dev, (const void*)fn, C, smem);
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  int n = 0;
  cudaError_t e = prepare_kernel(fn);
  if (e == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(C, 1, 1);
    cfg.blockDim = dim3(NT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = C; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    e = cudaOccupancyMaxActiveClusters(&n, (const void*)fn, &cfg);
  }
  if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
  std::lock_guard<std::mutex> lk(mu);
  cache[key] = n;
  return n;
}

// Pick (C, BT, KS, GPT, weights-in-smem) minimising a simple cost model:
//   step = max(FMA issue, weight-slice streaming) + barrier;  total = waves * step.
bool choose_block_config(bool fwd, int B, int Hb, int nb, BlockScanConfig* out) {
  const DeviceInfo di = device_info();
  if (!di.ok) return false;
  double best = 1e300;
  bool found = false;
  const int bts[4] = {1, 2, 4, 8};
  const int cs[5] = {1, 2, 4, 8, 16};
  for (int ci = 0; ci < 5; ++ci) {
    const int C = cs[ci];
    if (C > 1 && Hb / C < 8) continue;                 // slices thinner than 8 units: not worth a barrier
    const int Hc = cdiv(Hb, C);
    const int Hcp = cdiv(Hc, 32) * 32;
    for (int bi = 0; bi < 4; ++bi) {
      const int BT = bts[bi];
      if (BT > 1 && BT / 2 >= B) continue;             // tile mostly empty
      if (C > 1 && (Hc * BT) % 4 != 0) continue;       // published slices move as float4
      const int HbP = C * Hc;                          // padded block width (>= Hb)
      if (BT * Hcp > 4 * NT) continue;
      const int gpt = (BT * Hcp <= NT) ? 1 : (BT * Hcp <= 2 * NT ? 2 : 4);
      const int nct = Hcp / 32;
      int KS = nct >= NW ? 1 : NW / nct;
      const int Kfull = fwd ? Hb : 3 * Hb;
      while (KS > 1 && Kfull / KS < 4) KS >>= 1;
      for (int ws = 1; ws >= 0; --ws) {
        const size_t smem = smem_bytes(fwd, BT, Hb, HbP, Hcp, KS, ws != 0);
        if (smem > di.smem_optin) continue;
        KernelFn fn = pick_kernel(fwd, BT, gpt);
        const int active = max_active_clusters(fn, C, smem);
        if (active <= 0) continue;
        const long long nclusters = (long long)nb * cdiv(B, BT);
        const double waves = (double)((nclusters + active - 1) / active);
        const double fma = 3.0 * Hcp * Hb * BT / 128.0;
        const double stream = 3.0 * Hcp * Hb * 4.0 / (ws ? 128.0 : 24.0);
        const double barrier = C > 1 ? 1400.0 + 40.0 * C : 250.0;
        const double cost = waves * ((fma > stream ? fma : stream) + barrier + 300.0);
        if (cost < best) {
          best = cost;
          found = true;
          out->C = C; out->BT = BT; out->Hc = Hc; out->Hcp = Hcp; out->HbP = HbP; out->KS = KS;
          out->GPT = gpt; out->w_in_smem = ws; out->smem = smem;
        }
        break;                                          // weights in smem fits: do not also try global
      }
    }
  }
  return found;
}

int launch_block_scan(bool fwd, const BlockScanConfig& c, BlockScanArgs args, int nb, cudaStream_t st) {
  args.C = c.C; args.Hc = c.Hc; args.Hcp = c.Hcp; args.HbP = c.HbP; args.KS = c.KS;
  args.w_in_smem = c.w_in_smem;
  KernelFn fn = pick_kernel(fwd, c.BT, c.GPT);
  const int active = max_active_clusters(fn, c.C, c.smem);                      // also sets the attributes
  static const bool debug = getenv("B200GRU_DEBUG") != nullptr;
  if (debug)
    fprintf(stderr, "[b200gru] %s T=%d B=%d H=%d nb=%d Hb=%d: C=%d BT=%d Hc=%d KS=%d GPT=%d w_in_smem=%d smem=%zu "
            "active_clusters=%d grid=(%d,%d)\n", fwd ? "block_fwd" : "block_bwd", args.T, args.B, args.H, nb, args.Hb,
            c.C, c.BT, c.Hc, c.KS, c.GPT, c.w_in_smem, c.smem, active, c.C * nb, cdiv(args.B, c.BT));
  if (active <= 0) return B200GRU_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(c.C * nb, cdiv(args.B, c.BT), 1);
  cfg.blockDim = dim3(NT, 1, 1);
  cfg.dynamicSmemBytes = c.smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = c.C; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, fn, args);
  note_launch();
  if (e != cudaSuccess) return check_launch(fwd ? "block_fwd_kernel" : "block_bwd_kernel");
  return check_launch(fwd ? "block_fwd_kernel" : "block_bwd_kernel");
}

}  // namespace b200gru
