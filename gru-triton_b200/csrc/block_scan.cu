// Dense and block-diagonal ("monarch") hidden weights: the serial part of the scan.
//
// Both kinds are `nb` independent GRUs of width Hb (dense: nb = 1, Hb = H) sharing
// gi / out.  Sequences are independent too, so the work splits into
// (hidden block n) x (batch tile of BT rows) problems with no traffic between
// them.  One thread-block CLUSTER of C CTAs owns one such problem for all T steps.
// CTA `rank` owns hidden units [rank*Hc, (rank+1)*Hc) of the block and keeps the rows
// W(g, own unit, all k) of the weights resident in shared memory for the whole launch
// (when that slice exceeds shared memory the same loops read a copy through L1/L2).
// The recurrence never round-trips through HBM or L2; `out[t]` / `dgi[t]` are written
// once, for the caller.  All arithmetic is FP32 FMA; every cross-thread sum has a fixed
// order (bitwise reproducible run to run).
//
// Forward step ("all-gather"):
//   a warp owns 4 output units x 3 gates; its lanes split the contraction index k, each
//   lane reading one float4 of weights per gate and the BT hidden values of its k; a
//   halving shuffle reduction leaves lane (b, unit) with the three gate sums of its
//   element, which then does the gate math in place and publishes fq_in(h_t) into the shared
//   memory of all C peers with st.async, which also counts the bytes on the consumer's mbarrier;
//   a consumer starts step t+1 when the bytes of step t have arrived.  No cluster barrier inside
//   the time loop (two per launch: start and end).
//
// Backward step ("reduce-scatter"), only dh_via = dgh . W is on the dependence chain:
//   gate gradients of the owned elements -> local partial products against the SAME
//   weight rows, for all Hb input positions -> each CTA sends the part that belongs to
//   peer r into r's receive buffer (st.async + the receiver's mbarrier) -> the owner waits for
//   the bytes and adds the C partials in rank order.
//
// The gate recompute for the backward (one big GEMM over all t, since every h_t is
// known) and the weight-gradient GEMM are off the chain and live in block_gemm.cu.
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

// Set to 1 by a kernel whose bounded mbarrier wait gave up (a peer CTA never delivered).
__device__ int g_scan_status;

namespace {

#ifndef B200GRU_FWD_NR
#define B200GRU_FWD_NR 6
#endif
constexpr int NT = BLOCK_SCAN_THREADS;   // threads per CTA
constexpr int NW = NT / 32;

__host__ __device__ constexpr int next_pow2(int x) { return x <= 1 ? 1 : (x <= 2 ? 2 : (x <= 4 ? 4 : 8)); }

// BT consecutive floats (the batch rows of one k) from shared memory.
template <int BT>
__device__ __forceinline__ void load_rows(const float* p, float (&v)[BT]) {
  if constexpr (BT % 4 == 0) {
#pragma unroll
    for (int q = 0; q < BT / 4; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(p + 4 * q);
      v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
    }
  } else if constexpr (BT % 2 == 0) {
#pragma unroll
    for (int q = 0; q < BT / 2; ++q) {
      const float2 x = *reinterpret_cast<const float2*>(p + 2 * q);
      v[2 * q] = x.x; v[2 * q + 1] = x.y;
    }
  } else {
#pragma unroll
    for (int q = 0; q < BT; ++q) v[q] = p[q];
  }
}

// The first BT floats of a 16-byte aligned row, in as few and as narrow loads as cover them
// (5 rows: one float4 and one scalar).  Every lane reads the same row, and a broadcast load still
// returns its full width to each lane, so loading the padding would cost return bandwidth.
template <int BT, int BTX>
__device__ __forceinline__ void load_rows_exact(const float* p, float (&v)[BTX]) {
  int at = 0;
  if constexpr (BT >= 4) {
#pragma unroll
    for (int q = 0; q < BT / 4; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(p + 4 * q);
      v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
    }
    at = (BT / 4) * 4;
  }
  if constexpr (BT % 4 >= 2) {
    const float2 x = *reinterpret_cast<const float2*>(p + at);
    v[at] = x.x; v[at + 1] = x.y;
    at += 2;
  }
  if constexpr (BT % 2 == 1) v[at] = p[at];
}

// Sum `vals` over the 32 lanes of the warp.  While more than one value is left, each
// step hands half of them to the partner lane (lane ^ off), so the whole reduction costs
// about N shuffles instead of 5N.  On return vals[0] holds the total of element
// `reduced_index<N>(lane)`; lanes that end up with the same element hold the same total.
template <int N>
__device__ __forceinline__ void warp_reduce_scatter(float (&vals)[N], int lane) {
  int n = N;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    if (n > 1) {
      const int half = n >> 1;
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        if (i < half) {
          const float send = upper ? vals[i] : vals[i + half];
          const float keep = upper ? vals[i + half] : vals[i];
          vals[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
      }
      n = half;
    } else {
      vals[0] += __shfl_xor_sync(0xffffffffu, vals[0], off);
    }
  }
}

template <int N>
__device__ __forceinline__ int reduced_index(int lane) {
  // N = 32 -> lane, 16 -> lane >> 1, 8 -> lane >> 2, 4 -> lane >> 3
  return N >= 32 ? lane : (N == 16 ? lane >> 1 : (N == 8 ? lane >> 2 : lane >> 3));
}
template <int N>
__device__ __forceinline__ bool reduced_owner(int lane) {
  // one lane per element: the lowest of the group that shares it
  return N >= 32 ? true : ((lane & ((32 / N) - 1)) == 0);
}

// ---- asynchronous DSMEM stores signalled through mbarriers -------------------------------
// The per-step exchange between the CTAs of a cluster is a data flow, not a barrier: every
// producer writes its values straight into each consumer's shared memory with st.async, which
// also counts the bytes on the CONSUMER's mbarrier; a consumer proceeds when the bytes of the
// step have arrived.  Two buffers / two mbarriers alternate by step parity.  Re-use is safe
// without a second ("empty") handshake: a producer can only be one step ahead, because its
// next step needs this consumer's own output of the current step.
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arm(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after WAIT_LIMIT polls (each poll already blocks for a hardware-defined
// time slice), records the failure in *status and lets the kernel run to its end.
constexpr int WAIT_LIMIT = 1 << 20;
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, bool& dead, int* status) {
  if (dead) return false;
  for (int i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  dead = true;
  if (status != nullptr) atomicExch(status, 1);
  return false;
}
__device__ __forceinline__ unsigned map_to_rank(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_async_f32(unsigned raddr, float v, unsigned rbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(raddr), "r"(__float_as_uint(v)), "r"(rbar) : "memory");
}
__device__ __forceinline__ void st_async_f32x4(unsigned raddr, float a, float b, float c, float d, unsigned rbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(raddr), "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)),
                 "r"(__float_as_uint(d)), "r"(rbar) : "memory");
}

// Weights of 4 units x 3 gates at contraction index k, and the BT hidden values of k.
template <int BT, bool SMEM>
__device__ __forceinline__ void fwd_load(const float* wp, int kstride, int gstride, const float* hcur, int k,
                                         float4 (&w)[3], float (&hv)[BT]) {
#pragma unroll
  for (int g = 0; g < 3; ++g) {
    if (SMEM) {
      w[g] = *reinterpret_cast<const float4*>(wp + k * kstride + g * gstride);
    } else {
      // rows of the transposed copy are WtR floats (a multiple of 4) and every slice starts on a
      // multiple of 4 when Hc does, which the configuration requires for this mode
      w[g] = __ldg(reinterpret_cast<const float4*>(wp + (size_t)k * kstride + g * gstride));
    }
  }
  load_rows<BT>(hcur + k * BT, hv);
}

// Packed FP32 FMA (two IEEE fused multiply-adds per instruction on sm_100): units (0,1) and
// (2,3) of a weight float4 share one instruction; the hidden value is duplicated once per row.
template <int BT>
__device__ __forceinline__ void fwd_fma(float2 (&acc)[3][2][BT], const float4 (&w)[3], const float (&hv)[BT]) {
#pragma unroll
  for (int b = 0; b < BT; ++b) {
    const float2 hh = make_float2(hv[b], hv[b]);
#pragma unroll
    for (int g = 0; g < 3; ++g) {
      acc[g][0][b] = __ffma2_rn(make_float2(w[g].x, w[g].y), hh, acc[g][0][b]);
      acc[g][1][b] = __ffma2_rn(make_float2(w[g].z, w[g].w), hh, acc[g][1][b]);
    }
  }
}

// acc[g][c][b] += sum over this lane's k (= lane, lane+32, ...) of W(g, unit c, k) * h[k][b].
template <int BT, bool SMEM>
__device__ __forceinline__ void fwd_contract(float2 (&acc)[3][2][BT], const float* wp, int kstride, int gstride,
                                             const float* hcur, int lane, int Hb) {
#pragma unroll 2
  for (int k = lane; k < Hb; k += 32) {
    float4 w[3];
    float hv[BT];
    fwd_load<BT, SMEM>(wp, kstride, gstride, hcur, k, w, hv);
    fwd_fma<BT>(acc, w, hv);
  }
}

}  // namespace

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
// shared memory:  full [2]            mbarriers, one per hbuf parity (16 bytes)
//                 hbuf [2][HbP][BT]  fq_in(h) of the whole block, k-major
//                 wsm  [Hb][RS]      W(g, u0+j, k) at [k][g*Hc4 + j]; RS = 4 (mod 8) floats so
//                                    that float4 reads by lanes with consecutive k hit all banks
// Warps run free: no CTA-wide barrier inside the time loop.
template <int BT, int IPW>
__global__ void __launch_bounds__(NT, 1)
block_fwd_kernel(const BlockScanArgs a) {
  extern __shared__ __align__(16) float smem[];
  cg::cluster_group cluster = cg::this_cluster();
  constexpr int BTP = next_pow2(BT);
  constexpr int NV = 4 * BTP;                          // values per gate in the warp reduction

  const int C = a.C, Hb = a.Hb, Hc = a.Hc, Hc4 = a.Hc4, H = a.H, HbP = a.HbP;
  const int rank = blockIdx.x % C;
  const int n = blockIdx.x / C;                        // hidden block
  const int b0 = blockIdx.y * BT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int u0 = rank * Hc;                            // first owned unit (inside the block)
  const int nown = max(0, min(Hc, Hb - u0));           // owned units

  const unsigned full0 = smem_u32(smem);               // two 8-byte mbarriers
  float* hbuf = smem + 4;
  float* wsm = hbuf + ((2 * HbP * BT + 3) & ~3);        // 16-byte aligned weight rows
  const unsigned step_bytes = (unsigned)(C * Hc * BT * sizeof(float));
  if (tid == 0) {
    mbar_init(full0, 1);
    mbar_init(full0 + 8, 1);
    mbar_fence_init();
    // the sends of steps 0 and 1 land in buffers 1 and 0
    if (a.T > 1) mbar_arm(full0 + 8, step_bytes);
    if (a.T > 2) mbar_arm(full0, step_bytes);
  }

  const float* wbase;
  int kstride, gstride;
  if (a.w_in_smem) {
    kstride = a.RS;
    gstride = Hc4;
    const float* Wn = a.W + (size_t)n * a.w_block_stride;
    // Transposing fill: a thread takes one k and four adjacent units, so the four global loads are
    // coalesced across the warp (consecutive k) and the one float4 store is conflict-free (row
    // stride = 4 mod 8 floats); several items in flight per thread hide the load latency.
    const int nq = 3 * (Hc4 >> 2);
    const int total = nq * Hb;
#pragma unroll 4
    for (int idx = tid; idx < total; idx += NT) {
      const int k = idx % Hb;
      const int q = idx / Hb;
      const int g = q / (Hc4 >> 2), j0 = (q - g * (Hc4 >> 2)) << 2;
      const float* src = Wn + (size_t)g * a.w_gate_stride + (size_t)(u0 + j0) * Hb + k;
      float4 v;
      v.x = (j0 + 0 < nown) ? __ldg(src) : 0.f;
      v.y = (j0 + 1 < nown) ? __ldg(src + Hb) : 0.f;
      v.z = (j0 + 2 < nown) ? __ldg(src + 2 * Hb) : 0.f;
      v.w = (j0 + 3 < nown) ? __ldg(src + 3 * Hb) : 0.f;
      *reinterpret_cast<float4*>(wsm + k * kstride + g * Hc4 + j0) = v;
    }
    wbase = wsm;
  } else {
    // transposed global copy, rows padded with zeros: Wt[((n*Hb + k)*3 + g)*WtR + u]
    kstride = 3 * a.WtR;
    gstride = a.WtR;
    wbase = a.Wt + (size_t)n * Hb * 3 * a.WtR + u0;
  }

  // h_{-1}: every CTA loads the whole block row itself
  for (int idx = tid; idx < HbP * BT; idx += NT) {
    const int k = idx / BT, b = idx - k * BT;
    float v = 0.f;
    if (k < Hb && b0 + b < a.B) v = a.h0[(size_t)(b0 + b) * H + n * Hb + k];
    hbuf[idx] = a.qin.enabled ? fake_quant<true>(v, a.qin) : v;
    hbuf[HbP * BT + idx] = 0.f;
  }

  // After the reduction lane `lane` owns element (b, c) = (ridx >> 2, ridx & 3) of every
  // item (group of 4 units) its warp processes.
  const int ridx = reduced_index<NV>(lane);
  const int eb = ridx >> 2, ec = ridx & 3;
  const bool esend = reduced_owner<NV>(lane) && eb < BT;       // this lane publishes element (eb, ec)
  const bool eown = esend && (b0 + eb) < a.B;
  const int nitems = Hc4 >> 2;

  float hown[IPW], gr[IPW], gz[IPW], gn[IPW], bias_r[IPW], bias_z[IPW], bias_n[IPW];
  bool valid[IPW];
#pragma unroll
  for (int q = 0; q < IPW; ++q) {
    const int item = warp + q * NW;
    const int j = item * 4 + ec;
    valid[q] = eown && item < nitems && j < nown;
    hown[q] = 0.f; gr[q] = gz[q] = gn[q] = 0.f; bias_r[q] = bias_z[q] = bias_n[q] = 0.f;
    if (valid[q]) {
      const int u = n * Hb + u0 + j;
      hown[q] = a.h0[(size_t)(b0 + eb) * H + u];
      bias_r[q] = a.bh[u]; bias_z[q] = a.bh[H + u]; bias_n[q] = a.bh[2 * H + u];
      const float* g = a.gi + (size_t)(b0 + eb) * 3 * H + u;
      gr[q] = __ldcs(g); gz[q] = __ldcs(g + H); gn[q] = __ldcs(g + 2 * H);
    }
  }
  cluster.sync();            // weights, h_{-1} and the armed mbarriers are in place everywhere

  // A warp meets the same weights at every step, so the first NR k-slabs of each of its items stay
  // in registers for the whole scan (the step is bound by the shared-memory return path, and a
  // quarter of the register file is otherwise unused).
  constexpr int NR = (IPW == 1) ? B200GRU_FWD_NR : (IPW == 2 ? B200GRU_FWD_NR / 2 : 0);
  float4 wreg[IPW][NR > 0 ? NR : 1][3];
  if (NR > 0 && a.w_in_smem) {
#pragma unroll
    for (int q = 0; q < IPW; ++q)
#pragma unroll
      for (int i = 0; i < NR; ++i)
#pragma unroll
        for (int g = 0; g < 3; ++g) {
          const int k = lane + 32 * i, item = warp + q * NW;
          wreg[q][i][g] = (item < nitems && k < Hb)
                              ? *reinterpret_cast<const float4*>(wsm + k * a.RS + g * Hc4 + item * 4)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
        }
  }

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;
  unsigned phase0 = 0u, phase1 = 0u;      // parity of the next completion of each mbarrier
  bool dead = false;

  PHASE_DECL;
  for (int t = 0; t < a.T; ++t) {
    const int p = t & 1;
    const float* hcur = hbuf + p * HbP * BT;
    float* hnxt = hbuf + (p ^ 1) * HbP * BT;
    PHASE_START();
    if (t > 0) {
      if (C == 1) {
        // a single CTA owns the whole block: plain stores and one CTA barrier per step
        __syncthreads();
      } else {
        mbar_wait(full0 + 8 * p, p ? phase1 : phase0, dead, a.status);
        if (p) phase1 ^= 1u; else phase0 ^= 1u;
        // buffer p is filled again by the sends of step t+1
        if (tid == 0 && t + 1 <= a.T - 2) mbar_arm(full0 + 8 * p, step_bytes);
      }
    }
    const unsigned nxt_addr = smem_u32(hnxt);
    const unsigned nxt_bar = full0 + 8 * (p ^ 1);
    PHASE_MARK(5);

#pragma unroll
    for (int q = 0; q < IPW; ++q) {
      const int item = warp + q * NW;
      if (item < nitems) {                              // warp-uniform
        // next step's gi goes in flight before the contraction
        float ngr = 0.f, ngz = 0.f, ngn = 0.f;
        if (valid[q] && t + 1 < a.T) {
          const float* g = a.gi + (size_t)(t + 1) * gi_step + (size_t)(b0 + eb) * 3 * H + n * Hb + u0 + item * 4 + ec;
          ngr = __ldcs(g); ngz = __ldcs(g + H); ngn = __ldcs(g + 2 * H);
        }

        float2 acc[3][2][BT];                            // [gate][unit pair][row]
#pragma unroll
        for (int g = 0; g < 3; ++g)
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[g][c][b] = make_float2(0.f, 0.f);

        const float* wp = wbase + item * 4;
        if (a.w_in_smem) {
          if (NR > 0) {
#pragma unroll
            for (int i = 0; i < NR; ++i) {
              const int k = lane + 32 * i;
              float hv[BT];
              if (k < Hb) {
                load_rows<BT>(hcur + k * BT, hv);
                fwd_fma<BT>(acc, wreg[q][i], hv);
              }
            }
          }
          fwd_contract<BT, true>(acc, wp, kstride, gstride, hcur, lane + 32 * NR, Hb);
        } else {
          fwd_contract<BT, false>(acc, wp, kstride, gstride, hcur, lane, Hb);
        }
        PHASE_MARK(0);

        float s[3];
#pragma unroll
        for (int g = 0; g < 3; ++g) {
          float vals[NV];
#pragma unroll
          for (int b = 0; b < BTP; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float2 pr = acc[g][c >> 1][b < BT ? b : 0];
              vals[b * 4 + c] = (b < BT) ? ((c & 1) ? pr.y : pr.x) : 0.f;
            }
          warp_reduce_scatter<NV>(vals, lane);
          s[g] = vals[0];
        }
        PHASE_MARK(1);

        const int j = item * 4 + ec;
        if (esend && j < Hc) {
          float hq = 0.f;
          if (valid[q]) {
            const float ghn = s[2] + bias_n[q];
            const GateOut go = gru_gates(gr[q], gz[q], gn[q], s[0] + bias_r[q], s[1] + bias_z[q], ghn, hown[q]);
            const float hnew = a.qout.enabled ? fake_quant<true>(go.h_raw, a.qout) : go.h_raw;
            hown[q] = hnew;
            const size_t o = (size_t)t * out_step + (size_t)(b0 + eb) * H + n * Hb + u0 + j;
            a.out[o] = hnew;
            if (a.save != nullptr) {
              __stcs(a.save + o, go.r);
              __stcs(a.save + comp + o, go.z);
              __stcs(a.save + 2 * comp + o, go.n);
              __stcs(a.save + 3 * comp + o, ghn);
            }
            hq = a.qin.enabled ? fake_quant<true>(hnew, a.qin) : hnew;
          }
          if (t + 1 < a.T) {
            if (C == 1) {
              hnxt[(u0 + j) * BT + eb] = hq;
            } else {
              // publish fq_in(h_t) of this element to every CTA of the cluster (itself included)
              const unsigned eoff = (unsigned)(((u0 + j) * BT + eb) * sizeof(float));
              for (int r = 0; r < C; ++r)
                st_async_f32(map_to_rank(nxt_addr + eoff, r), hq, map_to_rank(nxt_bar, r));
            }
          }
        }
        gr[q] = ngr; gz[q] = ngz; gn[q] = ngn;
        PHASE_MARK(2);
      }
    }
  }
  cluster.sync();            // nobody leaves while a peer could still be reading or writing
}

// ---------------------------------------------------------------------------
// backward (serial part): dgi[t], dh chain, dh0.  Gate activations come from `S`.
// ---------------------------------------------------------------------------
// shared memory:  full [2]              mbarriers, one per recv parity (16 bytes)
//                 recv [2][C][Hc][BT]   partial dh_via sent by every rank (parity = step)
//                 xs   [2][3][Hc4][BTX] dgh of the owned units (parity = step), rows padded to float4
//                 wsm  [3*Hc4][Hb4]     W(g, u0+j, k) at [(g*Hc4 + j)][k]   (k contiguous)
// The second contraction half parks its sums in the idle parity half of `recv`.
template <int BT, int TW, int GPT>
__global__ void __launch_bounds__(NT, 1)
block_bwd_kernel(const BlockScanArgs a) {
  extern __shared__ __align__(16) float smem[];
  cg::cluster_group cluster = cg::this_cluster();

  const int C = a.C, Hb = a.Hb, Hc = a.Hc, Hc4 = a.Hc4, H = a.H, HbP = a.HbP, Hb4 = a.Hb4;
  const int rank = blockIdx.x % C;
  const int n = blockIdx.x / C;
  const int b0 = blockIdx.y * BT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int u0 = rank * Hc;
  const int nown = max(0, min(Hc, Hb - u0));
  const int slice = Hc * BT;                           // floats one rank sends to one peer
  constexpr int BTX = (BT + 3) & ~3;                   // dgh rows padded to float4

  const unsigned full0 = smem_u32(smem);               // two 8-byte mbarriers
  float* recv = smem + 4;                              // [2][C*slice]
  float* xs2 = recv + ((2 * C * slice + 3) & ~3);      // [2][3*Hc4][BTX]
  const unsigned step_bytes = (unsigned)(C * slice * sizeof(float));
  if (tid == 0) {
    mbar_init(full0, 1);
    mbar_init(full0 + 8, 1);
    mbar_fence_init();
    mbar_arm(full0, step_bytes);
    if (a.T > 1) mbar_arm(full0 + 8, step_bytes);
  }
  float* wsm = xs2 + 2 * 3 * Hc4 * BTX;

  const float* wbase;
  size_t gstride;      // between gates
  int rstride;         // between units
  if (a.w_in_smem) {
    gstride = (size_t)Hc4 * Hb4;
    rstride = Hb4;
    const float* Wn = a.W + (size_t)n * a.w_block_stride;
    const int total = 3 * Hc4 * Hb4;
    const bool vec4 = (Hb % 4 == 0) && (a.w_gate_stride % 4 == 0) && (a.w_block_stride % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(a.W) & 15u) == 0);
    if (vec4) {
      // rows are copied as they lie (k contiguous on both sides): float4s, several in flight per thread
      const int kq = Hb4 >> 2;
#pragma unroll 4
      for (int idx = tid; idx < 3 * Hc4 * kq; idx += NT) {
        const int k4 = idx % kq;
        const int gj = idx / kq;
        const int g = gj / Hc4, j = gj - g * Hc4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < nown && 4 * k4 < Hb)                  // the padding beyond Hb stays zero
          v = __ldg(reinterpret_cast<const float4*>(Wn + (size_t)g * a.w_gate_stride + (size_t)(u0 + j) * Hb) + k4);
        reinterpret_cast<float4*>(wsm)[idx] = v;
      }
    } else {
      for (int idx = tid; idx < total; idx += NT) {
        const int k = idx % Hb4;
        const int gj = idx / Hb4;
        const int g = gj / Hc4, j = gj - g * Hc4;
        float v = 0.f;
        if (j < nown && k < Hb) v = Wn[(size_t)g * a.w_gate_stride + (size_t)(u0 + j) * Hb + k];
        wsm[idx] = v;
      }
    }
    wbase = wsm;
  } else {
    gstride = (size_t)a.w_gate_stride;
    rstride = Hb;
    wbase = a.W + (size_t)n * a.w_block_stride + (size_t)u0 * Hb;
  }
  for (int idx = tid; idx < 2 * C * slice; idx += NT) recv[idx] = 0.f;
  for (int idx = tid; idx < 2 * 3 * Hc4 * BTX; idx += NT) xs2[idx] = 0.f;

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;

  // element ownership for the gate phase: idx -> (j, b), b fastest so that `recv` reads are contiguous
  float dh_acc[GPT];
  float c_do[GPT], c_r[GPT], c_z[GPT], c_n[GPT], c_ghn[GPT], c_hp[GPT];
  bool valid[GPT];
  int ib[GPT], ij[GPT];
  size_t off[GPT];
#pragma unroll
  for (int q = 0; q < GPT; ++q) {
    const int idx = tid + q * NT;
    ij[q] = idx / BT;
    ib[q] = idx - ij[q] * BT;
    valid[q] = (idx < Hc * BT) && (ij[q] < nown) && (b0 + ib[q] < a.B);
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
  cluster.sync();            // weights, zeroed buffers and the armed mbarriers are in place everywhere
  unsigned phase0 = 0u, phase1 = 0u;      // parity of the next completion of each mbarrier
  bool dead = false;

  // contraction geometry: k tiles of 32*TW positions, NH halves of the (gate, unit) index;
  // ntiles * NH <= NW whenever NH > 1, so one round of warps covers both halves of a tile.
  const int ktile = 32 * TW;
  const int ntiles = (HbP + ktile - 1) / ktile;
  const int NH = a.NH;
  const int ncon = 3 * Hc4;
  const int con_per = (ncon + NH - 1) / NH;

  PHASE_DECL;
  for (int t = a.T - 1; t >= 0; --t) {
    PHASE_START();
    const int par = (a.T - 1 - t) & 1;
    float* rcur = recv + par * C * slice;
    // The other parity buffer is idle during this step's contraction, so the second-half sums
    // park there.  A peer one step ahead may already write its slice [r*slice, (r+1)*slice) of
    // that buffer; this is exactly the park rows of the positions rank r owns, and r can only be
    // ahead after it has received the combined values of those rows -- i.e. after they were read.
    float* park = recv + (par ^ 1) * C * slice;
    const unsigned rcur_addr = smem_u32(rcur);
    const unsigned rcur_bar = full0 + 8 * par;
    // dgh alternates between two buffers: a warp that already has its partials for this step may
    // run ahead into the next step's gate phase while a slower warp still reads this step's dgh.
    float* xs = xs2 + par * 3 * Hc4 * BTX;

    // ---- gate gradients of the owned elements
    float dh_direct[GPT], mask_in[GPT];
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      dh_direct[q] = 0.f; mask_in[q] = 1.f;
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
        xs[(0 * Hc4 + ij[q]) * BTX + ib[q]] = gg.dgr;
        xs[(1 * Hc4 + ij[q]) * BTX + ib[q]] = gg.dgz;
        xs[(2 * Hc4 + ij[q]) * BTX + ib[q]] = gg.dghn;
      }
    }
    // operands of step t-1 go in flight now
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
    PHASE_MARK(8);
    __syncthreads();
    PHASE_MARK(9);

    // ---- partial[k][b] = sum over own (g, j) of W(g, u0+j, k) * dgh[b, g, j]
    for (int item0 = 0; item0 < ntiles * NH; item0 += NW) {
      const int item = item0 + warp;
      const bool live = item < ntiles * NH;
      const int kt = live ? item % ntiles : 0, half = live ? item / ntiles : 0;
      const int kbase = kt * ktile + lane * TW;
      float acc[TW * BT];                               // [i][b], the layout of `recv` rows
#pragma unroll
      for (int i = 0; i < TW * BT; ++i) acc[i] = 0.f;
      if (live) {
        const int c0 = half * con_per, c1 = min(ncon, c0 + con_per);
        if (a.w_in_smem) {
          if (kbase < Hb4) {
            const float* wp = wsm + (size_t)c0 * Hb4 + kbase;
            const float* xp = xs + c0 * BTX;
#pragma unroll 8
            for (int c = c0; c < c1; ++c, wp += Hb4, xp += BTX) {
              float w[TW];
              if constexpr (TW == 4) {
                const float4 x = *reinterpret_cast<const float4*>(wp);
                w[0] = x.x; w[1] = x.y; w[2] = x.z; w[3] = x.w;
              } else {
                w[0] = wp[0];
              }
              float xv[BTX];
              load_rows_exact<BT, BTX>(xp, xv);
              if constexpr (TW == 4) {
                // packed FP32 FMA: positions (0,1) and (2,3) of the weight float4 share an instruction
#pragma unroll
                for (int bb = 0; bb < BT; ++bb) {
                  const float2 xx = make_float2(xv[bb], xv[bb]);
                  const float2 r01 = __ffma2_rn(make_float2(w[0], w[1]), xx, make_float2(acc[0 * BT + bb], acc[1 * BT + bb]));
                  const float2 r23 = __ffma2_rn(make_float2(w[2], w[3]), xx, make_float2(acc[2 * BT + bb], acc[3 * BT + bb]));
                  acc[0 * BT + bb] = r01.x; acc[1 * BT + bb] = r01.y;
                  acc[2 * BT + bb] = r23.x; acc[3 * BT + bb] = r23.y;
                }
              } else {
#pragma unroll
                for (int i = 0; i < TW; ++i)
#pragma unroll
                  for (int bb = 0; bb < BT; ++bb) acc[i * BT + bb] = fmaf(w[i], xv[bb], acc[i * BT + bb]);
              }
            }
          }
        } else {
          int g = c0 / Hc4, j = c0 - g * Hc4;
          for (int c = c0; c < c1; ++c) {
            float w[TW];
#pragma unroll
            for (int i = 0; i < TW; ++i)
              w[i] = (j < nown && kbase + i < Hb)
                         ? __ldg(wbase + (size_t)g * gstride + (size_t)j * rstride + kbase + i) : 0.f;
            float xv[BTX];
            load_rows_exact<BT, BTX>(xs + c * BTX, xv);
#pragma unroll
            for (int i = 0; i < TW; ++i)
#pragma unroll
              for (int bb = 0; bb < BT; ++bb) acc[i * BT + bb] = fmaf(w[i], xv[bb], acc[i * BT + bb]);
            if (++j == Hc4) { j = 0; ++g; }
          }
        }
        if (half > 0 && kbase < HbP) {
          // park: [k][b] of the second half -- it fits in the idle receive buffer
          float* pp = park + (size_t)kbase * BT;
          if constexpr ((TW * BT) % 4 == 0) {
#pragma unroll
            for (int v = 0; v < TW * BT / 4; ++v)
              *reinterpret_cast<float4*>(pp + 4 * v) = make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < TW * BT; ++i)
              if (kbase + i / BT < HbP) pp[i] = acc[i];
          }
        }
      }
      PHASE_MARK(10);
      if (NH > 1) __syncthreads();
      PHASE_MARK(11);
      if (live && half == 0 && kbase < HbP) {
        // combine the halves and hand each position to the rank that owns it
        if (NH > 1) {
          const float* pp = park + (size_t)kbase * BT;
          if constexpr ((TW * BT) % 4 == 0) {
#pragma unroll
            for (int v = 0; v < TW * BT / 4; ++v) {
              const float4 x = *reinterpret_cast<const float4*>(pp + 4 * v);
              acc[4 * v] += x.x; acc[4 * v + 1] += x.y; acc[4 * v + 2] += x.z; acc[4 * v + 3] += x.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < TW * BT; ++i)
              if (kbase + i / BT < HbP) acc[i] += pp[i];
          }
        }
        const int dst0 = kbase / Hc, jj0 = kbase - dst0 * Hc;
        if (C == 1) {
          // single CTA: the "receive" rows are local
#pragma unroll
          for (int i = 0; i < TW; ++i) {
            const int k = kbase + i;
            if (k < HbP) {
#pragma unroll
              for (int bb = 0; bb < BT; ++bb) rcur[k * BT + bb] = acc[i * BT + bb];
            }
          }
        } else if ((TW * BT) % 4 == 0 && jj0 + TW <= Hc) {
          // the TW positions of this lane belong to one rank and form one contiguous run there
          const unsigned doff = (unsigned)((rank * slice + jj0 * BT) * sizeof(float));
          const unsigned daddr = map_to_rank(rcur_addr + doff, dst0), dbar = map_to_rank(rcur_bar, dst0);
#pragma unroll
          for (int v = 0; v < TW * BT / 4; ++v)
            st_async_f32x4(daddr + 16 * v, acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3], dbar);
        } else {
#pragma unroll
          for (int i = 0; i < TW; ++i) {
            const int k = kbase + i;
            if (k < HbP) {
              const int dst = k / Hc, jj = k - dst * Hc;
              const unsigned doff = (unsigned)((rank * slice + jj * BT) * sizeof(float));
              const unsigned daddr = map_to_rank(rcur_addr + doff, dst), dbar = map_to_rank(rcur_bar, dst);
#pragma unroll
              for (int bb = 0; bb < BT; ++bb) st_async_f32(daddr + 4 * bb, acc[i * BT + bb], dbar);
            }
          }
        }
      }
    }
    PHASE_MARK(12);
    if (C == 1) {
      __syncthreads();
    } else {
      mbar_wait(rcur_bar, par ? phase1 : phase0, dead, a.status);
      if (par) phase1 ^= 1u; else phase0 ^= 1u;
      if (tid == 0 && t >= 2) mbar_arm(rcur_bar, step_bytes);     // this buffer receives again two steps on
    }
    PHASE_MARK(13);

    // ---- dh for the owned elements: C partials in rank order
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      if (valid[q]) {
        float s = 0.f;
        for (int r = 0; r < C; ++r) s += rcur[r * slice + ij[q] * BT + ib[q]];
        dh_acc[q] = dh_direct[q] + s * mask_in[q];
      }
    }
    PHASE_MARK(14);
  }

#pragma unroll
  for (int q = 0; q < GPT; ++q)
    if (valid[q]) a.dh0[off[q]] = dh_acc[q];
  cluster.sync();            // nobody leaves while a peer could still be reading or writing
}

// ---------------------------------------------------------------------------
// host side: configuration and launch
// ---------------------------------------------------------------------------

using KernelFn = void (*)(const BlockScanArgs);

template <int BT>
static KernelFn pick_fwd(int ipw) {
  if (ipw <= 1) return block_fwd_kernel<BT, 1>;
  if (ipw <= 2) return block_fwd_kernel<BT, 2>;
  return block_fwd_kernel<BT, 8>;
}
template <int BT>
static KernelFn pick_bwd(int tw, int gpt) {
  if (tw == 4) return gpt <= 1 ? block_bwd_kernel<BT, 4, 1> : block_bwd_kernel<BT, 4, 8>;
  return gpt <= 1 ? block_bwd_kernel<BT, 1, 1> : block_bwd_kernel<BT, 1, 8>;
}

static KernelFn pick_kernel(bool fwd, const BlockScanConfig& c) {
#define B200GRU_PICK(B) return fwd ? pick_fwd<B>(c.IPW) : pick_bwd<B>(c.TW, c.GPT)
  switch (c.BT) {
    case 1: B200GRU_PICK(1);
    case 2: B200GRU_PICK(2);
    case 3: B200GRU_PICK(3);
    case 4: B200GRU_PICK(4);
    case 5: B200GRU_PICK(5);
    case 6: B200GRU_PICK(6);
    default: B200GRU_PICK(8);
  }
#undef B200GRU_PICK
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

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Device address of g_scan_status on the current device (looked up once per device).
static int* scan_status_address() {
  constexpr int MAX_DEV = 64;
  static std::mutex mu;
  static int* table[MAX_DEV] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (table[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_scan_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    table[dev] = static_cast<int*>(p);
  }
  return table[dev];
}

// Pick the cluster size, batch tile and weight placement that minimise a simple cost model:
//   step = max(FMA issue, shared-memory streaming) + barrier;  total = waves * step.
bool choose_block_config(bool fwd, int B, int Hb, int nb, BlockScanConfig* out) {
  const DeviceInfo di = device_info();
  if (!di.ok) return false;
  double best = 1e300;
  bool found = false;
  const int bts[7] = {1, 2, 3, 4, 5, 6, 8};
  const int cs[5] = {1, 2, 4, 8, 16};
  // Every cluster size is tried with the exact slice width ceil(Hb / C) and, when that is no multiple
  // of 4, with the width rounded up to one (the last ranks then own fewer units or none): the
  // streamed-weight form and the float4 exchange need Hc % 4 == 0, and widths such as Hb = 520 or
  // 1000 have no cluster size that gives it exactly.
  for (int cv = 0; cv < 10; ++cv) {
    const int ci = cv >> 1;
    const int C = cs[ci];
    if (C > 1 && Hb / C < 8) continue;                 // slices thinner than 8 units: not worth a barrier
    int Hc = cdiv(Hb, C);
    if (cv & 1) {
      if (C == 1 || Hc % 4 == 0) continue;             // nothing to round
      Hc = round_up(Hc, 4);
    }
    const int Hc4 = round_up(Hc, 4);
    const int HbP = C * Hc;
    const int Hb4 = round_up(HbP, 4);
    const int nitems = Hc4 / 4;
    const int ipw = cdiv(nitems, NW);
    if (ipw > 8) continue;
    for (int bi = 0; bi < 7; ++bi) {
      const int BT = bts[bi];
      if (bi > 0 && bts[bi - 1] >= B) continue;        // a smaller tile already covers the batch
      if (C > 1 && (Hc * BT) % 4 != 0) continue;       // published slices move as float4
      if (Hc * BT > 8 * NT) continue;
      BlockScanConfig c;
      c.C = C; c.BT = BT; c.Hc = Hc; c.Hc4 = Hc4; c.HbP = HbP; c.Hb4 = Hb4;
      c.IPW = ipw <= 1 ? 1 : (ipw <= 2 ? 2 : 8);
      int rs = 3 * Hc4;
      while (rs % 8 != 4) ++rs;
      c.RS = rs;
      c.TW = (HbP >= 64 * NW) ? 4 : 1;
      const int ntiles = cdiv(HbP, 32 * c.TW);
      c.NH = (2 * ntiles <= NW) ? 2 : 1;
      c.GPT = (Hc * BT <= NT) ? 1 : 8;
      for (int ws = 1; ws >= 0; --ws) {
        if (ws == 0 && fwd && C > 1 && Hc % 4 != 0) continue;   // streamed weights are read as float4
        size_t fl;
        if (fwd) fl = 4 + (size_t)((2 * HbP * BT + 3) & ~3) + (ws ? (size_t)Hb * c.RS : 0);
        else fl = 4 + (size_t)((2 * C * Hc * BT + 3) & ~3) + (size_t)2 * 3 * Hc4 * ((BT + 3) & ~3) + (ws ? (size_t)3 * Hc4 * Hb4 : 0);
        const size_t smem = fl * sizeof(float);
        if (smem > di.smem_optin) continue;
        c.w_in_smem = ws; c.smem = smem;
        KernelFn fn = pick_kernel(fwd, c);
        const int active = max_active_clusters(fn, C, smem);
        if (active <= 0) continue;
        const long long nclusters = (long long)nb * cdiv(B, BT);
        const double waves = (double)((nclusters + active - 1) / active);
        const double fma = 3.0 * Hc4 * Hb * BT / 128.0;
        const double stream = 3.0 * Hc4 * Hb * 4.0 / (ws ? 128.0 : 24.0) + (double)Hb * BT * 4.0 * NW / 128.0;
        const double barrier = C > 1 ? 1200.0 + 40.0 * C : 200.0;
        const double cost = waves * ((fma > stream ? fma : stream) + barrier + 400.0);
        if (cost < best) { best = cost; found = true; *out = c; }
        break;                                          // weights in smem fit: do not also try global
      }
    }
  }
  return found;
}

int launch_block_scan(bool fwd, const BlockScanConfig& c, BlockScanArgs args, int nb, cudaStream_t st) {
  args.C = c.C; args.Hc = c.Hc; args.Hc4 = c.Hc4; args.HbP = c.HbP; args.Hb4 = c.Hb4; args.RS = c.RS;
  args.NH = c.NH; args.w_in_smem = c.w_in_smem; args.WtR = c.Hb4 + 4;
  args.status = scan_status_address();
  KernelFn fn = pick_kernel(fwd, c);
  const int active = max_active_clusters(fn, c.C, c.smem);                      // also sets the attributes
  static const bool debug = getenv("B200GRU_DEBUG") != nullptr;
  if (debug)
    fprintf(stderr, "[b200gru] %s T=%d B=%d H=%d nb=%d Hb=%d: C=%d BT=%d Hc=%d IPW=%d TW=%d NH=%d GPT=%d "
            "w_in_smem=%d smem=%zu active_clusters=%d grid=(%d,%d)\n", fwd ? "block_fwd" : "block_bwd", args.T,
            args.B, args.H, nb, args.Hb, c.C, c.BT, c.Hc, c.IPW, c.TW, c.NH, c.GPT, c.w_in_smem, c.smem, active,
            c.C * nb, cdiv(args.B, c.BT));
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
  cudaLaunchKernelEx(&cfg, fn, args);
  note_launch();
  return check_launch(fwd ? "block_fwd_kernel" : "block_bwd_kernel");
}

extern "C" int b200gru_device_status(int reset) {
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_scan_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_scan_status, &z, sizeof(int));
  }
  const int d = diag_read_status(reset);
  const int f = bfly_read_status(reset);
  const int g = tc::tc_read_status(reset);
  const int s = tc::tc_step_read_status(reset);
  if (d < 0 || f < 0 || g < 0 || s < 0) return -1;
  return (v != 0 || d != 0 || f != 0 || g != 0 || s != 0) ? 1 : 0;
}

}  // namespace b200gru

B200GRU_DEFINE_PHASE_READER(b200gru_debug_phase_cycles)
