// Butterfly scan, staged variant (aligned problems: H % 4 == 0, 16-byte aligned tensors).
//
// Same arithmetic and pass structure as butterfly_scan.cu, with the memory side rebuilt around
// bulk (1-D TMA) copies and mbarriers so that nothing on the per-step chain waits for L2:
//
//   * twiddles: resident in shared memory when all of them fit; otherwise STREAMED -- the
//     twiddle block of pass q+2 (three contiguous runs, one per gate) is copied while passes
//     q and q+1 compute, two buffers alternating;
//   * gi[t] (forward) and dout / gate activations / h_{t-1} (backward) arrive as row-sized bulk
//     copies issued one step ahead;
//   * the running vectors use a swizzled row layout, phys(i) = i + 8 * (i / 64), which makes the
//     strided accesses of the middle passes bank-conflict free; the stride-1 pass and the gate
//     phases move float4s.
//
// Every wait is a bounded poll of an mbarrier; a wait that gives up sets a device flag and the
// kernel runs to its end (results invalid, flag visible through b200gru_device_status).

#include <cooperative_groups.h>
#include <type_traits>

#include "butterfly_scan.cuh"

namespace b200gru {

namespace cg = cooperative_groups;

namespace {

constexpr int NT = 384;                 // 12 warps: one radix-8 item per thread per pass at Hpad = 1024
constexpr int WAIT_LIMIT = 1 << 20;

static __device__ int g_bfly_status;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arm(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_wait(unsigned bar, unsigned parity, bool& dead) {
  if (dead) return;
  for (int i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return;
  dead = true;
  atomicExch(&g_bfly_status, 1);
}

__device__ __forceinline__ int sw(int i) { return i + ((i >> 6) << 3); }

// ---- distributed shared memory: stores into the peer CTA that count their bytes on its mbarrier ----
__device__ __forceinline__ unsigned map_to_rank(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_async_v4(unsigned raddr, float4 v, unsigned rbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(raddr), "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)), "r"(__float_as_uint(v.z)),
                 "r"(__float_as_uint(v.w)), "r"(rbar) : "memory");
}
template <int V>
__device__ __forceinline__ void st_async_v(unsigned raddr, const float (&x)[V], unsigned rbar) {
  if constexpr (V == 4) {
    st_async_v4(raddr, make_float4(x[0], x[1], x[2], x[3]), rbar);
  } else {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];"
                 ::"r"(raddr), "r"(__float_as_uint(x[0])), "r"(__float_as_uint(x[1])), "r"(rbar) : "memory");
  }
}

// V (2 or 4) adjacent floats as one vector access; STREAM: evict-first store
template <int V>
__device__ __forceinline__ void ldv(const float* p, float (&x)[V]) {
  if constexpr (V == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
    const float2 v = *reinterpret_cast<const float2*>(p);
    x[0] = v.x; x[1] = v.y;
  }
}
template <int V, bool STREAM>
__device__ __forceinline__ void stv(float* p, const float (&x)[V]) {
  if constexpr (V == 4) {
    if (STREAM) __stcs(reinterpret_cast<float4*>(p), make_float4(x[0], x[1], x[2], x[3]));
    else *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  } else {
    if (STREAM) __stcs(reinterpret_cast<float2*>(p), make_float2(x[0], x[1]));
    else *reinterpret_cast<float2*>(p) = make_float2(x[0], x[1]);
  }
}

template <int R, int P, int BT, bool TRANSPOSE>
__device__ __forceinline__ void stage_regs(float (&v)[BT][1 << R], const float4 (&tw)[(1 << R) / 2]) {
  int idx = 0;
#pragma unroll
  for (int e = 0; e < (1 << R); ++e) {
    if (e & (1 << P)) continue;
    const float4 t = tw[idx];
#pragma unroll
    for (int b = 0; b < BT; ++b) {
      const float a0 = v[b][e], a1 = v[b][e | (1 << P)];
      if (!TRANSPOSE) {
        v[b][e] = fmaf(t.y, a1, t.x * a0);
        v[b][e | (1 << P)] = fmaf(t.z, a0, t.w * a1);
      } else {
        v[b][e] = fmaf(t.z, a1, t.x * a0);
        v[b][e | (1 << P)] = fmaf(t.y, a0, t.w * a1);
      }
    }
    ++idx;
  }
}

template <int R, int BT, bool TRANSPOSE>
__device__ __forceinline__ void stage_dispatch(float (&v)[BT][1 << R], const float4 (&tw)[(1 << R) / 2], int p) {
  if (R >= 3 && p == 2) stage_regs<R, (R >= 3 ? 2 : 0), BT, TRANSPOSE>(v, tw);
  else if (R >= 2 && p == 1) stage_regs<R, (R >= 2 ? 1 : 0), BT, TRANSPOSE>(v, tw);
  else stage_regs<R, 0, BT, TRANSPOSE>(v, tw);
}

// Twiddle order used by the staged kernels.  Within one stage the reference order is by pair
// index; a thread of a radix-2^R pass needs pairs pair0(q) + (idx << lb), idx < 2^(R-1), which are
// 2^(R-1) * 16 bytes (or more) apart between neighbouring lanes: a 4-way bank conflict on every
// float4 load.  The staged kernels therefore read a copy in which every stage is stored in the
// order its pass consumes it, position idx * G + q (G items per gate), so that a warp reads 32
// consecutive float4.  tw_source_index maps such a position back to the pair index.
__host__ __device__ inline int tw_source_index(const BflyPass& pd, int logn, int half, int k) {
  if (pd.r >= 2) {
    const int R = pd.r, lb = pd.lb;
    const int G = half >> (R - 1);
    const int idx = k / G, q = k - idx * G;
    const int low = q & ((1 << lb) - 1), high = q >> lb;
    return ((high << (lb + R - 1)) | low) + (idx << lb);
  }
  if (pd.nst == 1 && pd.lb >= 2 && logn >= 3) {      // the 4-pairs-per-thread single-stage pass
    const int G4 = half >> 2;
    const int j = k / G4, q = k - j * G4;
    return 4 * q + j;
  }
  return k;
}

// dst[g][l][k] = src[g][l][tw_source_index(pass of l, k)]
__global__ void __launch_bounds__(256)
bfly_permute_twiddles_kernel(const float4* __restrict__ src, float4* __restrict__ dst, const BflyArgs a) {
  const int half = a.Hpad >> 1;
  const int total = 3 * a.nstages * half;
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  const int k = i % half;
  const int gl = i / half;
  const int l = gl % a.nstages;
  int p = 0;
  while (p + 1 < a.npasses && l >= a.passes[p].l0 + a.passes[p].nst) ++p;
  dst[i] = src[(size_t)gl * half + tw_source_index(a.passes[p], a.logn, half, k)];
}

// A float4 of twiddles from shared memory (by 32-bit shared address) or from global memory.
template <bool TW_SMEM>
__device__ __forceinline__ float4 tw_load(const float4* p) {
  if (TW_SMEM) {
    float4 v;
    asm("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
        : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(p)));
    return v;
  }
  return __ldg(p);
}

// One pass over the three gates on swizzled rows of stride RSZ.  Twiddle of (gate g, stage l,
// pair) is twp[g * tw_gate + (l - tw_l0) * half + pair].
template <int R, int BT, bool TRANSPOSE, bool TW_SMEM>
__device__ __forceinline__ void run_pass2_r(const BflyPass pd, const float* src, int src_gate, float* dst,
                                            int dst_gate, const float4* twp, int tw_gate, int tw_l0, int Hpad,
                                            int RSZ, int logn, int ngates = 3, int nthr = NT) {
  constexpr int E = 1 << R;
  const int lb = pd.lb;
  const int pb0 = pd.pb[0], pb1 = pd.pb[1], pb2 = pd.pb[2];
  const int lgG = logn - R;                             // log2 of the groups per gate
  const int G = 1 << lgG;
  const int half = Hpad >> 1;
  for (int item = threadIdx.x; item < ngates * G; item += nthr) {
    const int g = item >> lgG, q = item & (G - 1);
    const int low = q & ((1 << lb) - 1), high = q >> lb;
    const int base = (high << (lb + R)) | low;

    // The idx-th pair of this group has the same twiddle index at every stage of the pass
    // (removing the stage's own bit from the position leaves (high, idx, low)); in the permuted
    // copy it sits at idx * G + q.
    float4 t[3][E / 2];
    int pbit[3];
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      pbit[s] = 0;
      if (s < pd.nst) {
        const int so = TRANSPOSE ? (pd.nst - 1 - s) : s;          // stage offset inside the pass
        pbit[s] = so == 0 ? pb0 : (so == 1 ? pb1 : pb2);
        const float4* tl = twp + (g * tw_gate + (pd.l0 + so - tw_l0) * half + q);
#pragma unroll
        for (int idx = 0; idx < E / 2; ++idx) t[s][idx] = tw_load<TW_SMEM>(tl + (idx << lgG));
      }
    }

    float v[BT][E];
    const float* sp = src + (size_t)g * src_gate;
    float* dp = dst + (size_t)g * dst_gate;
    const bool contiguous = (lb == 0);
    const int pbase = sw(base);
    // the swizzle is affine in the element number unless the pass straddles bit 6
    const bool uniform = (lb + R <= 6) || (lb >= 6);
    const int estride = (lb >= 6) ? ((1 << lb) + (8 << (lb - 6))) : (1 << lb);
    if (contiguous) {
#pragma unroll
      for (int b = 0; b < BT; ++b) {
        if constexpr (E == 8) {
          const float4 x0 = *reinterpret_cast<const float4*>(sp + b * RSZ + pbase);
          const float4 x1 = *reinterpret_cast<const float4*>(sp + b * RSZ + pbase + 4);
          v[b][0] = x0.x; v[b][1] = x0.y; v[b][2] = x0.z; v[b][3] = x0.w;
          v[b][4] = x1.x; v[b][5] = x1.y; v[b][6] = x1.z; v[b][7] = x1.w;
        } else if constexpr (E == 4) {
          const float4 x0 = *reinterpret_cast<const float4*>(sp + b * RSZ + pbase);
          v[b][0] = x0.x; v[b][1] = x0.y; v[b][2] = x0.z; v[b][3] = x0.w;
        } else {
          const float2 x0 = *reinterpret_cast<const float2*>(sp + b * RSZ + pbase);
          v[b][0] = x0.x; v[b][1] = x0.y;
        }
      }
    } else if (uniform) {
#pragma unroll
      for (int b = 0; b < BT; ++b)
#pragma unroll
        for (int e = 0; e < E; ++e) v[b][e] = sp[b * RSZ + pbase + e * estride];
    } else {
#pragma unroll
      for (int b = 0; b < BT; ++b)
#pragma unroll
        for (int e = 0; e < E; ++e) v[b][e] = sp[b * RSZ + sw(base + (e << lb))];
    }

#pragma unroll
    for (int s = 0; s < 3; ++s)
      if (s < pd.nst) stage_dispatch<R, BT, TRANSPOSE>(v, t[s], pbit[s]);

    if (contiguous) {
#pragma unroll
      for (int b = 0; b < BT; ++b) {
        if constexpr (E == 8) {
          *reinterpret_cast<float4*>(dp + b * RSZ + pbase) = make_float4(v[b][0], v[b][1], v[b][2], v[b][3]);
          *reinterpret_cast<float4*>(dp + b * RSZ + pbase + 4) = make_float4(v[b][4], v[b][5], v[b][6], v[b][7]);
        } else if constexpr (E == 4) {
          *reinterpret_cast<float4*>(dp + b * RSZ + pbase) = make_float4(v[b][0], v[b][1], v[b][2], v[b][3]);
        } else {
          *reinterpret_cast<float2*>(dp + b * RSZ + pbase) = make_float2(v[b][0], v[b][1]);
        }
      }
    } else if (uniform) {
#pragma unroll
      for (int b = 0; b < BT; ++b)
#pragma unroll
        for (int e = 0; e < E; ++e) dp[b * RSZ + pbase + e * estride] = v[b][e];
    } else {
#pragma unroll
      for (int b = 0; b < BT; ++b)
#pragma unroll
        for (int e = 0; e < E; ++e) dp[b * RSZ + sw(base + (e << lb))] = v[b][e];
    }
  }
}

// Single-stage pass at a stride of at least 4: a thread takes 4 adjacent pairs (float4 on both
// sides of the stride), so the pass needs a quarter of the items.
template <int BT, bool TRANSPOSE, bool TW_SMEM>
__device__ __forceinline__ void run_pass2_r1w4(const BflyPass pd, const float* src, int src_gate, float* dst,
                                               int dst_gate, const float4* twp, int tw_gate, int tw_l0, int Hpad,
                                               int RSZ, int logn, int ngates = 3, int nthr = NT) {
  const int lb = pd.lb;
  const int lgG = logn - 3;                             // groups of 4 pairs per gate
  const int G = 1 << lgG;
  const int half = Hpad >> 1;
  const int S = 1 << lb;
  for (int item = threadIdx.x; item < ngates * G; item += nthr) {
    const int g = item >> lgG, q = item & (G - 1);
    const int pair = q << 2;                            // first of 4 adjacent pairs
    const int low = pair & (S - 1), high = pair >> lb;
    const int i0 = (high << (lb + 1)) | low;
    const float4* tl = twp + (g * tw_gate + (pd.l0 - tw_l0) * half + q);
    float4 t[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) t[j] = tw_load<TW_SMEM>(tl + (j << lgG));
    const int p0 = sw(i0), p1 = sw(i0 + S);
    const float* sp = src + (size_t)g * src_gate;
    float* dp = dst + (size_t)g * dst_gate;
#pragma unroll
    for (int b = 0; b < BT; ++b) {
      const float4 x0 = *reinterpret_cast<const float4*>(sp + b * RSZ + p0);
      const float4 x1 = *reinterpret_cast<const float4*>(sp + b * RSZ + p1);
      const float a0[4] = {x0.x, x0.y, x0.z, x0.w}, a1[4] = {x1.x, x1.y, x1.z, x1.w};
      float r0[4], r1[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (!TRANSPOSE) {
          r0[j] = fmaf(t[j].y, a1[j], t[j].x * a0[j]);
          r1[j] = fmaf(t[j].z, a0[j], t[j].w * a1[j]);
        } else {
          r0[j] = fmaf(t[j].z, a1[j], t[j].x * a0[j]);
          r1[j] = fmaf(t[j].y, a0[j], t[j].w * a1[j]);
        }
      }
      *reinterpret_cast<float4*>(dp + b * RSZ + p0) = make_float4(r0[0], r0[1], r0[2], r0[3]);
      *reinterpret_cast<float4*>(dp + b * RSZ + p1) = make_float4(r1[0], r1[1], r1[2], r1[3]);
    }
  }
}

template <int BT, bool TRANSPOSE, bool TW_SMEM>
__device__ __forceinline__ void run_pass2_s(const BflyPass pd, const float* src, int src_gate, float* dst,
                                            int dst_gate, const float4* twp, int tw_gate, int tw_l0, int Hpad,
                                            int RSZ, int logn, int ngates = 3, int nthr = NT) {
  if (pd.r == 3) run_pass2_r<3, BT, TRANSPOSE, TW_SMEM>(pd, src, src_gate, dst, dst_gate, twp, tw_gate, tw_l0, Hpad, RSZ, logn, ngates, nthr);
  else if (pd.r == 2) run_pass2_r<2, BT, TRANSPOSE, TW_SMEM>(pd, src, src_gate, dst, dst_gate, twp, tw_gate, tw_l0, Hpad, RSZ, logn, ngates, nthr);
  else if (pd.nst == 1 && pd.lb >= 2 && logn >= 3)
    run_pass2_r1w4<BT, TRANSPOSE, TW_SMEM>(pd, src, src_gate, dst, dst_gate, twp, tw_gate, tw_l0, Hpad, RSZ, logn, ngates, nthr);
  else run_pass2_r<1, BT, TRANSPOSE, TW_SMEM>(pd, src, src_gate, dst, dst_gate, twp, tw_gate, tw_l0, Hpad, RSZ, logn, ngates, nthr);
}

// Twiddle supply shared by the forward and the backward kernel.
struct TwiddleFeed {
  const float4* gtw;      // global twiddles [3][nstages][half]
  float4* buf;            // shared: resident copy, or two streaming buffers of 3 * 3 * half float4
  unsigned bar0;          // streaming: mbarriers of the two buffers (bar0, bar0 + 8)
  int mode;               // 0 global, 1 resident, 2 streamed
  int half, nstages, npasses;
};

// thread 0: start the copies of launch-wide pass number q (pass p of its step) into buffer q & 1
__device__ __forceinline__ void feed_issue(const TwiddleFeed& f, const BflyPass* passes, unsigned q, int p) {
  const int l0 = passes[p].l0, nst = passes[p].nst;
  const unsigned bytes = (unsigned)(nst * f.half) * 16u;
  const unsigned par = q & 1u;
  const unsigned bar = f.bar0 + 8u * par;
  mbar_arm(bar, 3u * bytes);
  const unsigned dst = smem_u32(f.buf) + par * (unsigned)(9 * f.half) * 16u;
  const float4* src = f.gtw + l0 * f.half;
#pragma unroll
  for (int g = 0; g < 3; ++g)
    bulk_load(dst + (unsigned)(g * 3 * f.half) * 16u, src + (size_t)g * f.nstages * f.half, bytes, bar);
}

}  // namespace

// shared memory (floats unless noted), in this order:
//   mbarriers      4 x 8 bytes: twiddle buffer 0 / 1, step operands, spare
//   twiddles       resident: 3*nstages*half float4; streamed: 2*3*3*half float4; global: none
//   st             [3][BT][RSZ]   running vectors of the gates (swizzled rows)
//   hq             [BT][RSZ]      forward: fq_in(h), zero beyond H
//   hraw / opnd    forward: [BT][H] raw h and [3][BT][H] gi;  backward: [6][BT][H] operands,
//                  [BT][H] dh, [BT][H] direct term, [BT][H] mask
//   bias           forward: [3][H]

// TW_SMEM: twiddles come from shared memory (resident or streamed) rather than from global memory
template <int BT, bool TW_SMEM>
__global__ void __launch_bounds__(NT)
bfly_fwd2_kernel(const BflyArgs a) {
  extern __shared__ __align__(128) float smem[];
  // pass table in shared memory: indexing the kernel parameter with a run-time pass number
  // would move the whole argument block to local memory
  __shared__ BflyPass spass[BFLY_MAX_PASSES];
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < BFLY_MAX_PASSES; ++i) spass[i] = a.passes[i];
  }
  __syncthreads();
  const int H = a.H, Hpad = a.Hpad, half = Hpad >> 1, RSZ = a.RSZ, H4g = H >> 2;
  const int row0 = blockIdx.x * BT;
  const int tid = threadIdx.x;
  const int nrows = min(BT, a.B - row0);

  const unsigned bar0 = smem_u32(smem);
  float4* twbuf = reinterpret_cast<float4*>(smem + 8);
  const size_t tw_f4 = a.tw_mode == 1 ? (size_t)3 * a.nstages * half : (a.tw_mode == 2 ? (size_t)2 * 9 * half : 0);
  float* st = smem + 8 + 4 * tw_f4;
  float* hq = st + 3 * BT * RSZ;
  float* hraw = hq + BT * RSZ;
  float* gbuf = hraw + BT * H;
  float* bias = gbuf + 3 * BT * H;
  const unsigned gbar = bar0 + 16;

  TwiddleFeed feed;
  feed.gtw = reinterpret_cast<const float4*>(a.twp);
  feed.buf = twbuf; feed.bar0 = bar0; feed.mode = a.tw_mode; feed.half = half; feed.nstages = a.nstages;
  feed.npasses = a.npasses;
  const unsigned total_passes = (unsigned)a.T * (unsigned)a.npasses;

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;
  const unsigned row_bytes = (unsigned)H * sizeof(float);

  auto issue_gi = [&](int t) {          // thread 0
    mbar_arm(gbar, 3u * nrows * row_bytes);
    for (int g = 0; g < 3; ++g)
      for (int b = 0; b < nrows; ++b)
        bulk_load(smem_u32(gbuf + (g * BT + b) * H),
                  a.gi + (size_t)t * gi_step + (size_t)(row0 + b) * 3 * H + (size_t)g * H, row_bytes, gbar);
  };

  if (tid == 0) {
    mbar_init(bar0); mbar_init(bar0 + 8); mbar_init(gbar);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (feed.mode == 2) {
      feed_issue(feed, spass, 0u, 0);
      if (total_passes > 1) feed_issue(feed, spass, 1u, a.npasses > 1 ? 1 : 0);
    }
    issue_gi(0);
  }
  if (feed.mode == 1) {
    const int n4 = 3 * a.nstages * half;
    for (int i = tid; i < n4; i += NT) twbuf[i] = feed.gtw[i];
  }
  for (int i = tid; i < 3 * H; i += NT) bias[i] = a.bh[i];
  for (int idx = tid; idx < BT * RSZ; idx += NT) hq[idx] = 0.f;
  __syncthreads();
  for (int idx = tid; idx < BT * H; idx += NT) {
    const int b = idx / H, i = idx - b * H;
    const int row = row0 + b;
    float v = 0.f;
    if (row < a.B)
      v = (row < a.h0_rows) ? a.h0[(size_t)row * H + i] : a.h0_tail[(size_t)(row - a.h0_rows) * H + i];
    hraw[idx] = v;
    hq[b * RSZ + sw(i)] = a.qin.enabled ? fake_quant<true>(v, a.qin) : v;
  }
  __syncthreads();

  const float4* twp = feed.mode == 0 ? feed.gtw : twbuf;
  const int tw_gate_res = a.nstages * half;
  bool dead = false;
  unsigned q = 0;

  PHASE_DECL;
  for (int t = 0; t < a.T; ++t) {
    PHASE_START();
    for (int p = 0; p < a.npasses; ++p, ++q) {
      const float4* tp = twp;
      int tgate = tw_gate_res, tl0 = 0;
      if (feed.mode == 2) {
        mbar_wait(bar0 + 8u * (unsigned)(q & 1), (unsigned)(q >> 1) & 1u, dead);
        PHASE_MARK(0);
        tp = twbuf + (size_t)(q & 1) * 9 * half;
        tgate = 3 * half;
        tl0 = spass[p].l0;
      }
      // one call site: every inlined copy of the pass body costs registers across the whole kernel
      run_pass2_s<BT, false, TW_SMEM>(spass[p], p == 0 ? hq : st, p == 0 ? 0 : BT * RSZ, st, BT * RSZ, tp, tgate, tl0,
                                      Hpad, RSZ, a.logn);
      PHASE_MARK(1 + (p < 4 ? p : 4));
      __syncthreads();
      PHASE_MARK(6);
      if (feed.mode == 2 && tid == 0 && q + 2 < total_passes) {
        int p2 = p + 2;
        while (p2 >= a.npasses) p2 -= a.npasses;
        feed_issue(feed, spass, q + 2, p2);
      }
      PHASE_MARK(7);
    }
    mbar_wait(gbar, (unsigned)t & 1u, dead);
    PHASE_MARK(8);

    // gate phase: an item is V adjacent units of one row; narrower items when the row would otherwise
    // leave most of the threads idle (the phase is a chain of transcendental latencies per element)
    auto gate_phase = [&](auto vtag) {
      constexpr int V = decltype(vtag)::value;
      const int HV = H / V;
      for (int idx = tid; idx < nrows * HV; idx += NT) {
        const int b = (BT == 1) ? 0 : idx / HV, i = (idx - b * HV) * V;   // one row: no division on the chain
        const int row = row0 + b;
        const int ps = b * RSZ + sw(i);
        float sr[V], sz[V], sn[V], gr[V], gz[V], gn[V], hv[V], bb[V];
        ldv<V>(st + 0 * BT * RSZ + ps, sr); ldv<V>(bias + i, bb);
#pragma unroll
        for (int v = 0; v < V; ++v) sr[v] += bb[v];
        ldv<V>(st + 1 * BT * RSZ + ps, sz); ldv<V>(bias + H + i, bb);
#pragma unroll
        for (int v = 0; v < V; ++v) sz[v] += bb[v];
        ldv<V>(st + 2 * BT * RSZ + ps, sn); ldv<V>(bias + 2 * H + i, bb);
#pragma unroll
        for (int v = 0; v < V; ++v) sn[v] += bb[v];
        ldv<V>(gbuf + (0 * BT + b) * H + i, gr);
        ldv<V>(gbuf + (1 * BT + b) * H + i, gz);
        ldv<V>(gbuf + (2 * BT + b) * H + i, gn);
        ldv<V>(hraw + b * H + i, hv);
        float hn[V], hqv[V], rr[V], zz[V], nn[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
          const GateOut go = gru_gates(gr[v], gz[v], gn[v], sr[v], sz[v], sn[v], hv[v]);
          hn[v] = a.qout.enabled ? fake_quant<true>(go.h_raw, a.qout) : go.h_raw;
          hqv[v] = a.qin.enabled ? fake_quant<true>(hn[v], a.qin) : hn[v];
          rr[v] = go.r; zz[v] = go.z; nn[v] = go.n;
        }
        const size_t o = (size_t)t * out_step + (size_t)row * H + i;
        if (a.out != nullptr) stv<V, false>(a.out + o, hn);
        if (a.save != nullptr) {
          stv<V, true>(a.save + o, rr);
          stv<V, true>(a.save + comp + o, zz);
          stv<V, true>(a.save + 2 * comp + o, nn);
          stv<V, true>(a.save + 3 * comp + o, sn);
        }
        stv<V, false>(hraw + b * H + i, hn);
        stv<V, false>(hq + ps, hqv);
      }
    };
    if (2 * nrows * H4g <= NT) gate_phase(std::integral_constant<int, 2>{});
    else gate_phase(std::integral_constant<int, 4>{});
    PHASE_MARK(9);
    __syncthreads();
    PHASE_MARK(10);
    if (tid == 0 && t + 1 < a.T) issue_gi(t + 1);
    PHASE_MARK(11);
  }
}

// Two-CTA variant of the forward kernel for hidden sizes whose three gates' twiddles miss one CTA's
// shared memory while two gates' fit (H = 1024): a cluster of two CTAs per batch-row block.  Rank 0
// keeps the twiddles of gates r and z resident and runs their products, rank 1 those of gate n;
// after the passes each hands the other the half of its result vectors that the other's gate
// phase needs (rank 0 owns units [0, H/2), rank 1 units [H/2, H)), both do the gate math of their
// half and write the new fq_in(h) half into both CTAs' copies.  Both hand-overs are st.async stores
// counted on an mbarrier of the receiver (no fence, no cluster barrier inside the time loop: a
// release at a cluster barrier would wait for the step's global stores); a buffer is only written
// again after its reader has sent the data the writer needs first.  No twiddle leaves shared
// memory after the first step.  Same pass functions and gate math as the
// one-CTA kernel, so the results are bit-identical to it.
// shared memory: as bfly_fwd2_kernel with a resident block of 2 * nstages * half twiddles.
template <int BT>
__global__ void __launch_bounds__(NT)
bfly_fwd2_pair_kernel(const BflyArgs a) {
  extern __shared__ __align__(128) float smem[];
  __shared__ BflyPass spass[BFLY_MAX_PASSES];
  cg::cluster_group cluster = cg::this_cluster();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < BFLY_MAX_PASSES; ++i) spass[i] = a.passes[i];
  }
  __syncthreads();
  const int H = a.H, Hpad = a.Hpad, half = Hpad >> 1, RSZ = a.RSZ, Hh = H >> 1;
  const int rank = (int)cluster.block_rank();              // 0: gates r, z; 1: gate n
  const int row0 = (blockIdx.x >> 1) * BT;
  const int tid = threadIdx.x;
  const int nrows = min(BT, a.B - row0);
  const int g0 = rank == 0 ? 0 : 2, ng = rank == 0 ? 2 : 1;  // own gates
  const int u0 = rank * Hh;                                  // own units [u0, u0 + Hh)

  const unsigned bar0 = smem_u32(smem);
  float4* twbuf = reinterpret_cast<float4*>(smem + 8);
  const size_t tw_f4 = (size_t)2 * a.nstages * half;
  float* st = smem + 8 + 4 * tw_f4;
  float* hq = st + 3 * BT * RSZ;
  float* hraw = hq + BT * RSZ;
  float* gbuf = hraw + BT * H;
  float* bias = gbuf + 3 * BT * H;
  const unsigned gbar = bar0 + 16;
  // the peer's copies and mbarriers, as addresses in the cluster's shared window
  const unsigned pbar = bar0, hbar = bar0 + 8;             // products / new h of the peer have landed here
  const unsigned peer_st = map_to_rank(smem_u32(st), (unsigned)(rank ^ 1));
  const unsigned peer_hq = map_to_rank(smem_u32(hq), (unsigned)(rank ^ 1));
  const unsigned peer_pbar = map_to_rank(pbar, (unsigned)(rank ^ 1));
  const unsigned peer_hbar = map_to_rank(hbar, (unsigned)(rank ^ 1));
  const unsigned recv_p = (unsigned)((3 - ng) * nrows * Hh) * 4u;   // bytes per step: the peer's gates, own half
  const unsigned recv_h = (unsigned)(nrows * Hh) * 4u;              // the peer's half of fq_in(h_t)

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;
  const unsigned half_bytes = (unsigned)Hh * sizeof(float);

  auto issue_gi = [&](int t) {          // thread 0: the own half of every gate's row
    mbar_arm(gbar, 3u * nrows * half_bytes);
    for (int g = 0; g < 3; ++g)
      for (int b = 0; b < nrows; ++b)
        bulk_load(smem_u32(gbuf + (g * BT + b) * H + u0),
                  a.gi + (size_t)t * gi_step + (size_t)(row0 + b) * 3 * H + (size_t)g * H + u0, half_bytes, gbar);
  };

  if (tid == 0) {
    mbar_init(pbar); mbar_init(hbar); mbar_init(gbar);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_arm(pbar, recv_p);
    if (a.T > 1) mbar_arm(hbar, recv_h);
    issue_gi(0);
  }
  {
    const float4* gtw = reinterpret_cast<const float4*>(a.twp) + (size_t)g0 * a.nstages * half;
    const int n4 = ng * a.nstages * half;
    for (int i = tid; i < n4; i += NT) twbuf[i] = gtw[i];
  }
  for (int i = tid; i < 3 * H; i += NT) bias[i] = a.bh[i];
  for (int idx = tid; idx < BT * RSZ; idx += NT) hq[idx] = 0.f;
  __syncthreads();
  for (int idx = tid; idx < BT * H; idx += NT) {
    const int b = idx / H, i = idx - b * H;
    const int row = row0 + b;
    float v = 0.f;
    if (row < a.B)
      v = (row < a.h0_rows) ? a.h0[(size_t)row * H + i] : a.h0_tail[(size_t)(row - a.h0_rows) * H + i];
    hraw[idx] = v;
    hq[b * RSZ + sw(i)] = a.qin.enabled ? fake_quant<true>(v, a.qin) : v;
  }
  cluster.sync();            // both CTAs run, their mbarriers are armed, before anything crosses between them

  float* st_own = st + g0 * BT * RSZ;
  const int tw_gate_res = a.nstages * half;
  const int Hh4 = Hh >> 2;
  bool dead = false;

#if defined(B200GRU_PHASE_TIMING) && defined(B200GRU_PHASE_CTA)
  long long ph_last = 0;
  const bool ph_on = (blockIdx.x == B200GRU_PHASE_CTA && threadIdx.x == 0);     // time the other rank of the pair
#else
  PHASE_DECL;
#endif
  for (int t = 0; t < a.T; ++t) {
    PHASE_START();
    for (int p = 0; p < a.npasses; ++p) {
      run_pass2_s<BT, false, true>(spass[p], p == 0 ? hq : st_own, p == 0 ? 0 : BT * RSZ, st_own, BT * RSZ, twbuf,
                                   tw_gate_res, 0, Hpad, RSZ, a.logn, ng, NT);
      PHASE_MARK(p < 4 ? p : 4);
      __syncthreads();
      PHASE_MARK(5);
    }
    // hand the peer's half of the own result vectors over (float4 runs of the swizzled rows); the
    // stores count their bytes on the peer's mbarrier, so nobody fences or meets at a barrier
    for (int g = 0; g < ng; ++g)
      for (int b = 0; b < nrows; ++b)
        for (int j = tid; j < Hh4; j += NT) {               // no division on the chain
          const int i = (Hh - u0) + j * 4;                  // a unit of the peer's half
          const int off = ((g0 + g) * BT + b) * RSZ + sw(i);
          const float4 v = *reinterpret_cast<const float4*>(st + off);
          st_async_v4(peer_st + 4u * (unsigned)off, v, peer_pbar);
        }
    PHASE_MARK(6);
    mbar_wait(pbar, (unsigned)t & 1u, dead);
    if (tid == 0 && t + 1 < a.T) mbar_arm(pbar, recv_p);
    PHASE_MARK(7);
    mbar_wait(gbar, (unsigned)t & 1u, dead);
    PHASE_MARK(8);

    auto gate_phase = [&](auto vtag) {
      constexpr int V = decltype(vtag)::value;
      const int HV = Hh / V;
      for (int b = 0; b < nrows; ++b)
      for (int j = tid; j < HV; j += NT) {
        const int i = u0 + j * V;
        const int row = row0 + b;
        const int ps = b * RSZ + sw(i);
        float sr[V], sz[V], sn[V], gr[V], gz[V], gn[V], hv[V], bb[V];
        ldv<V>(st + 0 * BT * RSZ + ps, sr); ldv<V>(bias + i, bb);
#pragma unroll
        for (int v = 0; v < V; ++v) sr[v] += bb[v];
        ldv<V>(st + 1 * BT * RSZ + ps, sz); ldv<V>(bias + H + i, bb);
#pragma unroll
        for (int v = 0; v < V; ++v) sz[v] += bb[v];
        ldv<V>(st + 2 * BT * RSZ + ps, sn); ldv<V>(bias + 2 * H + i, bb);
#pragma unroll
        for (int v = 0; v < V; ++v) sn[v] += bb[v];
        ldv<V>(gbuf + (0 * BT + b) * H + i, gr);
        ldv<V>(gbuf + (1 * BT + b) * H + i, gz);
        ldv<V>(gbuf + (2 * BT + b) * H + i, gn);
        ldv<V>(hraw + b * H + i, hv);
        float hn[V], hqv[V], rr[V], zz[V], nn[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
          const GateOut go = gru_gates(gr[v], gz[v], gn[v], sr[v], sz[v], sn[v], hv[v]);
          hn[v] = a.qout.enabled ? fake_quant<true>(go.h_raw, a.qout) : go.h_raw;
          hqv[v] = a.qin.enabled ? fake_quant<true>(hn[v], a.qin) : hn[v];
          rr[v] = go.r; zz[v] = go.z; nn[v] = go.n;
        }
        const size_t o = (size_t)t * out_step + (size_t)row * H + i;
        if (a.out != nullptr) stv<V, false>(a.out + o, hn);
        if (a.save != nullptr) {
          stv<V, true>(a.save + o, rr);
          stv<V, true>(a.save + comp + o, zz);
          stv<V, true>(a.save + 2 * comp + o, nn);
          stv<V, true>(a.save + 3 * comp + o, sn);
        }
        stv<V, false>(hraw + b * H + i, hn);
        stv<V, false>(hq + ps, hqv);
        if (t + 1 < a.T) st_async_v<V>(peer_hq + 4u * (unsigned)ps, hqv, peer_hbar);
      }
    };
    if (2 * nrows * Hh4 <= NT) gate_phase(std::integral_constant<int, 2>{});
    else gate_phase(std::integral_constant<int, 4>{});
    PHASE_MARK(9);
    __syncthreads();         // own half of fq_in(h_t) is in place; gbuf and the result vectors are free again
    if (t + 1 < a.T) {
      if (tid == 0) issue_gi(t + 1);
      mbar_wait(hbar, (unsigned)t & 1u, dead);             // the peer's half
      if (tid == 0 && t + 2 < a.T) mbar_arm(hbar, recv_h);
    }
    PHASE_MARK(10);
  }
  cluster.sync();            // nobody leaves while the peer could still address its shared memory
}

template <int BT, bool TW_SMEM>
__global__ void __launch_bounds__(NT)
bfly_bwd2_kernel(const BflyArgs a) {
  extern __shared__ __align__(128) float smem[];
  // pass table in shared memory: indexing the kernel parameter with a run-time pass number
  // would move the whole argument block to local memory
  __shared__ BflyPass spass[BFLY_MAX_PASSES];
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < BFLY_MAX_PASSES; ++i) spass[i] = a.passes[i];
  }
  __syncthreads();
  const int H = a.H, Hpad = a.Hpad, half = Hpad >> 1, RSZ = a.RSZ, H4g = H >> 2, P4g = Hpad >> 2;
  const int row0 = blockIdx.x * BT;
  const int tid = threadIdx.x;
  const int nrows = min(BT, a.B - row0);

  const unsigned bar0 = smem_u32(smem);
  float4* twbuf = reinterpret_cast<float4*>(smem + 8);
  const size_t tw_f4 = a.tw_mode == 1 ? (size_t)3 * a.nstages * half : (a.tw_mode == 2 ? (size_t)2 * 9 * half : 0);
  float* st = smem + 8 + 4 * tw_f4;
  float* pbuf = st + 3 * BT * RSZ;       // [6][BT][H]: dout, r, z, n, gh_n, h_prev
  float* dhacc = pbuf + 6 * BT * H;
  float* dhdir = dhacc + BT * H;
  float* mk = dhdir + BT * H;
  const unsigned pbar = bar0 + 16;

  TwiddleFeed feed;
  feed.gtw = reinterpret_cast<const float4*>(a.twp);
  feed.buf = twbuf; feed.bar0 = bar0; feed.mode = a.tw_mode; feed.half = half; feed.nstages = a.nstages;
  feed.npasses = a.npasses;
  const unsigned total_passes = (unsigned)a.T * (unsigned)a.npasses;

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;
  const unsigned row_bytes = (unsigned)H * sizeof(float);

  auto issue_operands = [&](int t) {    // thread 0
    mbar_arm(pbar, 6u * nrows * row_bytes);
    for (int c = 0; c < 6; ++c)
      for (int b = 0; b < nrows; ++b) {
        const size_t o = (size_t)t * out_step + (size_t)(row0 + b) * H;
        const float* src;
        if (c == 0) src = a.dout + o;
        else if (c <= 4) src = a.S + (size_t)(c - 1) * comp + o;
        else src = (t > 0) ? (a.out_c + o - out_step) : (a.h0 + (size_t)(row0 + b) * H);
        bulk_load(smem_u32(pbuf + (c * BT + b) * H), src, row_bytes, pbar);
      }
  };

  if (tid == 0) {
    mbar_init(bar0); mbar_init(bar0 + 8); mbar_init(pbar);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (feed.mode == 2) {
      feed_issue(feed, spass, 0u, a.npasses - 1);
      if (total_passes > 1) feed_issue(feed, spass, 1u, a.npasses > 1 ? a.npasses - 2 : 0);
    }
    issue_operands(a.T - 1);
  }
  if (feed.mode == 1) {
    const int n4 = 3 * a.nstages * half;
    for (int i = tid; i < n4; i += NT) twbuf[i] = feed.gtw[i];
  }
  for (int idx = tid; idx < BT * H; idx += NT) dhacc[idx] = 0.f;
  for (int idx = tid; idx < 3 * BT * RSZ; idx += NT) st[idx] = 0.f;
  __syncthreads();

  const float4* twp = feed.mode == 0 ? feed.gtw : twbuf;
  const int tw_gate_res = a.nstages * half;
  bool dead = false;
  unsigned q = 0;

  for (int t = a.T - 1; t >= 0; --t) {
    mbar_wait(pbar, (unsigned)(a.T - 1 - t) & 1u, dead);

    // gate gradients -> st (and zero the padded tail, which the transposed passes dirty)
    for (int idx = tid; idx < nrows * P4g; idx += NT) {
      const int b = (BT == 1) ? 0 : idx / P4g, i = (idx - b * P4g) << 2;
      const int row = row0 + b;
      const int ps = b * RSZ + sw(i);
      float x0[4] = {0.f, 0.f, 0.f, 0.f}, x1[4] = {0.f, 0.f, 0.f, 0.f}, x2[4] = {0.f, 0.f, 0.f, 0.f};
      if (i < H) {
        const int e = b * H + i;
        const float4 d4 = *reinterpret_cast<const float4*>(pbuf + 0 * BT * H + e);
        const float4 r4 = *reinterpret_cast<const float4*>(pbuf + 1 * BT * H + e);
        const float4 z4 = *reinterpret_cast<const float4*>(pbuf + 2 * BT * H + e);
        const float4 n4 = *reinterpret_cast<const float4*>(pbuf + 3 * BT * H + e);
        const float4 g4 = *reinterpret_cast<const float4*>(pbuf + 4 * BT * H + e);
        const float4 h4 = *reinterpret_cast<const float4*>(pbuf + 5 * BT * H + e);
        const float4 a4 = *reinterpret_cast<const float4*>(dhacc + e);
        const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
        const float zz[4] = {z4.x, z4.y, z4.z, z4.w}, nn[4] = {n4.x, n4.y, n4.z, n4.w};
        const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, hh[4] = {h4.x, h4.y, h4.z, h4.w};
        const float aa[4] = {a4.x, a4.y, a4.z, a4.w};
        float dir[4], msk[4], dgn[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          float dh = dd[v] + aa[v];
          if (a.qout.enabled) {
            const float h_raw = (1.0f - zz[v]) * nn[v] + zz[v] * hh[v];
            dh = dh * ste_mask<true>(h_raw, a.qout);
          }
          const GateGrad q4 = gru_gate_grads(dh, rr[v], zz[v], nn[v], gg[v], hh[v]);
          dir[v] = q4.dh_direct;
          msk[v] = a.qin.enabled ? ste_mask<true>(hh[v], a.qin) : 1.0f;
          x0[v] = q4.dgr; x1[v] = q4.dgz; x2[v] = q4.dghn; dgn[v] = q4.dgn;
        }
        *reinterpret_cast<float4*>(dhdir + e) = make_float4(dir[0], dir[1], dir[2], dir[3]);
        *reinterpret_cast<float4*>(mk + e) = make_float4(msk[0], msk[1], msk[2], msk[3]);
        float* d = a.dgi + (size_t)t * gi_step + (size_t)row * 3 * H + i;
        __stcs(reinterpret_cast<float4*>(d), make_float4(x0[0], x0[1], x0[2], x0[3]));
        __stcs(reinterpret_cast<float4*>(d + H), make_float4(x1[0], x1[1], x1[2], x1[3]));
        __stcs(reinterpret_cast<float4*>(d + 2 * H), make_float4(dgn[0], dgn[1], dgn[2], dgn[3]));
      }
      *reinterpret_cast<float4*>(st + 0 * BT * RSZ + ps) = make_float4(x0[0], x0[1], x0[2], x0[3]);
      *reinterpret_cast<float4*>(st + 1 * BT * RSZ + ps) = make_float4(x1[0], x1[1], x1[2], x1[3]);
      *reinterpret_cast<float4*>(st + 2 * BT * RSZ + ps) = make_float4(x2[0], x2[1], x2[2], x2[3]);
    }
    __syncthreads();
    if (tid == 0 && t > 0) issue_operands(t - 1);

    for (int p = a.npasses - 1; p >= 0; --p, ++q) {
      const float4* tp = twp;
      int tgate = tw_gate_res, tl0 = 0;
      if (feed.mode == 2) {
        mbar_wait(bar0 + 8u * (unsigned)(q & 1), (unsigned)(q >> 1) & 1u, dead);
        tp = twbuf + (size_t)(q & 1) * 9 * half;
        tgate = 3 * half;
        tl0 = spass[p].l0;
      }
      run_pass2_s<BT, true, TW_SMEM>(spass[p], st, BT * RSZ, st, BT * RSZ, tp, tgate, tl0, Hpad, RSZ, a.logn);
      __syncthreads();
      if (feed.mode == 2 && tid == 0 && q + 2 < total_passes) {
        int p2 = p - 2;
        while (p2 < 0) p2 += a.npasses;
        feed_issue(feed, spass, q + 2, p2);
      }
    }

    for (int idx = tid; idx < nrows * H4g; idx += NT) {
      const int b = (BT == 1) ? 0 : idx / H4g, i = (idx - b * H4g) << 2;
      const int ps = b * RSZ + sw(i);
      const int e = b * H + i;
      const float4 s0 = *reinterpret_cast<const float4*>(st + 0 * BT * RSZ + ps);
      const float4 s1 = *reinterpret_cast<const float4*>(st + 1 * BT * RSZ + ps);
      const float4 s2 = *reinterpret_cast<const float4*>(st + 2 * BT * RSZ + ps);
      const float4 dr = *reinterpret_cast<const float4*>(dhdir + e);
      const float4 m4 = *reinterpret_cast<const float4*>(mk + e);
      float4 r;
      r.x = dr.x + (s0.x + s1.x + s2.x) * m4.x;
      r.y = dr.y + (s0.y + s1.y + s2.y) * m4.y;
      r.z = dr.z + (s0.z + s1.z + s2.z) * m4.z;
      r.w = dr.w + (s0.w + s1.w + s2.w) * m4.w;
      *reinterpret_cast<float4*>(dhacc + e) = r;
    }
    __syncthreads();
  }

  for (int idx = tid; idx < nrows * H4g; idx += NT) {
    const int b = idx / H4g, i = (idx - b * H4g) << 2;
    *reinterpret_cast<float4*>(a.dh0 + (size_t)(row0 + b) * H + i) = *reinterpret_cast<const float4*>(dhacc + b * H + i);
  }
}

// Two-CTA variant of the backward kernel, for the same problems as bfly_fwd2_pair_kernel.  Both CTAs
// of a pair load the step's operands and compute the gate gradients of all units (elementwise, so
// the full vectors dgh_g exist in both without an exchange); rank 0 stores dgi_r, dgi_z and runs
// the transposed products of gates r and z from resident twiddles, rank 1 does the same for gate n.
// After the passes rank 0 sends s_r + s_z and rank 1 s_n (st.async stores counted on an mbarrier of
// the receiver, into a buffer that alternates with the step), and both form
// dh = direct + ((s_r + s_z) + s_n) * mask in the order of the one-CTA kernel: bit-identical results.
template <int BT>
__global__ void __launch_bounds__(NT)
bfly_bwd2_pair_kernel(const BflyArgs a) {
  extern __shared__ __align__(128) float smem[];
  __shared__ BflyPass spass[BFLY_MAX_PASSES];
  cg::cluster_group cluster = cg::this_cluster();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < BFLY_MAX_PASSES; ++i) spass[i] = a.passes[i];
  }
  __syncthreads();
  const int H = a.H, Hpad = a.Hpad, half = Hpad >> 1, RSZ = a.RSZ, H4g = H >> 2, P4g = Hpad >> 2;
  const int rank = (int)cluster.block_rank();              // 0: gates r, z; 1: gate n
  const int row0 = (blockIdx.x >> 1) * BT;
  const int tid = threadIdx.x;
  const int nrows = min(BT, a.B - row0);
  const int g0 = rank == 0 ? 0 : 2, ng = rank == 0 ? 2 : 1;

  const unsigned bar0 = smem_u32(smem);
  float4* twbuf = reinterpret_cast<float4*>(smem + 8);
  const size_t tw_f4 = (size_t)2 * a.nstages * half;
  float* st = smem + 8 + 4 * tw_f4;
  float* pbuf = st + 3 * BT * RSZ;       // [6][BT][H]: dout, r, z, n, gh_n, h_prev
  float* dhacc = pbuf + 6 * BT * H;
  float* dhdir = dhacc + BT * H;
  float* mk = dhdir + BT * H;
  float* recv = mk + BT * H;             // [2][BT][H]: the peer's partial sum, buffer = step parity
  const unsigned xbar = bar0, pbar = bar0 + 16;
  const unsigned peer_recv = map_to_rank(smem_u32(recv), (unsigned)(rank ^ 1));
  const unsigned peer_xbar = map_to_rank(xbar, (unsigned)(rank ^ 1));
  const unsigned recv_bytes = (unsigned)(nrows * H) * 4u;

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;
  const unsigned row_bytes = (unsigned)H * sizeof(float);

  auto issue_operands = [&](int t) {    // thread 0
    mbar_arm(pbar, 6u * nrows * row_bytes);
    for (int c = 0; c < 6; ++c)
      for (int b = 0; b < nrows; ++b) {
        const size_t o = (size_t)t * out_step + (size_t)(row0 + b) * H;
        const float* src;
        if (c == 0) src = a.dout + o;
        else if (c <= 4) src = a.S + (size_t)(c - 1) * comp + o;
        else src = (t > 0) ? (a.out_c + o - out_step) : (a.h0 + (size_t)(row0 + b) * H);
        bulk_load(smem_u32(pbuf + (c * BT + b) * H), src, row_bytes, pbar);
      }
  };

  if (tid == 0) {
    mbar_init(xbar); mbar_init(pbar);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_arm(xbar, recv_bytes);
    issue_operands(a.T - 1);
  }
  {
    const float4* gtw = reinterpret_cast<const float4*>(a.twp) + (size_t)g0 * a.nstages * half;
    const int n4 = ng * a.nstages * half;
    for (int i = tid; i < n4; i += NT) twbuf[i] = gtw[i];
  }
  for (int idx = tid; idx < BT * H; idx += NT) dhacc[idx] = 0.f;
  for (int idx = tid; idx < 3 * BT * RSZ; idx += NT) st[idx] = 0.f;
  cluster.sync();            // both CTAs run and their mbarriers are armed before anything crosses

  float* st_own = st + g0 * BT * RSZ;
  const int tw_gate_res = a.nstages * half;
  bool dead = false;

  for (int t = a.T - 1; t >= 0; --t) {
    const unsigned par = (unsigned)(a.T - 1 - t) & 1u;
    mbar_wait(pbar, par, dead);

    // gate gradients of all units; the own gates' dgh go to st (padded tail zeroed: the transposed
    // passes dirty it), the own gates' dgi to global memory
    for (int idx = tid; idx < nrows * P4g; idx += NT) {
      const int b = (BT == 1) ? 0 : idx / P4g, i = (idx - b * P4g) << 2;
      const int row = row0 + b;
      const int ps = b * RSZ + sw(i);
      float x0[4] = {0.f, 0.f, 0.f, 0.f}, x1[4] = {0.f, 0.f, 0.f, 0.f}, x2[4] = {0.f, 0.f, 0.f, 0.f};
      if (i < H) {
        const int e = b * H + i;
        const float4 d4 = *reinterpret_cast<const float4*>(pbuf + 0 * BT * H + e);
        const float4 r4 = *reinterpret_cast<const float4*>(pbuf + 1 * BT * H + e);
        const float4 z4 = *reinterpret_cast<const float4*>(pbuf + 2 * BT * H + e);
        const float4 n4 = *reinterpret_cast<const float4*>(pbuf + 3 * BT * H + e);
        const float4 g4 = *reinterpret_cast<const float4*>(pbuf + 4 * BT * H + e);
        const float4 h4 = *reinterpret_cast<const float4*>(pbuf + 5 * BT * H + e);
        const float4 a4 = *reinterpret_cast<const float4*>(dhacc + e);
        const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
        const float zz[4] = {z4.x, z4.y, z4.z, z4.w}, nn[4] = {n4.x, n4.y, n4.z, n4.w};
        const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, hh[4] = {h4.x, h4.y, h4.z, h4.w};
        const float aa[4] = {a4.x, a4.y, a4.z, a4.w};
        float dir[4], msk[4], dgn[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          float dh = dd[v] + aa[v];
          if (a.qout.enabled) {
            const float h_raw = (1.0f - zz[v]) * nn[v] + zz[v] * hh[v];
            dh = dh * ste_mask<true>(h_raw, a.qout);
          }
          const GateGrad q4 = gru_gate_grads(dh, rr[v], zz[v], nn[v], gg[v], hh[v]);
          dir[v] = q4.dh_direct;
          msk[v] = a.qin.enabled ? ste_mask<true>(hh[v], a.qin) : 1.0f;
          x0[v] = q4.dgr; x1[v] = q4.dgz; x2[v] = q4.dghn; dgn[v] = q4.dgn;
        }
        *reinterpret_cast<float4*>(dhdir + e) = make_float4(dir[0], dir[1], dir[2], dir[3]);
        *reinterpret_cast<float4*>(mk + e) = make_float4(msk[0], msk[1], msk[2], msk[3]);
        float* d = a.dgi + (size_t)t * gi_step + (size_t)row * 3 * H + i;
        if (rank == 0) {
          __stcs(reinterpret_cast<float4*>(d), make_float4(x0[0], x0[1], x0[2], x0[3]));
          __stcs(reinterpret_cast<float4*>(d + H), make_float4(x1[0], x1[1], x1[2], x1[3]));
        } else {
          __stcs(reinterpret_cast<float4*>(d + 2 * H), make_float4(dgn[0], dgn[1], dgn[2], dgn[3]));
        }
      }
      if (rank == 0) {
        *reinterpret_cast<float4*>(st + 0 * BT * RSZ + ps) = make_float4(x0[0], x0[1], x0[2], x0[3]);
        *reinterpret_cast<float4*>(st + 1 * BT * RSZ + ps) = make_float4(x1[0], x1[1], x1[2], x1[3]);
      } else {
        *reinterpret_cast<float4*>(st + 2 * BT * RSZ + ps) = make_float4(x2[0], x2[1], x2[2], x2[3]);
      }
    }
    __syncthreads();
    if (tid == 0 && t > 0) issue_operands(t - 1);

    for (int p = a.npasses - 1; p >= 0; --p) {
      run_pass2_s<BT, true, true>(spass[p], st_own, BT * RSZ, st_own, BT * RSZ, twbuf, tw_gate_res, 0, Hpad, RSZ,
                                  a.logn, ng, NT);
      __syncthreads();
    }

    // the own partial sum of every unit goes to the peer's buffer of this step's parity
    for (int idx = tid; idx < nrows * H4g; idx += NT) {
      const int b = (BT == 1) ? 0 : idx / H4g, i = (idx - b * H4g) << 2;
      const int ps = b * RSZ + sw(i);
      float4 v;
      if (rank == 0) {
        const float4 s0 = *reinterpret_cast<const float4*>(st + 0 * BT * RSZ + ps);
        const float4 s1 = *reinterpret_cast<const float4*>(st + 1 * BT * RSZ + ps);
        v = make_float4(s0.x + s1.x, s0.y + s1.y, s0.z + s1.z, s0.w + s1.w);
      } else {
        v = *reinterpret_cast<const float4*>(st + 2 * BT * RSZ + ps);
      }
      st_async_v4(peer_recv + 4u * (unsigned)((par * BT + b) * H + i), v, peer_xbar);
    }
    mbar_wait(xbar, par, dead);
    if (tid == 0 && t > 0) mbar_arm(xbar, recv_bytes);

    const float* rc = recv + par * BT * H;
    for (int idx = tid; idx < nrows * H4g; idx += NT) {
      const int b = (BT == 1) ? 0 : idx / H4g, i = (idx - b * H4g) << 2;
      const int ps = b * RSZ + sw(i);
      const int e = b * H + i;
      const float4 pr = *reinterpret_cast<const float4*>(rc + e);
      float4 s01, s2;
      if (rank == 0) {
        const float4 s0 = *reinterpret_cast<const float4*>(st + 0 * BT * RSZ + ps);
        const float4 s1 = *reinterpret_cast<const float4*>(st + 1 * BT * RSZ + ps);
        s01 = make_float4(s0.x + s1.x, s0.y + s1.y, s0.z + s1.z, s0.w + s1.w);
        s2 = pr;
      } else {
        s01 = pr;
        s2 = *reinterpret_cast<const float4*>(st + 2 * BT * RSZ + ps);
      }
      const float4 dr = *reinterpret_cast<const float4*>(dhdir + e);
      const float4 m4 = *reinterpret_cast<const float4*>(mk + e);
      float4 r;
      r.x = dr.x + (s01.x + s2.x) * m4.x;
      r.y = dr.y + (s01.y + s2.y) * m4.y;
      r.z = dr.z + (s01.z + s2.z) * m4.z;
      r.w = dr.w + (s01.w + s2.w) * m4.w;
      *reinterpret_cast<float4*>(dhacc + e) = r;
    }
    __syncthreads();
  }

  if (rank == 0) {
    for (int idx = tid; idx < nrows * H4g; idx += NT) {
      const int b = (BT == 1) ? 0 : idx / H4g, i = (idx - b * H4g) << 2;
      *reinterpret_cast<float4*>(a.dh0 + (size_t)(row0 + b) * H + i) = *reinterpret_cast<const float4*>(dhacc + b * H + i);
    }
  }
  cluster.sync();            // nobody leaves while the peer could still address its shared memory
}


// ---------------------------------------------------------------------------
// twiddle gradients: dt[g][l][pair][m_new][m_old] = sum over rows (t, b) of d_new[m_new] * old[m_old]
// ---------------------------------------------------------------------------
// Rows are independent here (every h_{t-1} and every dgh_t is known), so the grid is
// (row splits, 3 gates).  A CTA keeps its gate's twiddles and one accumulator per twiddle in shared
// memory.  Per batch of RB rows it runs the forward passes, keeping the input vector of every pass,
// then walks the passes backwards: a thread re-runs the stages of its item in registers (so the
// inputs of the inner stages never touch memory), forms the four products of each of its pairs,
// sums them over the rows of the batch in registers and adds them to the shared accumulators once
// per batch, and pushes d through the transposed stages.  Every (stage, pair) belongs to exactly
// one thread, and the split partials are added in a fixed order afterwards: no atomics.
constexpr int WG_NT = 128;

template <int R, int P>
__device__ __forceinline__ void wgrad_stage(float (&d)[1 << R], const float (&in)[1 << R],
                                            const float4 (&tw)[(1 << R) / 2], float4 (&g)[(1 << R) / 2]) {
  int idx = 0;
#pragma unroll
  for (int e = 0; e < (1 << R); ++e) {
    if (e & (1 << P)) continue;
    const float4 t = tw[idx];
    const float d0 = d[e], d1 = d[e | (1 << P)];
    const float o0 = in[e], o1 = in[e | (1 << P)];
    g[idx].x = fmaf(d0, o0, g[idx].x); g[idx].y = fmaf(d0, o1, g[idx].y);
    g[idx].z = fmaf(d1, o0, g[idx].z); g[idx].w = fmaf(d1, o1, g[idx].w);
    d[e] = fmaf(t.z, d1, t.x * d0);
    d[e | (1 << P)] = fmaf(t.y, d0, t.w * d1);
    ++idx;
  }
}

template <int R>
__device__ __forceinline__ void wgrad_stage_dispatch(float (&d)[1 << R], const float (&in)[1 << R],
                                                     const float4 (&tw)[(1 << R) / 2], float4 (&g)[(1 << R) / 2], int p) {
  if (R >= 3 && p == 2) wgrad_stage<R, (R >= 3 ? 2 : 0)>(d, in, tw, g);
  else if (R >= 2 && p == 1) wgrad_stage<R, (R >= 2 ? 1 : 0)>(d, in, tw, g);
  else wgrad_stage<R, 0>(d, in, tw, g);
}

// One pass (NST stages spanning R adjacent stride bits) of the backward walk for the rows
// [0, nrows) of the batch.  xin: the pass's input vectors [RB][RSZ]; dv: gradient w.r.t. the pass's
// output on entry, w.r.t. its input on return.
template <int R, int NST>
__device__ __forceinline__ void wgrad_pass_r(const BflyPass pd, const float* xin, float* dv, int nrows,
                                             const float4* twsm, float4* acc, int Hpad, int RSZ, int logn) {
  constexpr int E = 1 << R;
  const int lb = pd.lb;
  const int lgG = logn - R;
  const int G = 1 << lgG;
  const int half = Hpad >> 1;
  const int pb0 = pd.pb[0], pb1 = pd.pb[1], pb2 = pd.pb[2];
  const bool w4 = pd.r < 2 && pd.nst == 1 && pd.lb >= 2 && logn >= 3;
  const bool uniform = (lb + R <= 6) || (lb >= 6);
  const int estride = (lb >= 6) ? ((1 << lb) + (8 << (lb - 6))) : (1 << lb);
  for (int q = threadIdx.x; q < G; q += WG_NT) {
    const int low = q & ((1 << lb) - 1), high = q >> lb;
    const int base = (high << (lb + R)) | low;
    float4 t[NST][E / 2], g[NST][E / 2];            // twiddles and accumulators in the permuted order
    // a lone stage at stride >= 4 is stored for the 4-pairs-per-thread forward pass: pair p sits at
    // (p & 3) * (half / 4) + (p >> 2)
    const int tpos = (R == 1 && w4) ? ((q & 3) * (half >> 2) + (q >> 2)) : q;
#pragma unroll
    for (int s = 0; s < NST; ++s) {
      const float4* tl = twsm + ((pd.l0 + s) * half + tpos);
#pragma unroll
      for (int idx = 0; idx < E / 2; ++idx) {
        t[s][idx] = tl[idx << lgG];
        g[s][idx] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const int pbase = sw(base);
    int off[E];
#pragma unroll
    for (int e = 0; e < E; ++e) off[e] = uniform ? pbase + e * estride : sw(base + (e << lb));

#pragma unroll 1
    for (int b = 0; b < nrows; ++b) {
      float v[1][E], d[E], in[NST][E];
      if (E == 8 && lb == 0) {                     // 8 adjacent positions: two float4 per vector
        const float4 x0 = *reinterpret_cast<const float4*>(xin + b * RSZ + pbase);
        const float4 x1 = *reinterpret_cast<const float4*>(xin + b * RSZ + pbase + 4);
        const float4 d0 = *reinterpret_cast<const float4*>(dv + b * RSZ + pbase);
        const float4 d1 = *reinterpret_cast<const float4*>(dv + b * RSZ + pbase + 4);
        const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        const float ds[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
        for (int e = 0; e < E; ++e) { v[0][e] = xs[e & 7]; d[e] = ds[e & 7]; }
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) { v[0][e] = xin[b * RSZ + off[e]]; d[e] = dv[b * RSZ + off[e]]; }
      }
#pragma unroll
      for (int s = 0; s < NST; ++s) {
#pragma unroll
        for (int e = 0; e < E; ++e) in[s][e] = v[0][e];
        if (s + 1 < NST) stage_dispatch<R, 1, false>(v, t[s], s == 0 ? pb0 : pb1);
      }
      if (NST >= 3) wgrad_stage_dispatch<R>(d, in[NST >= 3 ? 2 : 0], t[NST >= 3 ? 2 : 0], g[NST >= 3 ? 2 : 0], pb2);
      if (NST >= 2) wgrad_stage_dispatch<R>(d, in[NST >= 2 ? 1 : 0], t[NST >= 2 ? 1 : 0], g[NST >= 2 ? 1 : 0], pb1);
      wgrad_stage_dispatch<R>(d, in[0], t[0], g[0], pb0);
      if (E == 8 && lb == 0) {
        *reinterpret_cast<float4*>(dv + b * RSZ + pbase) = make_float4(d[0], d[1], d[2 % E], d[3 % E]);
        *reinterpret_cast<float4*>(dv + b * RSZ + pbase + 4) = make_float4(d[4 % E], d[5 % E], d[6 % E], d[7 % E]);
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) dv[b * RSZ + off[e]] = d[e];
      }
    }
#pragma unroll
    for (int s = 0; s < NST; ++s) {
      float4* al = acc + ((pd.l0 + s) * half + tpos);
#pragma unroll
      for (int idx = 0; idx < E / 2; ++idx) {
        float4 c = al[idx << lgG];
        c.x += g[s][idx].x; c.y += g[s][idx].y; c.z += g[s][idx].z; c.w += g[s][idx].w;
        al[idx << lgG] = c;
      }
    }
  }
}

__device__ __forceinline__ void wgrad_pass(const BflyPass pd, const float* xin, float* dv, int nrows,
                                           const float4* twsm, float4* acc, int Hpad, int RSZ, int logn) {
  // a pass of span r has at least r stages (the stride moves by at most one bit per stage)
  if (pd.r == 3) wgrad_pass_r<3, 3>(pd, xin, dv, nrows, twsm, acc, Hpad, RSZ, logn);
  else if (pd.r == 2 && pd.nst == 3) wgrad_pass_r<2, 3>(pd, xin, dv, nrows, twsm, acc, Hpad, RSZ, logn);
  else if (pd.r == 2) wgrad_pass_r<2, 2>(pd, xin, dv, nrows, twsm, acc, Hpad, RSZ, logn);
  else if (pd.nst == 3) wgrad_pass_r<1, 3>(pd, xin, dv, nrows, twsm, acc, Hpad, RSZ, logn);
  else if (pd.nst == 2) wgrad_pass_r<1, 2>(pd, xin, dv, nrows, twsm, acc, Hpad, RSZ, logn);
  else wgrad_pass_r<1, 1>(pd, xin, dv, nrows, twsm, acc, Hpad, RSZ, logn);
}

// shared memory: twiddles [ns][half] float4 | accumulators [ns][half] float4 |
//                pass inputs [npasses][RB][RSZ] | d [RB][RSZ]
template <int RB>
__global__ void __launch_bounds__(WG_NT)
bfly_wgrad2_kernel(const BflyArgs a, float* __restrict__ partial, int rows_per_split) {
  extern __shared__ __align__(128) float smem[];
  __shared__ BflyPass spass[BFLY_MAX_PASSES];
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < BFLY_MAX_PASSES; ++i) spass[i] = a.passes[i];
  }
  const int H = a.H, Hpad = a.Hpad, half = Hpad >> 1, ns = a.nstages, RSZ = a.RSZ, P4 = Hpad >> 2;
  const int TB = a.T * a.B;
  const int g = blockIdx.y;
  const int r_begin = blockIdx.x * rows_per_split;
  const int r_end = min(TB, r_begin + rows_per_split);
  const int tid = threadIdx.x;
  const int nacc = ns * half;

  float4* twsm = reinterpret_cast<float4*>(smem);
  float4* acc = twsm + nacc;
  float* bnd = reinterpret_cast<float*>(acc + nacc);
  float* dvec = bnd + (size_t)a.npasses * RB * RSZ;
  const float4* twg = reinterpret_cast<const float4*>(a.twp) + (size_t)g * nacc;
  for (int i = tid; i < nacc; i += WG_NT) {
    twsm[i] = twg[i];
    acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int i = tid; i < (a.npasses + 1) * RB * RSZ; i += WG_NT) bnd[i] = 0.f;     // includes dvec
  __syncthreads();

  for (int r0 = r_begin; r0 < r_end; r0 += RB) {
    const int nrows = min(RB, r_end - r0);
#pragma unroll 4
    for (int idx = tid; idx < RB * P4; idx += WG_NT) {
      const int b = idx >> (a.logn - 2), i = (idx & (P4 - 1)) << 2;     // P4 = Hpad / 4, a power of two
      const int tb = r0 + b;
      float4 hv = make_float4(0.f, 0.f, 0.f, 0.f), dv = hv;
      if (b < nrows && i < H) {
        hv = (tb < a.B) ? *reinterpret_cast<const float4*>(a.h0 + (size_t)tb * H + i)
                        : *reinterpret_cast<const float4*>(a.out_c + (size_t)(tb - a.B) * H + i);
        if (a.qin.enabled) {
          hv.x = fake_quant<true>(hv.x, a.qin); hv.y = fake_quant<true>(hv.y, a.qin);
          hv.z = fake_quant<true>(hv.z, a.qin); hv.w = fake_quant<true>(hv.w, a.qin);
        }
        dv = __ldcs(reinterpret_cast<const float4*>(a.dgi_c + (size_t)tb * 3 * H + (size_t)g * H + i));
        if (g == 2) {                                             // dgh_n = dgi_n * r
          const float4 r = __ldcs(reinterpret_cast<const float4*>(a.S + (size_t)tb * H + i));
          dv.x *= r.x; dv.y *= r.y; dv.z *= r.z; dv.w *= r.w;
        }
      }
      *reinterpret_cast<float4*>(bnd + b * RSZ + sw(i)) = hv;
      *reinterpret_cast<float4*>(dvec + b * RSZ + sw(i)) = dv;
    }
    __syncthreads();
    for (int p = 0; p + 1 < a.npasses; ++p) {
      run_pass2_s<RB, false, true>(spass[p], bnd + (size_t)p * RB * RSZ, 0, bnd + (size_t)(p + 1) * RB * RSZ, 0, twsm, 0, 0,
                                   Hpad, RSZ, a.logn, 1, WG_NT);
      __syncthreads();
    }
    for (int p = a.npasses - 1; p >= 0; --p) {
      wgrad_pass(spass[p], bnd + (size_t)p * RB * RSZ, dvec, nrows, twsm, acc, Hpad, RSZ, a.logn);
      __syncthreads();
    }
  }
  // partial sums leave in the reference's pair order
  float4* dst = reinterpret_cast<float4*>(partial) + ((size_t)blockIdx.x * 3 + g) * nacc;
  for (int p = 0; p < a.npasses; ++p) {
    const BflyPass pd = spass[p];
    for (int i = tid; i < pd.nst * half; i += WG_NT) {
      const int s = i / half, k = i - s * half;
      dst[(pd.l0 + s) * half + tw_source_index(pd, a.logn, half, k)] = acc[(pd.l0 + s) * half + k];
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

static size_t optin_smem2() {
  int dev = 0, v = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 48 * 1024;
  return (size_t)v;
}

static int sm_count2() {
  int dev = 0, v = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return v;
}

static int rsz_of(int Hpad) { return (Hpad + (Hpad >> 3) + 3) & ~3; }

static size_t smem2(bool fwd, int BT, int H, int Hpad, int nstages, int mode) {
  const size_t half = Hpad / 2;
  const size_t tw = mode == 1 ? (size_t)3 * nstages * half * 16 : (mode == 2 ? (size_t)2 * 9 * half * 16 : 0);
  const size_t RSZ = rsz_of(Hpad);
  size_t fl;
  if (fwd) fl = (size_t)4 * BT * RSZ + (size_t)4 * BT * H + (size_t)3 * H;
  else fl = (size_t)3 * BT * RSZ + (size_t)9 * BT * H;
  return 32 + tw + fl * sizeof(float);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Chooses BT and the twiddle mode; false if this variant does not apply.
static bool plan2(bool fwd, const BflyArgs& a, int want_bt, int* BT, int* mode, size_t* smem) {
  if (a.H % 4 != 0 || a.Hpad < 4) return false;
  const size_t lim = optin_smem2();
  for (int bt = want_bt; bt >= 1; bt >>= 1) {
    const int modes[3] = {1, 2, 0};
    for (int m = 0; m < 3; ++m) {
      const size_t s = smem2(fwd, bt, a.H, a.Hpad, a.nstages, modes[m]);
      if (s <= lim) { *BT = bt; *mode = modes[m]; *smem = s; return true; }
    }
  }
  return false;
}

template <typename K>
static int set_smem2(K kernel, size_t bytes) {
  return allow_dynamic_smem((const void*)kernel, bytes);
}

// Writes the copy of the twiddles the staged kernels read (see tw_source_index) into `twp`.
int bfly2_permute_twiddles(const BflyArgs& a, float* twp, cudaStream_t st) {
  if (!aligned16(a.tw) || !aligned16(twp)) return B200GRU_INVALID_ARGUMENT;
  const int total = 3 * a.nstages * (a.Hpad / 2);
  bfly_permute_twiddles_kernel<<<cdiv(total, 256), 256, 0, st>>>(reinterpret_cast<const float4*>(a.tw),
                                                                  reinterpret_cast<float4*>(twp), a);
  note_launch();
  return check_launch("bfly_permute_twiddles_kernel");
}

// returns -1 if the staged variant does not apply (caller falls back), else a status
int bfly2_launch_forward(BflyArgs a, int want_bt, cudaStream_t st) {
  if (a.twp == nullptr || !(aligned16(a.gi) && aligned16(a.h0) && aligned16(a.twp) && aligned16(a.out) &&
                            aligned16(a.save) && aligned16(a.h0_tail) && aligned16(a.bh))) return -1;
  int BT, mode; size_t smem;
  if (!plan2(true, a, want_bt, &BT, &mode, &smem)) return -1;
  a.tw_mode = mode; a.RSZ = rsz_of(a.Hpad);
  if (mode != 1 && a.H % 8 == 0 && 2 * a.B <= sm_count2()) {
    // three gates' twiddles do not fit one CTA: a pair of CTAs per row if two gates' do and all pairs
    // run at once (with more rows the one-CTA kernel with several rows per CTA uses the GPU better)
    const size_t pair_smem = 32 + (size_t)2 * a.nstages * (a.Hpad / 2) * 16 +
                             ((size_t)4 * a.RSZ + (size_t)4 * a.H + (size_t)3 * a.H) * sizeof(float);
    if (pair_smem <= optin_smem2()) {
      int rc = set_smem2(bfly_fwd2_pair_kernel<1>, pair_smem);
      if (rc) return rc;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2u * (unsigned)a.B); cfg.blockDim = dim3(NT); cfg.dynamicSmemBytes = pair_smem; cfg.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      BflyArgs pa = a;
      pa.tw_mode = 1;
      if (cudaLaunchKernelEx(&cfg, bfly_fwd2_pair_kernel<1>, pa) == cudaSuccess) {
        note_launch();
        return check_launch("bfly_fwd2_pair_kernel");
      }
      cudaGetLastError();        // no cluster launch on this device / partition: the one-CTA kernel below
    }
  }
  const unsigned grid = (unsigned)cdiv(a.B, BT);
  int rc = 0;
  switch (BT) {
    case 1:
      if (mode) { rc = set_smem2(bfly_fwd2_kernel<1, true>, smem); if (!rc) bfly_fwd2_kernel<1, true><<<grid, NT, smem, st>>>(a); }
      else { rc = set_smem2(bfly_fwd2_kernel<1, false>, smem); if (!rc) bfly_fwd2_kernel<1, false><<<grid, NT, smem, st>>>(a); }
      break;
    default:
      if (mode) { rc = set_smem2(bfly_fwd2_kernel<2, true>, smem); if (!rc) bfly_fwd2_kernel<2, true><<<grid, NT, smem, st>>>(a); }
      else { rc = set_smem2(bfly_fwd2_kernel<2, false>, smem); if (!rc) bfly_fwd2_kernel<2, false><<<grid, NT, smem, st>>>(a); }
      break;
  }
  if (rc) return rc;
  note_launch();
  return check_launch("bfly_fwd2_kernel");
}

int bfly2_launch_backward(BflyArgs a, int want_bt, cudaStream_t st) {
  if (a.twp == nullptr || !(aligned16(a.gi) && aligned16(a.h0) && aligned16(a.twp) && aligned16(a.out_c) &&
                            aligned16(a.S) && aligned16(a.dout) && aligned16(a.dgi) && aligned16(a.dh0))) return -1;
  int BT, mode; size_t smem;
  if (!plan2(false, a, want_bt, &BT, &mode, &smem)) return -1;
  a.tw_mode = mode; a.RSZ = rsz_of(a.Hpad);
  if (mode != 1 && a.H % 8 == 0 && 2 * a.B <= sm_count2()) {
    // as in the forward: a pair of CTAs per row when two gates' twiddles fit one CTA and all pairs run at once
    const size_t pair_smem = 32 + (size_t)2 * a.nstages * (a.Hpad / 2) * 16 +
                             ((size_t)3 * a.RSZ + (size_t)11 * a.H) * sizeof(float);
    if (pair_smem <= optin_smem2()) {
      int rc = set_smem2(bfly_bwd2_pair_kernel<1>, pair_smem);
      if (rc) return rc;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2u * (unsigned)a.B); cfg.blockDim = dim3(NT); cfg.dynamicSmemBytes = pair_smem; cfg.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      BflyArgs pa = a;
      pa.tw_mode = 1;
      if (cudaLaunchKernelEx(&cfg, bfly_bwd2_pair_kernel<1>, pa) == cudaSuccess) {
        note_launch();
        return check_launch("bfly_bwd2_pair_kernel");
      }
      cudaGetLastError();        // no cluster launch on this device / partition: the one-CTA kernel below
    }
  }
  const unsigned grid = (unsigned)cdiv(a.B, BT);
  int rc = 0;
  switch (BT) {
    case 1:
      if (mode) { rc = set_smem2(bfly_bwd2_kernel<1, true>, smem); if (!rc) bfly_bwd2_kernel<1, true><<<grid, NT, smem, st>>>(a); }
      else { rc = set_smem2(bfly_bwd2_kernel<1, false>, smem); if (!rc) bfly_bwd2_kernel<1, false><<<grid, NT, smem, st>>>(a); }
      break;
    default:
      if (mode) { rc = set_smem2(bfly_bwd2_kernel<2, true>, smem); if (!rc) bfly_bwd2_kernel<2, true><<<grid, NT, smem, st>>>(a); }
      else { rc = set_smem2(bfly_bwd2_kernel<2, false>, smem); if (!rc) bfly_bwd2_kernel<2, false><<<grid, NT, smem, st>>>(a); }
      break;
  }
  if (rc) return rc;
  note_launch();
  return check_launch("bfly_bwd2_kernel");
}


// Geometry of the staged twiddle-gradient kernel; false if it does not apply (twiddles and
// accumulators of one gate must fit shared memory next to two rows of pass inputs).
static bool wgrad2_geometry(int T, int B, int H, int Hpad, int ns, int npasses, int* RB, int* nsplit,
                            int* rows_per_split, size_t* smem) {
  if (H % 4 != 0 || Hpad < 8 || npasses < 1) return false;
  const size_t lim = optin_smem2() - 1024;             // static: the pass table
  const size_t fixed = (size_t)2 * ns * (Hpad / 2) * 16;
  const size_t per_row = (size_t)(npasses + 1) * rsz_of(Hpad) * sizeof(float);
  int rb = 0;
  if (fixed + 4 * per_row <= lim) rb = 4;
  else if (fixed + 2 * per_row <= lim) rb = 2;
  if (rb == 0) return false;
  *RB = rb;
  *smem = fixed + rb * per_row;
  const int per_sm = (int)((lim + 1024) / (*smem + 1024)) > 0 ? (int)((lim + 1024) / (*smem + 1024)) : 1;
  const int TB = T * B;
  int want = (148 * per_sm) / 3;
  const int max_by_rows = cdiv(TB, 4 * rb);
  if (want > max_by_rows) want = max_by_rows;
  if (want < 1) want = 1;
  const int rps = cdiv(cdiv(TB, want), rb) * rb;
  *rows_per_split = rps;
  *nsplit = cdiv(TB, rps);
  return true;
}

size_t bfly2_wgrad_scratch_bytes(int T, int B, int H, int Hpad, int ns) {
  BflyPass tmp[BFLY_MAX_PASSES];
  int logn = 0;
  while ((1 << logn) < Hpad) ++logn;
  const int np = build_bfly_passes(logn, ns / (logn > 0 ? logn : 1), tmp, BFLY_MAX_PASSES);
  int RB, nsplit, rps; size_t smem;
  if (np < 1 || !wgrad2_geometry(T, B, H, Hpad, ns, np, &RB, &nsplit, &rps, &smem)) return 0;
  return align_up((size_t)nsplit * 3 * ns * (Hpad / 2) * 16, 256);
}

// returns -1 if the staged variant does not apply (caller falls back), else a status
int bfly2_launch_wgrad(BflyArgs a, float* partial, float* dtw, cudaStream_t st) {
  if (a.twp == nullptr || !(aligned16(a.h0) && aligned16(a.twp) && aligned16(a.out_c) && aligned16(a.S) &&
                            aligned16(a.dgi_c) && aligned16(partial)))
    return -1;
  int RB, nsplit, rps; size_t smem;
  if (!wgrad2_geometry(a.T, a.B, a.H, a.Hpad, a.nstages, a.npasses, &RB, &nsplit, &rps, &smem)) return -1;
  a.RSZ = rsz_of(a.Hpad);
  dim3 grid(nsplit, 3);
  int rc;
  if (RB == 4) { rc = set_smem2(bfly_wgrad2_kernel<4>, smem); if (!rc) bfly_wgrad2_kernel<4><<<grid, WG_NT, smem, st>>>(a, partial, rps); }
  else         { rc = set_smem2(bfly_wgrad2_kernel<2>, smem); if (!rc) bfly_wgrad2_kernel<2><<<grid, WG_NT, smem, st>>>(a, partial, rps); }
  if (rc) return rc;
  note_launch();
  rc = check_launch("bfly_wgrad2_kernel");
  if (rc) return rc;
  const size_t n = (size_t)3 * a.nstages * (a.Hpad / 2) * 4;
  launch_reduce_partials(partial, nsplit, n, n, dtw, st);
  return check_launch("reduce_partials");
}

int bfly_read_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_bfly_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_bfly_status, &z, sizeof(int));
  }
  return v;
}

}  // namespace b200gru

B200GRU_DEFINE_PHASE_READER(b200gru_debug_phase_cycles_bfly2)
