// Butterfly hidden weights: gh_g = Butterfly_g(fq_in(h)) + b_g.
//
// One gate's butterfly is nblocks*log2(Hpad) stages of 2x2 mixing between positions
// i and i ^ S (S = stage stride).  twiddle[g][l][pair][m_new][m_old], l = blk*log_n + s;
// even blocks walk strides 1,2,4,.., odd blocks the reverse; the stage axis is indexed by
// iteration number (src/gru_qat/triton_kernels/scan_butterfly.py:276-317).
//
// One CTA owns BT batch rows x the whole padded hidden width for all T steps.  The
// running vectors of the three gates live in shared memory.  Consecutive stages whose
// strides span at most three adjacent bits are fused into one PASS: a thread loads the
// 2^r positions that those stages mix among themselves, runs the stages in registers
// and writes them back -- one barrier per pass instead of one per stage, no global
// scratch round-trip.  A thread's twiddles (one float4 per pair per stage) are the same
// for every row of the tile, so they are fetched once per pass and reused BT times.
// gi[t] (forward) and dout/activations (backward) arrive by cp.async one step ahead.
//
// Backward = three kernels: (1) gate recompute, which is this same forward kernel run
// teacher-forced over all T*B rows at once; (2) the serial reverse scan below, whose
// only on-chain work is the TRANSPOSED butterfly of dgh; (3) twiddle gradients,
// parallel over rows, accumulated per CTA in shared memory (bfly_wgrad_kernel).

#include <cstdlib>

#include "butterfly_scan.cuh"

namespace b200gru {

namespace {

constexpr int NT = BFLY_THREADS;

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gsrc) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

__device__ __forceinline__ int stage_log_stride(int l, int logn) {
  const int blk = l / logn, s = l - blk * logn;
  return (blk & 1) ? (logn - 1 - s) : s;
}

// One 2x2 stage on register vector v[1<<R] along local bit P; tw[idx] belongs to the idx-th pair.
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
        v[b][e] = fmaf(t.y, a1, t.x * a0);              // t00*a0 + t01*a1
        v[b][e | (1 << P)] = fmaf(t.z, a0, t.w * a1);   // t11*a1 + t10*a0
      } else {
        v[b][e] = fmaf(t.z, a1, t.x * a0);              // t00*d0 + t10*d1
        v[b][e | (1 << P)] = fmaf(t.y, a0, t.w * a1);   // t11*d1 + t01*d0
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

// Run one pass over the three gates.  `src` (stride src_gate between gates, 0 = shared
// input) is read, `dst` (stride dst_gate) written; they may alias.  Rows are Hpad apart.
template <int R, int BT, bool TRANSPOSE>
__device__ __forceinline__ void run_pass_r(const BflyPass pd, const float* src, int src_gate, float* dst,
                                           int dst_gate, const float* __restrict__ tw, int Hpad, int logn,
                                           int nstages) {
  constexpr int E = 1 << R;
  const int lb = pd.lb;
  const int G = Hpad >> R;
  const int half = Hpad >> 1;
  for (int item = threadIdx.x; item < 3 * G; item += NT) {
    const int g = item / G, q = item - g * G;
    const int low = q & ((1 << lb) - 1), high = q >> lb;
    const int base = (high << (lb + R)) | low;

    float4 t[3][E / 2];
    int pbit[3];
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      pbit[s] = 0;
      if (s < pd.nst) {
        const int l = TRANSPOSE ? (pd.l0 + pd.nst - 1 - s) : (pd.l0 + s);
        const int ls = stage_log_stride(l, logn);
        const int p = ls - lb;
        pbit[s] = p;
        const int S = 1 << ls;
        const float4* tl = reinterpret_cast<const float4*>(tw) + ((size_t)g * nstages + l) * half;
#pragma unroll
        for (int idx = 0; idx < E / 2; ++idx) {
          // idx-th pair of the group: local index with a zero inserted at bit p
          const int e0 = ((idx >> p) << (p + 1)) | (idx & ((1 << p) - 1));
          const int i0 = base + (e0 << lb);
          const int pair = ((i0 >> (ls + 1)) << ls) | (i0 & (S - 1));
          t[s][idx] = tl[pair];
        }
      }
    }

    float v[BT][E];
    const float* sp = src + (size_t)g * src_gate + base;
#pragma unroll
    for (int b = 0; b < BT; ++b)
#pragma unroll
      for (int e = 0; e < E; ++e) v[b][e] = sp[b * Hpad + (e << lb)];

#pragma unroll
    for (int s = 0; s < 3; ++s)
      if (s < pd.nst) stage_dispatch<R, BT, TRANSPOSE>(v, t[s], pbit[s]);

    float* dp = dst + (size_t)g * dst_gate + base;
#pragma unroll
    for (int b = 0; b < BT; ++b)
#pragma unroll
      for (int e = 0; e < E; ++e) dp[b * Hpad + (e << lb)] = v[b][e];
  }
}

template <int BT, bool TRANSPOSE>
__device__ __forceinline__ void run_pass(const BflyPass pd, const float* src, int src_gate, float* dst,
                                         int dst_gate, const float* tw, int Hpad, int logn, int nstages) {
  if (pd.r == 3) run_pass_r<3, BT, TRANSPOSE>(pd, src, src_gate, dst, dst_gate, tw, Hpad, logn, nstages);
  else if (pd.r == 2) run_pass_r<2, BT, TRANSPOSE>(pd, src, src_gate, dst, dst_gate, tw, Hpad, logn, nstages);
  else run_pass_r<1, BT, TRANSPOSE>(pd, src, src_gate, dst, dst_gate, tw, Hpad, logn, nstages);
}

}  // namespace

// ---------------------------------------------------------------------------
// forward scan (also the teacher-forced gate recompute: T = 1 over flattened rows)
// ---------------------------------------------------------------------------
template <int BT>
__global__ void __launch_bounds__(NT)
bfly_fwd_kernel(const BflyArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int H = a.H, Hpad = a.Hpad;
  const int row0 = blockIdx.x * BT;
  const int tid = threadIdx.x;

  const int n4 = a.tw_in_smem ? 3 * a.nstages * (Hpad >> 1) : 0;
  float* twsm = smem;                       // optional twiddle copy (16-byte aligned, first)
  float* st = smem + 4 * n4;                // [3][BT][Hpad]
  float* hq = st + 3 * BT * Hpad;           // [BT][Hpad]  fq_in(h), zero beyond H
  float* hraw = hq + BT * Hpad;             // [BT][Hpad]
  float* gbuf = hraw + BT * Hpad;           // [3][BT][H]  gi of the current step
  const float* tw = a.tw;
  if (a.tw_in_smem) {
    const float4* s4 = reinterpret_cast<const float4*>(a.tw);
    float4* d4 = reinterpret_cast<float4*>(twsm);
    for (int i = tid; i < n4; i += NT) d4[i] = s4[i];
    tw = twsm;
  }

  for (int idx = tid; idx < BT * Hpad; idx += NT) {
    const int b = idx / Hpad, i = idx - b * Hpad;
    const int row = row0 + b;
    float v = 0.f;
    if (row < a.B && i < H)
      v = (row < a.h0_rows) ? a.h0[(size_t)row * H + i] : a.h0_tail[(size_t)(row - a.h0_rows) * H + i];
    hraw[idx] = v;
    hq[idx] = (a.qin.enabled && i < H) ? fake_quant<true>(v, a.qin) : v;
  }
  __syncthreads();

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;

  PHASE_DECL;
  for (int t = 0; t < a.T; ++t) {
    PHASE_START();
    // gi[t] for the tile: lands while the butterflies run
    for (int idx = tid; idx < 3 * BT * H; idx += NT) {
      const int g = idx / (BT * H);
      const int rem = idx - g * BT * H;
      const int b = rem / H, i = rem - b * H;
      const int row = row0 + b;
      if (row < a.B) cp_async4(gbuf + idx, a.gi + (size_t)t * gi_step + (size_t)row * 3 * H + g * H + i);
    }
    cp_async_commit();
    PHASE_MARK(0);

    for (int p = 0; p < a.npasses; ++p) {
      if (p == 0) run_pass<BT, false>(a.passes[0], hq, 0, st, BT * Hpad, tw, Hpad, a.logn, a.nstages);
      else run_pass<BT, false>(a.passes[p], st, BT * Hpad, st, BT * Hpad, tw, Hpad, a.logn, a.nstages);
      PHASE_MARK(1 + (p < 4 ? p : 4));
      __syncthreads();
      PHASE_MARK(6);
    }
    cp_async_wait_all();
    __syncthreads();
    PHASE_MARK(7);

    for (int idx = tid; idx < BT * H; idx += NT) {
      const int b = idx / H, i = idx - b * H;
      const int row = row0 + b;
      if (row >= a.B) continue;
      const float ghr = st[(0 * BT + b) * Hpad + i] + a.bh[i];
      const float ghz = st[(1 * BT + b) * Hpad + i] + a.bh[H + i];
      const float ghn = st[(2 * BT + b) * Hpad + i] + a.bh[2 * H + i];
      const float hp = hraw[b * Hpad + i];
      const GateOut g = gru_gates(gbuf[(0 * BT + b) * H + i], gbuf[(1 * BT + b) * H + i],
                                  gbuf[(2 * BT + b) * H + i], ghr, ghz, ghn, hp);
      const float hnew = a.qout.enabled ? fake_quant<true>(g.h_raw, a.qout) : g.h_raw;
      const size_t o = (size_t)t * out_step + (size_t)row * H + i;
      if (a.out != nullptr) a.out[o] = hnew;
      if (a.save != nullptr) {
        __stcs(a.save + o, g.r);
        __stcs(a.save + comp + o, g.z);
        __stcs(a.save + 2 * comp + o, g.n);
        __stcs(a.save + 3 * comp + o, ghn);
      }
      hraw[b * Hpad + i] = hnew;
      hq[b * Hpad + i] = a.qin.enabled ? fake_quant<true>(hnew, a.qin) : hnew;
    }
    PHASE_MARK(8);
    __syncthreads();
    PHASE_MARK(9);
  }
}

// ---------------------------------------------------------------------------
// backward, serial part
// ---------------------------------------------------------------------------
template <int BT>
__global__ void __launch_bounds__(NT)
bfly_bwd_kernel(const BflyArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int H = a.H, Hpad = a.Hpad;
  const int row0 = blockIdx.x * BT;
  const int tid = threadIdx.x;

  const int n4 = a.tw_in_smem ? 3 * a.nstages * (Hpad >> 1) : 0;
  float* twsm = smem;                       // optional twiddle copy (16-byte aligned, first)
  float* st = smem + 4 * n4;                // [3][BT][Hpad]  dgh -> transposed butterfly in place
  float* pbuf = st + 3 * BT * Hpad;         // [6][BT][H]     dout, r, z, n, gh_n, h_prev of the step
  float* dhacc = pbuf + 6 * BT * H;         // [BT][H]
  float* dhdir = dhacc + BT * H;            // [BT][H]
  float* mk = dhdir + BT * H;               // [BT][H]        fq_in straight-through mask
  const float* tw = a.tw;
  if (a.tw_in_smem) {
    const float4* s4 = reinterpret_cast<const float4*>(a.tw);
    float4* d4 = reinterpret_cast<float4*>(twsm);
    for (int i = tid; i < n4; i += NT) d4[i] = s4[i];
    tw = twsm;
  }
  for (int idx = tid; idx < BT * H; idx += NT) dhacc[idx] = 0.f;

  const size_t gi_step = (size_t)a.B * 3 * H;
  const size_t out_step = (size_t)a.B * H;
  const size_t comp = (size_t)a.T * out_step;

  auto prefetch = [&](int t) {
    for (int idx = tid; idx < 6 * BT * H; idx += NT) {
      const int c = idx / (BT * H);
      const int rem = idx - c * BT * H;
      const int b = rem / H, i = rem - b * H;
      const int row = row0 + b;
      if (row >= a.B) continue;
      const size_t o = (size_t)t * out_step + (size_t)row * H + i;
      const float* src;
      if (c == 0) src = a.dout + o;
      else if (c <= 4) src = a.S + (size_t)(c - 1) * comp + o;
      else src = (t > 0) ? (a.out_c + o - out_step) : (a.h0 + (size_t)row * H + i);
      cp_async4(pbuf + idx, src);
    }
    cp_async_commit();
  };
  prefetch(a.T - 1);
  cp_async_wait_all();
  __syncthreads();

  for (int t = a.T - 1; t >= 0; --t) {
    for (int idx = tid; idx < BT * Hpad; idx += NT) {
      const int b = idx / Hpad, i = idx - b * Hpad;
      const int row = row0 + b;
      float x0 = 0.f, x1 = 0.f, x2 = 0.f;
      if (row < a.B && i < H) {
        const int e = b * H + i;
        const float r = pbuf[1 * BT * H + e], z = pbuf[2 * BT * H + e], nn = pbuf[3 * BT * H + e];
        const float ghn = pbuf[4 * BT * H + e], hp = pbuf[5 * BT * H + e];
        float dh = pbuf[e] + dhacc[e];
        if (a.qout.enabled) {
          const float h_raw = (1.0f - z) * nn + z * hp;
          dh = dh * ste_mask<true>(h_raw, a.qout);
        }
        const GateGrad gg = gru_gate_grads(dh, r, z, nn, ghn, hp);
        dhdir[e] = gg.dh_direct;
        mk[e] = a.qin.enabled ? ste_mask<true>(hp, a.qin) : 1.0f;
        float* d = a.dgi + (size_t)t * gi_step + (size_t)row * 3 * H + i;
        __stcs(d, gg.dgr); __stcs(d + H, gg.dgz); __stcs(d + 2 * H, gg.dgn);
        x0 = gg.dgr; x1 = gg.dgz; x2 = gg.dghn;
      }
      st[(0 * BT + b) * Hpad + i] = x0;
      st[(1 * BT + b) * Hpad + i] = x1;
      st[(2 * BT + b) * Hpad + i] = x2;
    }
    __syncthreads();
    if (t > 0) prefetch(t - 1);

    for (int p = a.npasses - 1; p >= 0; --p) {
      run_pass<BT, true>(a.passes[p], st, BT * Hpad, st, BT * Hpad, tw, Hpad, a.logn, a.nstages);
      __syncthreads();
    }

    for (int idx = tid; idx < BT * H; idx += NT) {
      const int b = idx / H, i = idx - b * H;
      if (row0 + b >= a.B) continue;
      const float via = st[(0 * BT + b) * Hpad + i] + st[(1 * BT + b) * Hpad + i] + st[(2 * BT + b) * Hpad + i];
      dhacc[idx] = dhdir[idx] + via * mk[idx];
    }
    cp_async_wait_all();
    __syncthreads();
  }

  for (int idx = tid; idx < BT * H; idx += NT) {
    const int b = idx / H, i = idx - b * H;
    const int row = row0 + b;
    if (row < a.B) a.dh0[(size_t)row * H + i] = dhacc[idx];
  }
}

// ---------------------------------------------------------------------------
// twiddle gradients: dt[g][l][pair][m_new][m_old] = sum_rows d_new[m_new] * old[m_old]
// ---------------------------------------------------------------------------
// grid = (row splits, 3 gates, stage groups).  Per tile of RT rows the CTA recomputes
// the forward stage inputs into shared memory, then walks the stages backwards,
// accumulating the four products of every pair it owns into a shared accumulator.
template <int RT>
__global__ void __launch_bounds__(NT)
bfly_wgrad_kernel(const BflyArgs a, float* __restrict__ partial, int rows_per_split, int stages_per_group) {
  extern __shared__ __align__(16) float smem[];
  const int H = a.H, Hpad = a.Hpad, half = Hpad >> 1, ns = a.nstages;
  const int TB = a.T * a.B;
  const int g = blockIdx.y;
  const int l_lo = blockIdx.z * stages_per_group;
  const int l_hi = min(ns, l_lo + stages_per_group);
  const int r_begin = blockIdx.x * rows_per_split;
  const int r_end = min(TB, r_begin + rows_per_split);
  const int tid = threadIdx.x;

  const int nacc = (l_hi - l_lo) * half;
  float4* acc = reinterpret_cast<float4*>(smem);      // [l_hi - l_lo][half] (16-byte aligned, first)
  float* states = smem + (size_t)4 * stages_per_group * half;   // [RT][ns][Hpad]  input of every stage
  float* dvec = states + (size_t)RT * ns * Hpad;      // [RT][Hpad]
  for (int i = tid; i < nacc; i += NT) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* twg = reinterpret_cast<const float4*>(a.tw) + (size_t)g * ns * half;

  for (int r0 = r_begin; r0 < r_end; r0 += RT) {
    for (int idx = tid; idx < RT * Hpad; idx += NT) {
      const int b = idx / Hpad, i = idx - b * Hpad;
      const int tb = r0 + b;
      float hv = 0.f, dv = 0.f;
      if (tb < r_end && i < H) {
        hv = (tb < a.B) ? a.h0[(size_t)tb * H + i] : a.out_c[(size_t)(tb - a.B) * H + i];
        if (a.qin.enabled) hv = fake_quant<true>(hv, a.qin);
        dv = a.dgi_c[(size_t)tb * 3 * H + (size_t)g * H + i];
        if (g == 2) dv = dv * a.S[(size_t)tb * H + i];          // dgh_n = dgi_n * r
      }
      states[((size_t)b * ns) * Hpad + i] = hv;
      dvec[idx] = dv;
    }
    __syncthreads();
    // forward: states[l+1] from states[l]
    for (int l = 0; l + 1 < ns; ++l) {
      const int ls = stage_log_stride(l, a.logn);
      const int S = 1 << ls;
      for (int idx = tid; idx < RT * half; idx += NT) {
        const int b = idx / half, p = idx - b * half;
        const int i0 = ((p >> ls) << (ls + 1)) | (p & (S - 1));
        const float4 t = twg[(size_t)l * half + p];
        const float* in = states + ((size_t)b * ns + l) * Hpad;
        float* o = states + ((size_t)b * ns + l + 1) * Hpad;
        const float a0 = in[i0], a1 = in[i0 + S];
        o[i0] = fmaf(t.y, a1, t.x * a0);
        o[i0 + S] = fmaf(t.z, a0, t.w * a1);
      }
      __syncthreads();
    }
    // backward
    for (int l = ns - 1; l >= 0; --l) {
      const int ls = stage_log_stride(l, a.logn);
      const int S = 1 << ls;
      const bool mine = (l >= l_lo && l < l_hi);
      for (int p = tid; p < half; p += NT) {
        const int i0 = ((p >> ls) << (ls + 1)) | (p & (S - 1));
        const float4 t = twg[(size_t)l * half + p];
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int b = 0; b < RT; ++b) {
          const float* in = states + ((size_t)b * ns + l) * Hpad;
          float* d = dvec + b * Hpad;
          const float d0 = d[i0], d1 = d[i0 + S];
          const float o0 = in[i0], o1 = in[i0 + S];
          s.x = fmaf(d0, o0, s.x); s.y = fmaf(d0, o1, s.y);
          s.z = fmaf(d1, o0, s.z); s.w = fmaf(d1, o1, s.w);
          d[i0] = fmaf(t.z, d1, t.x * d0);
          d[i0 + S] = fmaf(t.y, d0, t.w * d1);
        }
        if (mine) {
          float4 c = acc[(l - l_lo) * half + p];
          c.x += s.x; c.y += s.y; c.z += s.z; c.w += s.w;
          acc[(l - l_lo) * half + p] = c;
        }
      }
      __syncthreads();
    }
  }
  float4* dst = reinterpret_cast<float4*>(partial) + ((size_t)blockIdx.x * 3 + g) * ns * half;
  for (int i = tid; i < nacc; i += NT) dst[(size_t)l_lo * half + i] = acc[i];
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

int build_bfly_passes(int logn, int nblocks, BflyPass* passes, int max_passes) {
  const int ns = logn * nblocks;
  auto ls_of = [&](int l) { int blk = l / logn, s = l % logn; return (blk & 1) ? logn - 1 - s : s; };
  int np = 0, l = 0;
  while (l < ns) {
    int lo = ls_of(l), hi = lo, n = 1;
    while (l + n < ns && n < 3) {
      const int x = ls_of(l + n);
      const int nlo = x < lo ? x : lo, nhi = x > hi ? x : hi;
      if (nhi - nlo + 1 > 3) break;
      lo = nlo; hi = nhi; ++n;
    }
    if (np >= max_passes) return -1;
    passes[np].l0 = (short)l; passes[np].nst = (short)n; passes[np].lb = (short)lo; passes[np].r = (short)(hi - lo + 1);
    for (int s = 0; s < 4; ++s) passes[np].pb[s] = (short)(s < n ? ls_of(l + s) - lo : 0);
    ++np; l += n;
  }
  return np;
}

static size_t optin_smem() {
  int dev = 0, v = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 48 * 1024;
  return (size_t)v;
}

static int pick_bt(int B) {
  // keep >= ~32 CTAs when the batch allows, at most 4 rows per CTA
  int bt = 1;
  while (bt < 4 && B / (bt * 2) >= 32) bt *= 2;
  return bt;
}

// staged kernels: spread a small batch over as many SMs as possible (>= ~128 CTAs), up to 2 rows
static int pick_bt2(int B) { return B >= 256 ? 2 : 1; }

static size_t fwd_smem(int BT, int H, int Hpad, size_t tw_bytes) {
  return ((size_t)5 * BT * Hpad + (size_t)3 * BT * H) * sizeof(float) + tw_bytes;
}
static size_t bwd_smem(int BT, int H, int Hpad, size_t tw_bytes) {
  return ((size_t)3 * BT * Hpad + (size_t)9 * BT * H) * sizeof(float) + tw_bytes;
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  return allow_dynamic_smem((const void*)kernel, bytes);
}

int bfly_launch_forward(BflyArgs a, cudaStream_t st) {
  // The staged variant is the faster one wherever it applies; the test hook selects the kernel below
  // on aligned shapes too, so that both keep parity coverage.
  if (test_kernel_choice(0) == 0) {
    const int rc2 = bfly2_launch_forward(a, pick_bt2(a.B), st);
    if (rc2 >= 0) return rc2;
  }
  const size_t lim = optin_smem();
  const size_t twb = (size_t)3 * a.nstages * (a.Hpad / 2) * 16;
  int BT = pick_bt(a.B);
  while (BT > 1 && fwd_smem(BT, a.H, a.Hpad, 0) > lim) BT >>= 1;
  if (fwd_smem(BT, a.H, a.Hpad, 0) > lim) return B200GRU_UNSUPPORTED;
  a.tw_in_smem = (fwd_smem(BT, a.H, a.Hpad, twb) <= lim && a.T >= 4) ? 1 : 0;
  const size_t smem = fwd_smem(BT, a.H, a.Hpad, a.tw_in_smem ? twb : 0);
  const unsigned grid = (unsigned)cdiv(a.B, BT);
  int rc = 0;
  switch (BT) {
    case 1: rc = set_smem(bfly_fwd_kernel<1>, smem); if (!rc) bfly_fwd_kernel<1><<<grid, NT, smem, st>>>(a); break;
    case 2: rc = set_smem(bfly_fwd_kernel<2>, smem); if (!rc) bfly_fwd_kernel<2><<<grid, NT, smem, st>>>(a); break;
    default: rc = set_smem(bfly_fwd_kernel<4>, smem); if (!rc) bfly_fwd_kernel<4><<<grid, NT, smem, st>>>(a); break;
  }
  if (rc) return rc;
  note_launch();
  return check_launch("bfly_fwd_kernel");
}

int bfly_launch_backward(BflyArgs a, cudaStream_t st) {
  if (test_kernel_choice(0) == 0) {
    const int rc2 = bfly2_launch_backward(a, pick_bt2(a.B), st);
    if (rc2 >= 0) return rc2;
  }
  const size_t lim = optin_smem();
  const size_t twb = (size_t)3 * a.nstages * (a.Hpad / 2) * 16;
  int BT = pick_bt(a.B);
  while (BT > 1 && bwd_smem(BT, a.H, a.Hpad, 0) > lim) BT >>= 1;
  if (bwd_smem(BT, a.H, a.Hpad, 0) > lim) return B200GRU_UNSUPPORTED;
  a.tw_in_smem = (bwd_smem(BT, a.H, a.Hpad, twb) <= lim && a.T >= 4) ? 1 : 0;
  const size_t smem = bwd_smem(BT, a.H, a.Hpad, a.tw_in_smem ? twb : 0);
  const unsigned grid = (unsigned)cdiv(a.B, BT);
  int rc = 0;
  switch (BT) {
    case 1: rc = set_smem(bfly_bwd_kernel<1>, smem); if (!rc) bfly_bwd_kernel<1><<<grid, NT, smem, st>>>(a); break;
    case 2: rc = set_smem(bfly_bwd_kernel<2>, smem); if (!rc) bfly_bwd_kernel<2><<<grid, NT, smem, st>>>(a); break;
    default: rc = set_smem(bfly_bwd_kernel<4>, smem); if (!rc) bfly_bwd_kernel<4><<<grid, NT, smem, st>>>(a); break;
  }
  if (rc) return rc;
  note_launch();
  return check_launch("bfly_bwd_kernel");
}

// twiddle-gradient launch geometry (shared with the workspace query)
static bool wgrad_geometry(int T, int B, int Hpad, int ns, int* RT, int* spg, int* ngroups, int* nsplit,
                           int* rows_per_split, size_t* smem) {
  const size_t lim = optin_smem();
  const int half = Hpad / 2;
  for (int rt = 2; rt >= 1; --rt) {
    const size_t fixed = ((size_t)rt * ns * Hpad + (size_t)rt * Hpad) * sizeof(float);
    if (fixed + (size_t)half * 16 > lim) continue;
    int s = (int)((lim - fixed) / ((size_t)half * 16));
    if (s > ns) s = ns;
    if (s < 1) continue;
    *RT = rt; *spg = s; *ngroups = cdiv(ns, s);
    const int TB = T * B;
    int want = cdiv(2 * 148, 3 * *ngroups);
    const int max_by_rows = cdiv(TB, 8 * rt);
    if (want > max_by_rows) want = max_by_rows;
    if (want < 1) want = 1;
    const int rps = cdiv(cdiv(TB, want), rt) * rt;
    *rows_per_split = rps;
    *nsplit = cdiv(TB, rps);
    *smem = fixed + (size_t)s * half * 16;
    return true;
  }
  return false;
}

size_t bfly_wgrad_scratch_bytes(int T, int B, int H, int Hpad, int ns) {
  int RT, spg, ng, nsplit, rps; size_t smem;
  if (!wgrad_geometry(T, B, Hpad, ns, &RT, &spg, &ng, &nsplit, &rps, &smem)) return (size_t)-1;
  const size_t general = align_up((size_t)nsplit * 3 * ns * (Hpad / 2) * 16, 256);
  const size_t staged = bfly2_wgrad_scratch_bytes(T, B, H, Hpad, ns);
  return staged > general ? staged : general;
}

int bfly_launch_wgrad(BflyArgs a, float* partial, float* dtw, cudaStream_t st) {
  if (test_kernel_choice(0) == 0) {
    const int rc2 = bfly2_launch_wgrad(a, partial, dtw, st);
    if (rc2 >= 0) return rc2;
  }
  int RT, spg, ng, nsplit, rps; size_t smem;
  if (!wgrad_geometry(a.T, a.B, a.Hpad, a.nstages, &RT, &spg, &ng, &nsplit, &rps, &smem)) return B200GRU_UNSUPPORTED;
  dim3 grid(nsplit, 3, ng);
  int rc;
  if (RT == 2) { rc = set_smem(bfly_wgrad_kernel<2>, smem); if (!rc) bfly_wgrad_kernel<2><<<grid, NT, smem, st>>>(a, partial, rps, spg); }
  else         { rc = set_smem(bfly_wgrad_kernel<1>, smem); if (!rc) bfly_wgrad_kernel<1><<<grid, NT, smem, st>>>(a, partial, rps, spg); }
  if (rc) return rc;
  note_launch();
  rc = check_launch("bfly_wgrad_kernel");
  if (rc) return rc;
  const size_t n = (size_t)3 * a.nstages * (a.Hpad / 2) * 4;
  launch_reduce_partials(partial, nsplit, n, n, dtw, st);
  return check_launch("reduce_partials");
}

}  // namespace b200gru

B200GRU_DEFINE_PHASE_READER(b200gru_debug_phase_cycles_bfly)
