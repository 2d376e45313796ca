// Diagonal hidden weights: gh_g = w_g * fq_in(h) + b_g  (elementwise over H).
//
// Every (batch row, hidden unit) pair is an independent length-T recurrence, so
// the scan is a pure streaming kernel: one thread owns VEC adjacent hidden units
// of one row, carries h (forward) or dh plus six weight/bias gradient sums
// (backward) in registers for all T steps, and touches HBM exactly once per
// algorithmic byte: 16*H bytes per sequence-step forward (gi read, out write),
// 32*H backward (gi, h_prev, dout read; dgi write).  gi[t] does not depend on the
// recurrence, so loads run PF steps ahead of the arithmetic in a register ring
// that keeps PF*3*VEC*4 bytes per thread in flight.
//
// Follows the step arithmetic of src/gru_qat/triton_kernels/scan_diagonal.py
// (forward :79-124, backward :564-647).

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace b200gru {

template <int VEC> struct VecT;
template <> struct VecT<1> { using type = float; };
template <> struct VecT<2> { using type = float2; };
template <> struct VecT<4> { using type = float4; };

template <int VEC>
__device__ __forceinline__ void ld_stream(const float* p, float (&v)[VEC]) {
  using V = typename VecT<VEC>::type;
  V x = __ldcs(reinterpret_cast<const V*>(p));
  const float* f = reinterpret_cast<const float*>(&x);
#pragma unroll
  for (int i = 0; i < VEC; ++i) v[i] = f[i];
}

template <int VEC>
__device__ __forceinline__ void ld_plain(const float* p, float (&v)[VEC]) {
  using V = typename VecT<VEC>::type;
  V x = *reinterpret_cast<const V*>(p);
  const float* f = reinterpret_cast<const float*>(&x);
#pragma unroll
  for (int i = 0; i < VEC; ++i) v[i] = f[i];
}

template <int VEC>
__device__ __forceinline__ void st_vec(float* p, const float (&v)[VEC]) {
  using V = typename VecT<VEC>::type;
  V x;
  float* f = reinterpret_cast<float*>(&x);
#pragma unroll
  for (int i = 0; i < VEC; ++i) f[i] = v[i];
  *reinterpret_cast<V*>(p) = x;
}

template <int VEC>
__device__ __forceinline__ void st_stream(float* p, const float (&v)[VEC]) {
  using V = typename VecT<VEC>::type;
  V x;
  float* f = reinterpret_cast<float*>(&x);
#pragma unroll
  for (int i = 0; i < VEC; ++i) f[i] = v[i];
  __stcs(reinterpret_cast<V*>(p), x);
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <int VEC, int PF, bool QIN, bool QOUT>
__global__ void __launch_bounds__(128)
diag_fwd_kernel(const float* __restrict__ gi, const float* __restrict__ h0,
                const float* __restrict__ W, const float* __restrict__ bh,
                float* __restrict__ out, int T, int B, int H, Quant qin, Quant qout) {
  const int hv = H / VEC;                                   // vectors per row
  const long long chain = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (chain >= (long long)B * hv) return;
  const int b = (int)(chain / hv);
  const int i = (int)(chain % hv) * VEC;

  float wr[VEC], wz[VEC], wn[VEC], br[VEC], bz[VEC], bn[VEC], h[VEC];
  ld_plain<VEC>(W + i, wr);
  ld_plain<VEC>(W + H + i, wz);
  ld_plain<VEC>(W + 2 * H + i, wn);
  ld_plain<VEC>(bh + i, br);
  ld_plain<VEC>(bh + H + i, bz);
  ld_plain<VEC>(bh + 2 * H + i, bn);
  ld_plain<VEC>(h0 + (size_t)b * H + i, h);

  const size_t gi_step = (size_t)B * 3 * H;
  const size_t out_step = (size_t)B * H;
  const float* gp = gi + (size_t)b * 3 * H + i;
  float* op = out + (size_t)b * H + i;

  float gr[PF][VEC], gz[PF][VEC], gn[PF][VEC];
#pragma unroll
  for (int p = 0; p < PF; ++p) {
    if (p < T) {
      ld_stream<VEC>(gp + p * gi_step, gr[p]);
      ld_stream<VEC>(gp + p * gi_step + H, gz[p]);
      ld_stream<VEC>(gp + p * gi_step + 2 * H, gn[p]);
    }
  }

  for (int t0 = 0; t0 < T; t0 += PF) {
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int t = t0 + p;
      if (t < T) {
        float o[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          const float hq = fake_quant<QIN>(h[v], qin);
          const float ghr = wr[v] * hq + br[v];
          const float ghz = wz[v] * hq + bz[v];
          const float ghn = wn[v] * hq + bn[v];
          const GateOut g = gru_gates(gr[p][v], gz[p][v], gn[p][v], ghr, ghz, ghn, h[v]);
          h[v] = fake_quant<QOUT>(g.h_raw, qout);
          o[v] = h[v];
        }
        st_vec<VEC>(op + (size_t)t * out_step, o);
        const int tn = t + PF;
        if (tn < T) {
          ld_stream<VEC>(gp + tn * gi_step, gr[p]);
          ld_stream<VEC>(gp + tn * gi_step + H, gz[p]);
          ld_stream<VEC>(gp + tn * gi_step + 2 * H, gn[p]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// forward, TMA-staged (large problems)
// ---------------------------------------------------------------------------
// The register ring above cannot keep more than a few loads per warp in flight: a warp has
// only a handful of scoreboards, so waiting for an old load also waits for the youngest one.
// Here gi is staged through shared memory instead: one elected thread issues bulk copies
// (cp.async.bulk, the 1-D TMA path) DT_STAGES time steps ahead, completion is counted on an
// mbarrier per stage, and the threads of the CTA only ever read shared memory.  A CTA owns
// 256 adjacent hidden units of one batch row (3 x 1 KB per step); small CTAs keep the 148 SMs
// evenly loaded (about seven CTAs per SM at B*H = 256 Ki).  With gi off the critical path the
// kernel is bound by instruction issue (two sigmoids, a tanh and two exact fake-quants cost
// about 110 instructions per element-step), not by HBM.
constexpr int DT_STAGES = 8;
constexpr int DT_WAIT_LIMIT = 1 << 20;

static __device__ int g_diag_status;     // set to 1 if a bounded wait gave up

__device__ __forceinline__ unsigned dt_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dt_bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool dt_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// SAME: both quantisers are the same grid, so fq_in(h_t) = h_t for every t >= 0 (h_t is already a
// grid value) and only h0 needs the input rounding.
template <int DT_VEC, int DT_THREADS, bool QIN, bool QOUT, bool SAME>
__global__ void __launch_bounds__(DT_THREADS)
diag_fwd_tma_kernel(const float* __restrict__ gi, const float* __restrict__ h0,
                    const float* __restrict__ W, const float* __restrict__ bh,
                    float* __restrict__ out, int T, int B, int H, Quant qin, Quant qout) {
  constexpr int DT_COLS = DT_THREADS * DT_VEC;
  __shared__ __align__(128) float stage[DT_STAGES][3][DT_COLS];
  __shared__ __align__(8) unsigned long long full[DT_STAGES];
  const int tid = threadIdx.x;
  const int b = blockIdx.y;
  const int i0 = blockIdx.x * DT_COLS;
  const int ncols = min(DT_COLS, H - i0);                 // multiple of 4 (H % 4 == 0)
  const unsigned seg_bytes = (unsigned)ncols * sizeof(float);
  const bool active = DT_VEC * tid < ncols;
  const int i = i0 + DT_VEC * tid;

  const size_t gi_step = (size_t)B * 3 * H;
  const size_t out_step = (size_t)B * H;
  const float* grow = gi + (size_t)b * 3 * H + i0;        // + t*gi_step + g*H

  auto issue = [&](int t) {                                // thread 0 only
    const int s = t % DT_STAGES;
    const unsigned bar = dt_smem(&full[s]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(3u * seg_bytes) : "memory");
#pragma unroll
    for (int g = 0; g < 3; ++g)
      dt_bulk_load(dt_smem(&stage[s][g][0]), grow + (size_t)t * gi_step + (size_t)g * H, seg_bytes, bar);
  };

  if (tid == 0) {
    for (int s = 0; s < DT_STAGES; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dt_smem(&full[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int t = 0; t < DT_STAGES && t < T; ++t) issue(t);
  }

  float wr[DT_VEC], wz[DT_VEC], wn[DT_VEC], br[DT_VEC], bz[DT_VEC], bn[DT_VEC], h[DT_VEC];
#pragma unroll
  for (int v = 0; v < DT_VEC; ++v) { wr[v] = wz[v] = wn[v] = br[v] = bz[v] = bn[v] = h[v] = 0.f; }
  if (active) {
    ld_plain<DT_VEC>(W + i, wr); ld_plain<DT_VEC>(W + H + i, wz); ld_plain<DT_VEC>(W + 2 * H + i, wn);
    ld_plain<DT_VEC>(bh + i, br); ld_plain<DT_VEC>(bh + H + i, bz); ld_plain<DT_VEC>(bh + 2 * H + i, bn);
    ld_plain<DT_VEC>(h0 + (size_t)b * H + i, h);
  }
  __syncthreads();                                         // barriers initialised before anyone polls

  float hq[DT_VEC];
#pragma unroll
  for (int v = 0; v < DT_VEC; ++v) hq[v] = fake_quant<QIN>(h[v], qin);

  float* op = out + (size_t)b * H + i;
  bool dead = false;
  for (int t = 0; t < T; ++t) {
    const int s = t % DT_STAGES;
    const unsigned bar = dt_smem(&full[s]);
    const unsigned parity = (unsigned)(t / DT_STAGES) & 1u;
    if (!dead) {
      int spin = 0;
      while (!dt_try_wait(bar, parity)) {
        if (++spin > DT_WAIT_LIMIT) { dead = true; atomicExch(&g_diag_status, 1); break; }
      }
    }
    float gr[DT_VEC], gz[DT_VEC], gn[DT_VEC];
    if (active) {
      ld_plain<DT_VEC>(&stage[s][0][DT_VEC * tid], gr);
      ld_plain<DT_VEC>(&stage[s][1][DT_VEC * tid], gz);
      ld_plain<DT_VEC>(&stage[s][2][DT_VEC * tid], gn);
    }
    __syncthreads();                                       // stage s has been read by everyone
    if (tid == 0 && t + DT_STAGES < T) issue(t + DT_STAGES);
    if (active) {
      float o[DT_VEC];
#pragma unroll
      for (int v = 0; v < DT_VEC; ++v) {
        const float ghr = wr[v] * hq[v] + br[v];
        const float ghz = wz[v] * hq[v] + bz[v];
        const float ghn = wn[v] * hq[v] + bn[v];
        const GateOut g = gru_gates(gr[v], gz[v], gn[v], ghr, ghz, ghn, h[v]);
        h[v] = fake_quant<QOUT>(g.h_raw, qout);
        hq[v] = SAME ? h[v] : fake_quant<QIN>(h[v], qin);
        o[v] = h[v];
      }
      st_vec<DT_VEC>(op + (size_t)t * out_step, o);
    }
  }
}

int diag_read_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_diag_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_diag_status, &z, sizeof(int));
  }
  return v;
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
// Block = (32 hidden vectors) x (BY batch rows).  Each thread walks t = T-1..0 for
// its chain; the six per-unit sums (dW r,z,n and dbh r,z,n) are reduced over the
// BY rows of the block in shared memory and written as one partial row per block
// row-group: partial[part][6][H].  A second kernel sums the partial rows in a
// fixed order, which keeps the result bit-reproducible run to run.
constexpr int DIAG_BY = 4;

template <int VEC, int PF, bool QIN, bool QOUT>
__global__ void __launch_bounds__(32 * DIAG_BY)
diag_bwd_kernel(const float* __restrict__ gi, const float* __restrict__ h0,
                const float* __restrict__ W, const float* __restrict__ bh,
                const float* __restrict__ out, const float* __restrict__ dout,
                float* __restrict__ dgi, float* __restrict__ dh0,
                float* __restrict__ partial, int T, int B, int H, Quant qin, Quant qout) {
  const int hv = H / VEC;
  const int iv = blockIdx.x * 32 + threadIdx.x;
  const int b = blockIdx.y * DIAG_BY + threadIdx.y;
  const bool active = (iv < hv) && (b < B);
  const int i = iv * VEC;

  float acc[6][VEC];
#pragma unroll
  for (int k = 0; k < 6; ++k)
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[k][v] = 0.f;

  if (active) {
    float wr[VEC], wz[VEC], wn[VEC], br[VEC], bz[VEC], bn[VEC], dh_acc[VEC];
    ld_plain<VEC>(W + i, wr);
    ld_plain<VEC>(W + H + i, wz);
    ld_plain<VEC>(W + 2 * H + i, wn);
    ld_plain<VEC>(bh + i, br);
    ld_plain<VEC>(bh + H + i, bz);
    ld_plain<VEC>(bh + 2 * H + i, bn);
#pragma unroll
    for (int v = 0; v < VEC; ++v) dh_acc[v] = 0.f;

    const size_t gi_step = (size_t)B * 3 * H;
    const size_t out_step = (size_t)B * H;
    const float* gp = gi + (size_t)b * 3 * H + i;
    float* dgp = dgi + (size_t)b * 3 * H + i;
    const float* op = out + (size_t)b * H + i;
    const float* dop = dout + (size_t)b * H + i;
    const float* h0p = h0 + (size_t)b * H + i;

    // ring slot p holds step t = T-1-(k*PF+p)
    float gr[PF][VEC], gz[PF][VEC], gn[PF][VEC], hp[PF][VEC], dd[PF][VEC];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int t = T - 1 - p;
      if (t >= 0) {
        ld_stream<VEC>(gp + t * gi_step, gr[p]);
        ld_stream<VEC>(gp + t * gi_step + H, gz[p]);
        ld_stream<VEC>(gp + t * gi_step + 2 * H, gn[p]);
        ld_stream<VEC>(dop + t * out_step, dd[p]);
        if (t > 0) ld_stream<VEC>(op + (size_t)(t - 1) * out_step, hp[p]);
        else ld_plain<VEC>(h0p, hp[p]);
      }
    }

    for (int s0 = 0; s0 < T; s0 += PF) {
#pragma unroll
      for (int p = 0; p < PF; ++p) {
        const int t = T - 1 - (s0 + p);
        if (t >= 0) {
          float o_r[VEC], o_z[VEC], o_n[VEC];
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            const float h_prev = hp[p][v];
            const float hq = fake_quant<QIN>(h_prev, qin);
            const float ghr = wr[v] * hq + br[v];
            const float ghz = wz[v] * hq + bz[v];
            const float ghn = wn[v] * hq + bn[v];
            const GateOut g = gru_gates(gr[p][v], gz[p][v], gn[p][v], ghr, ghz, ghn, h_prev);
            float dh = dd[p][v] + dh_acc[v];
            dh = dh * ste_mask<QOUT>(g.h_raw, qout);
            const GateGrad q = gru_gate_grads(dh, g.r, g.z, g.n, ghn, h_prev);
            o_r[v] = q.dgr; o_z[v] = q.dgz; o_n[v] = q.dgn;
            acc[0][v] += q.dgr * hq;
            acc[1][v] += q.dgz * hq;
            acc[2][v] += q.dghn * hq;
            acc[3][v] += q.dgr;
            acc[4][v] += q.dgz;
            acc[5][v] += q.dghn;
            float via = q.dgr * wr[v] + q.dgz * wz[v] + q.dghn * wn[v];
            via = via * ste_mask<QIN>(h_prev, qin);
            dh_acc[v] = via + q.dh_direct;
          }
          st_stream<VEC>(dgp + t * gi_step, o_r);
          st_stream<VEC>(dgp + t * gi_step + H, o_z);
          st_stream<VEC>(dgp + t * gi_step + 2 * H, o_n);
          const int tn = t - PF;
          if (tn >= 0) {
            ld_stream<VEC>(gp + tn * gi_step, gr[p]);
            ld_stream<VEC>(gp + tn * gi_step + H, gz[p]);
            ld_stream<VEC>(gp + tn * gi_step + 2 * H, gn[p]);
            ld_stream<VEC>(dop + tn * out_step, dd[p]);
            if (tn > 0) ld_stream<VEC>(op + (size_t)(tn - 1) * out_step, hp[p]);
            else ld_plain<VEC>(h0p, hp[p]);
          }
        }
      }
    }
    st_vec<VEC>(dh0 + (size_t)b * H + i, dh_acc);
  }

  // reduce the six sums over the BY rows of this block (fixed order), one partial row out
  __shared__ float red[DIAG_BY][6][32 * VEC];
#pragma unroll
  for (int k = 0; k < 6; ++k)
#pragma unroll
    for (int v = 0; v < VEC; ++v) red[threadIdx.y][k][threadIdx.x * VEC + v] = acc[k][v];
  __syncthreads();
  if (threadIdx.y == 0 && iv < hv) {
#pragma unroll
    for (int k = 0; k < 6; ++k) {
      float s[VEC];
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        float a = red[0][k][threadIdx.x * VEC + v];
#pragma unroll
        for (int y = 1; y < DIAG_BY; ++y) a += red[y][k][threadIdx.x * VEC + v];
        s[v] = a;
      }
      st_vec<VEC>(partial + ((size_t)blockIdx.y * 6 + k) * H + i, s);
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int pick_vec(int B, int H, bool ptr_ok) {
  // Prefer the widest vector that still leaves enough threads to fill the machine.
  const long long chains = (long long)B * H;
  const long long want_threads = 148LL * 512;
  if (ptr_ok && H % 4 == 0 && chains / 4 >= want_threads) return 4;
  if (ptr_ok && H % 2 == 0 && chains / 2 >= want_threads) return 2;
  return 1;
}

size_t diag_bwd_workspace_bytes(int T, int B, int H) {
  (void)T;
  return align_up((size_t)cdiv(B, DIAG_BY) * 6 * H * sizeof(float), 256);
}

template <int VEC, int PF>
static void launch_fwd(const float* gi, const float* h0, const float* W, const float* bh, float* out,
                       int T, int B, int H, Quant qi, Quant qo, cudaStream_t st) {
  const long long threads = (long long)B * (H / VEC);
  const int block = 128;
  const unsigned grid = (unsigned)((threads + block - 1) / block);
#define DIAG_FWD(QI, QO) \
  diag_fwd_kernel<VEC, PF, QI, QO><<<grid, block, 0, st>>>(gi, h0, W, bh, out, T, B, H, qi, qo)
  if (qi.enabled) { if (qo.enabled) DIAG_FWD(true, true); else DIAG_FWD(true, false); }
  else            { if (qo.enabled) DIAG_FWD(false, true); else DIAG_FWD(false, false); }
#undef DIAG_FWD
  note_launch();
}

int diag_forward(const float* gi, const float* h0, const float* W, const float* bh, float* out,
                 int T, int B, int H, Quant qi, Quant qo, cudaStream_t st) {
  const bool ok = aligned16(gi) && aligned16(h0) && aligned16(W) && aligned16(bh) && aligned16(out);
  const bool no_tma = test_kernel_choice(1) != 0;       // test hook: register-ring kernel on every shape
  if (!no_tma && ok && H % 4 == 0 && T >= DT_STAGES && (long long)B * H >= 65536 && B <= 65535) {
    // 128 threads x 2 units: the best of the (units per thread, threads) shapes measured on B200
    constexpr int V = 2, N = 128;
    const dim3 grid(cdiv(H, V * N), B);
#define DIAG_TMA(QI, QO, SM) \
    diag_fwd_tma_kernel<V, N, QI, QO, SM><<<grid, N, 0, st>>>(gi, h0, W, bh, out, T, B, H, qi, qo)
    const bool same = qi.enabled && qo.enabled && qi.scale == qo.scale && qi.qmin == qo.qmin && qi.qmax == qo.qmax;
    if (qi.enabled) { if (same) DIAG_TMA(true, true, true); else if (qo.enabled) DIAG_TMA(true, true, false);
                      else DIAG_TMA(true, false, false); }
    else            { if (qo.enabled) DIAG_TMA(false, true, false); else DIAG_TMA(false, false, false); }
#undef DIAG_TMA
    note_launch();
    return check_launch("diag_fwd_tma_kernel");
  }
  const int vec = pick_vec(B, H, ok);
  if (vec == 4) launch_fwd<4, 4>(gi, h0, W, bh, out, T, B, H, qi, qo, st);
  else if (vec == 2) launch_fwd<2, 6>(gi, h0, W, bh, out, T, B, H, qi, qo, st);
  else launch_fwd<1, 8>(gi, h0, W, bh, out, T, B, H, qi, qo, st);
  return check_launch("diag_fwd_kernel");
}

template <int VEC, int PF>
static void launch_bwd(const float* gi, const float* h0, const float* W, const float* bh,
                       const float* out, const float* dout, float* dgi, float* dh0, float* partial,
                       int T, int B, int H, Quant qi, Quant qo, cudaStream_t st) {
  dim3 block(32, DIAG_BY);
  dim3 grid(cdiv(H / VEC, 32), cdiv(B, DIAG_BY));
#define DIAG_BWD(QI, QO)                                                                     \
  diag_bwd_kernel<VEC, PF, QI, QO><<<grid, block, 0, st>>>(gi, h0, W, bh, out, dout, dgi, dh0, \
                                                           partial, T, B, H, qi, qo)
  if (qi.enabled) { if (qo.enabled) DIAG_BWD(true, true); else DIAG_BWD(true, false); }
  else            { if (qo.enabled) DIAG_BWD(false, true); else DIAG_BWD(false, false); }
#undef DIAG_BWD
  note_launch();
}

int diag_backward(const float* gi, const float* h0, const float* W, const float* bh,
                  const float* out, const float* dout, float* dgi, float* dh0, float* dW, float* dbh,
                  void* workspace, int T, int B, int H, Quant qi, Quant qo, cudaStream_t st) {
  float* partial = static_cast<float*>(workspace);
  if (cdiv(B, DIAG_BY) > 65535) return B200GRU_UNSUPPORTED;        // grid.y of the backward kernel
  const bool ok = aligned16(gi) && aligned16(h0) && aligned16(W) && aligned16(bh) && aligned16(out) &&
                  aligned16(dout) && aligned16(dgi) && aligned16(dh0) && aligned16(partial);
  const int vec = pick_vec(B, H, ok);
  if (vec == 4) launch_bwd<4, 2>(gi, h0, W, bh, out, dout, dgi, dh0, partial, T, B, H, qi, qo, st);
  else if (vec == 2) launch_bwd<2, 3>(gi, h0, W, bh, out, dout, dgi, dh0, partial, T, B, H, qi, qo, st);
  else launch_bwd<1, 4>(gi, h0, W, bh, out, dout, dgi, dh0, partial, T, B, H, qi, qo, st);
  int rc = check_launch("diag_bwd_kernel");
  if (rc) return rc;
  // partial[part][0..2][H] -> dW[3][H];  partial[part][3..5][H] -> dbh[3H]
  const int nparts = cdiv(B, DIAG_BY);
  launch_reduce_partials(partial, nparts, (size_t)6 * H, (size_t)3 * H, dW, st);
  launch_reduce_partials(partial + (size_t)3 * H, nparts, (size_t)6 * H, (size_t)3 * H, dbh, st);
  return check_launch("reduce_partials");
}

// ---------------------------------------------------------------------------
// backward without caller scratch
// ---------------------------------------------------------------------------
// Some hosts of this library may not allocate device memory at all: a plugin that runs
// inside another runtime's memory budget, or a caller on a path where cudaMalloc is
// off limits (it synchronises the device and can fail under memory pressure).  For them
// the partial-sum scratch of the diagonal backward lives in this fixed array.  Every
// process that loads the library pays for it on each GPU it touches, until exit.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200GRU_NOALLOC_SCRATCH_BYTES];

// The array's name is only a host-side handle; kernels need its device address, which
// differs per GPU.  Looked up once per device (with that device current) and cached in a
// fixed table -- no allocation anywhere on this path.
static int noalloc_scratch_address(float** out) {
  constexpr int MAX_DEV = 64;
  static std::mutex mu;
  static float* table[MAX_DEV] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return B200GRU_LAUNCH_FAILURE;
  std::lock_guard<std::mutex> lk(mu);
  if (table[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess) {
      check_launch("cudaGetSymbolAddress");                 // records the CUDA error text
      return B200GRU_LAUNCH_FAILURE;
    }
    if (p == nullptr) return B200GRU_LAUNCH_FAILURE;
    table[dev] = static_cast<float*>(p);
  }
  *out = table[dev];
  return B200GRU_OK;
}

}  // namespace b200gru

extern "C" int b200gru_diagonal_backward_noalloc(const float* gi, const float* h0, const float* Wh_diag,
                                                 const float* bh_cat, const float* out, const float* dout,
                                                 int T, int B, int H, const b200gru_quant* q_in,
                                                 const b200gru_quant* q_out, float* dgi, float* dh0,
                                                 float* dWh_diag, float* dbh, void* stream) {
  using namespace b200gru;
  if (!gi || !h0 || !Wh_diag || !bh_cat || !out || !dout || !dgi || !dh0 || !dWh_diag || !dbh)
    return B200GRU_INVALID_ARGUMENT;
  if (T <= 0 || B <= 0 || H <= 0) return B200GRU_INVALID_ARGUMENT;
  if (q_in && q_in->enabled && !(q_in->scale > 0.f)) return B200GRU_INVALID_ARGUMENT;
  if (q_out && q_out->enabled && !(q_out->scale > 0.f)) return B200GRU_INVALID_ARGUMENT;
  if (diag_bwd_workspace_bytes(T, B, H) > (size_t)B200GRU_NOALLOC_SCRATCH_BYTES) return B200GRU_SCRATCH_EXCEEDED;
  if (cdiv(B, DIAG_BY) > 65535) return B200GRU_UNSUPPORTED;        // grid.y of the backward kernel
  float* scratch = nullptr;
  const int rc = noalloc_scratch_address(&scratch);
  if (rc) return rc;
  // Every element of the scratch that the reduction reads is first written by this call's
  // backward kernel, so nothing has to be cleared; what an earlier call left is ignored.
  return diag_backward(gi, h0, Wh_diag, bh_cat, out, dout, dgi, dh0, dWh_diag, dbh, scratch, T, B, H,
                       make_quant(q_in), make_quant(q_out), static_cast<cudaStream_t>(stream));
}
