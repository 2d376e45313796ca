// Dense scan at GEMM-sized batch on the tensor cores: one tcgen05 GEMM plus one elementwise gate
// kernel per time step; the stream order between launches is the recurrence.
//
// The cluster kernels of block_scan.cu keep a CTA's weight slice in shared memory and pay a fixed
// latency per step; once the slice no longer fits a 16-CTA cluster (H >= 544) and the batch is a
// real GEMM dimension (B >= 128), every step is a compute-bound product and runs here:
//
//   forward  step t : gh[B,3H]  = op(h_{t-1}) . W^T   (tc_gemm)   ->  gates, out[t], save, op(h_t)
//   backward step t : via[B,H]  = op(dgh_t)   . W     (tc_gemm, split over K)
//                     -> dh_{t-1}, STE masks, gate gradients of step t-1, dgi[t-1], op(dgh_{t-1})
//   every TC steps  : dW       += op(dgh)^T . op(h)   over the rows of the last TC steps
//
// op() is the operand form of the GEMM core: an fp32 tensor becomes three bf16 planes; a tensor on
// an int8 grid (the fake-quantised hidden state; weights handed over as int8 codes with one scale
// per output row) becomes one exact plane of integer codes, and where both operands of the forward
// product are codes the product is an exact int8 x int8 -> int32 contraction.  Scales are applied
// to the finished sums (or, for the contraction index of the backward product, folded into the
// fp32 operand before it is split).
//
// Reference: the same recurrence as src/gru_qat/triton_kernels/scan.py:120-184 (forward) and
// scan.py:389-616 (backward), where tl.dot tiles and a spin barrier across batch tiles play the
// roles of the GEMM and of the launch boundary.

#include <cstring>

#include <cuda_bf16.h>

#include "block_scan.cuh"
#include "butterfly_scan.cuh"
#include "tc_common.cuh"
#include "tc_gemm.cuh"
#include "tc_scan.cuh"
#include "tc_step.cuh"

namespace b200gru {
namespace tc {

namespace {

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4s(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }

__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 a, __nv_bfloat16 b) {
  return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}

// Three bf16 terms of four floats -> dst[pl * plane_stride + (0..3)]
__device__ __forceinline__ void store_planes4(__nv_bfloat16* dst, size_t plane_stride, int planes, float (&x)[4]) {
  for (int pl = 0; pl < planes; ++pl) {
    __nv_bfloat16 h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      h[e] = __float2bfloat16_rn(x[e]);
      x[e] = x[e] - __bfloat162float(h[e]);
    }
    uint2 o;
    o.x = pack_bf16(h[0], h[1]);
    o.y = pack_bf16(h[2], h[3]);
    *reinterpret_cast<uint2*>(dst + (size_t)pl * plane_stride) = o;
  }
}

// Operand form of four hidden values.  mode 0: int8 codes; 1: bf16 codes; 2: three bf16 planes of
// fq_in(h) (or of h itself when the input quantiser is off).
__device__ __forceinline__ void store_h_operand(void* base, size_t elem_off, size_t plane_stride, int mode,
                                                const float (&h)[4], const Quant& qin) {
  if (mode == 0 || mode == 1) {
    float c[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) c[e] = fminf(fmaxf(fq_code(h[e], qin), qin.qmin), qin.qmax);
    if (mode == 0) {
      char4 o = make_char4((signed char)(int)c[0], (signed char)(int)c[1], (signed char)(int)c[2], (signed char)(int)c[3]);
      *reinterpret_cast<char4*>(static_cast<signed char*>(base) + elem_off) = o;
    } else {
      uint2 o;
      o.x = pack_bf16(__float2bfloat16_rn(c[0]), __float2bfloat16_rn(c[1]));
      o.y = pack_bf16(__float2bfloat16_rn(c[2]), __float2bfloat16_rn(c[3]));
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + elem_off) = o;
    }
  } else {
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = qin.enabled ? fake_quant<true>(h[e], qin) : h[e];
    store_planes4(static_cast<__nv_bfloat16*>(base) + elem_off, plane_stride, 3, v);
  }
}

// ---- weights -------------------------------------------------------------------------------------
// int8 codes -> bf16 codes (exact)
__global__ void __launch_bounds__(256)
codes_to_bf16_kernel(const signed char* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n4) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const char4 c = reinterpret_cast<const char4*>(src)[i];
  uint2 o;
  o.x = pack_bf16(__float2bfloat16_rn((float)c.x), __float2bfloat16_rn((float)c.y));
  o.y = pack_bf16(__float2bfloat16_rn((float)c.z), __float2bfloat16_rn((float)c.w));
  reinterpret_cast<uint2*>(dst)[i] = o;
}

// ---- forward -------------------------------------------------------------------------------------
struct FwdStepArgs {
  const float* gi;       // [T][B][3H]
  const float* gh;       // [B][3H], hidden bias included
  const float* h_prev;   // [B][H]: h0 or out[t-1]
  float* out_t;          // [B][H]
  float* save;           // [4][T][B][H] or NULL
  void* op_next;         // operand form of h_t for step t+1 (NULL at the last step)
  size_t op_plane_stride;
  int op_mode;
  int t, T, B, H;
  Quant qin, qout;
};

__global__ void __launch_bounds__(256)
h0_operand_kernel(const float* __restrict__ h0, void* op, size_t plane_stride, int mode, int n4, Quant qin) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n4) return;
  const float4 v = ld4(h0 + (size_t)i * 4);
  const float h[4] = {v.x, v.y, v.z, v.w};
  store_h_operand(op, (size_t)i * 4, plane_stride, mode, h, qin);
}

__global__ void __launch_bounds__(256)
gate_fwd_kernel(const FwdStepArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int H4 = a.H >> 2;
  const int idx = blockIdx.x * 256 + threadIdx.x;
  if (idx >= a.B * H4) return;
  const int b = idx / H4, u = (idx - b * H4) * 4;
  const int H = a.H;
  const float* g = a.gi + ((size_t)a.t * a.B + b) * 3 * H + u;
  const float4 gr = ld4s(g), gz = ld4s(g + H), gn = ld4s(g + 2 * H);
  const float* hh = a.gh + (size_t)b * 3 * H + u;
  const float4 hr = ld4s(hh), hz = ld4s(hh + H), hn = ld4s(hh + 2 * H);
  const float4 hp = ld4(a.h_prev + (size_t)b * H + u);
  const float gir[4] = {gr.x, gr.y, gr.z, gr.w}, giz[4] = {gz.x, gz.y, gz.z, gz.w}, gin[4] = {gn.x, gn.y, gn.z, gn.w};
  const float ghr[4] = {hr.x, hr.y, hr.z, hr.w}, ghz[4] = {hz.x, hz.y, hz.z, hz.w}, ghn[4] = {hn.x, hn.y, hn.z, hn.w};
  const float hpv[4] = {hp.x, hp.y, hp.z, hp.w};
  float r[4], z[4], n[4], hnew[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const GateOut go = gru_gates(gir[e], giz[e], gin[e], ghr[e], ghz[e], ghn[e], hpv[e]);
    r[e] = go.r; z[e] = go.z; n[e] = go.n;
    hnew[e] = a.qout.enabled ? fake_quant<true>(go.h_raw, a.qout) : go.h_raw;
  }
  const size_t o = (size_t)b * H + u;
  *reinterpret_cast<float4*>(a.out_t + o) = make_float4(hnew[0], hnew[1], hnew[2], hnew[3]);
  if (a.save != nullptr) {
    const size_t comp = (size_t)a.T * a.B * H, so = (size_t)a.t * a.B * H + o;
    __stcs(reinterpret_cast<float4*>(a.save + so), make_float4(r[0], r[1], r[2], r[3]));
    __stcs(reinterpret_cast<float4*>(a.save + comp + so), make_float4(z[0], z[1], z[2], z[3]));
    __stcs(reinterpret_cast<float4*>(a.save + 2 * comp + so), make_float4(n[0], n[1], n[2], n[3]));
    __stcs(reinterpret_cast<float4*>(a.save + 3 * comp + so), make_float4(ghn[0], ghn[1], ghn[2], ghn[3]));
  }
  if (a.op_next != nullptr) store_h_operand(a.op_next, o, a.op_plane_stride, a.op_mode, hnew, a.qin);
}

// ---- backward ------------------------------------------------------------------------------------
struct BwdStepArgs {
  const float* h_t;        // [B][H] out[t] (mask of the via term); unused at t = T-1
  const float* h_prev;     // [B][H] out[t-1] or h0
  const float* S;          // [4][T][B][H]
  const float* dout;       // [T][B][H]
  const float* via;        // [nvia][B][H] partial products dgh_{t+1} . W (NULL at t = T-1)
  int nvia;
  float* direct;           // [B][H] dh * z of the step just processed (read, then overwritten)
  float* dgi;              // [T][B][3H]
  __nv_bfloat16* dgh_op;   // [3 planes][slot rows][3H]: rows of this step start at dgh_row0
  size_t dgh_plane_stride;
  const float* w_row_scale;  // [3H] or NULL: folded into dgh before the split
  void* h_op;              // operand form of h_{t-1} for the weight gradient, rows as dgh_op
  size_t h_plane_stride;
  int h_mode;              // 1: bf16 codes; 2: three planes
  int row0;                // first row of this step inside the chunk buffers
  int t, T, B, H;
  Quant qin, qout;
};

__global__ void __launch_bounds__(256)
gate_bwd_kernel(const BwdStepArgs a) {
  const int H4 = a.H >> 2;
  const int idx = blockIdx.x * 256 + threadIdx.x;
  if (idx >= a.B * H4) return;
  const int b = idx / H4, u = (idx - b * H4) * 4;
  const int H = a.H, B = a.B, t = a.t;
  const size_t o = (size_t)b * H + u;
  const size_t step = (size_t)B * H, comp = (size_t)a.T * step, so = (size_t)t * step + o;

  // inputs no kernel of the backward chain writes go in flight before the wait for the previous one
  pdl_launch_dependents();
  const float4 d4 = ld4s(a.dout + so);
  const float4 r4 = ld4s(a.S + so), z4 = ld4s(a.S + comp + so), n4 = ld4s(a.S + 2 * comp + so), g4 = ld4s(a.S + 3 * comp + so);
  const float4 h4 = ld4(a.h_prev + o);
  pdl_wait();

  float carry[4] = {0.f, 0.f, 0.f, 0.f};
  if (a.via != nullptr) {
    float4 s = ld4s(a.via + o);
    for (int p = 1; p < a.nvia; ++p) {
      const float4 v = ld4s(a.via + (size_t)p * step + o);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    const float4 dir = ld4(a.direct + o);
    const float4 ht = ld4(a.h_t + o);
    const float sv[4] = {s.x, s.y, s.z, s.w}, dv[4] = {dir.x, dir.y, dir.z, dir.w}, hv[4] = {ht.x, ht.y, ht.z, ht.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float mk = a.qin.enabled ? ste_mask<true>(hv[e], a.qin) : 1.0f;
      carry[e] = dv[e] + sv[e] * mk;
    }
  }
  const float dv[4] = {d4.x, d4.y, d4.z, d4.w}, rv[4] = {r4.x, r4.y, r4.z, r4.w}, zv[4] = {z4.x, z4.y, z4.z, z4.w};
  const float nv[4] = {n4.x, n4.y, n4.z, n4.w}, gv[4] = {g4.x, g4.y, g4.z, g4.w}, hv[4] = {h4.x, h4.y, h4.z, h4.w};
  float dgr[4], dgz[4], dgn[4], dghn[4], dir[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float dh = dv[e] + carry[e];
    if (a.qout.enabled) {
      const float h_raw = (1.0f - zv[e]) * nv[e] + zv[e] * hv[e];
      dh = dh * ste_mask<true>(h_raw, a.qout);
    }
    const GateGrad gg = gru_gate_grads(dh, rv[e], zv[e], nv[e], gv[e], hv[e]);
    dgr[e] = gg.dgr; dgz[e] = gg.dgz; dgn[e] = gg.dgn; dghn[e] = gg.dghn; dir[e] = gg.dh_direct;
  }
  float* d = a.dgi + ((size_t)t * B + b) * 3 * H + u;
  __stcs(reinterpret_cast<float4*>(d), make_float4(dgr[0], dgr[1], dgr[2], dgr[3]));
  __stcs(reinterpret_cast<float4*>(d + H), make_float4(dgz[0], dgz[1], dgz[2], dgz[3]));
  __stcs(reinterpret_cast<float4*>(d + 2 * H), make_float4(dgn[0], dgn[1], dgn[2], dgn[3]));
  *reinterpret_cast<float4*>(a.direct + o) = make_float4(dir[0], dir[1], dir[2], dir[3]);

  // operand planes of dgh (row scale of the weight codes folded in) and of h_{t-1}
  const size_t row = (size_t)a.row0 + b;
  if (a.w_row_scale != nullptr) {
    const float4 sr = ld4(a.w_row_scale + u), sz = ld4(a.w_row_scale + H + u), sn = ld4(a.w_row_scale + 2 * H + u);
    dgr[0] *= sr.x; dgr[1] *= sr.y; dgr[2] *= sr.z; dgr[3] *= sr.w;
    dgz[0] *= sz.x; dgz[1] *= sz.y; dgz[2] *= sz.z; dgz[3] *= sz.w;
    dghn[0] *= sn.x; dghn[1] *= sn.y; dghn[2] *= sn.z; dghn[3] *= sn.w;
  }
  __nv_bfloat16* dp = a.dgh_op + row * 3 * H + u;
  store_planes4(dp, a.dgh_plane_stride, 3, dgr);
  store_planes4(dp + H, a.dgh_plane_stride, 3, dgz);
  store_planes4(dp + 2 * H, a.dgh_plane_stride, 3, dghn);
  store_h_operand(a.h_op, row * H + u, a.h_plane_stride, a.h_mode, hv, a.qin);
}

// dh0 = direct_0 + mask_in(h0) * (dgh_0 . W)
__global__ void __launch_bounds__(256)
dh0_kernel(const float* __restrict__ via, int nvia, const float* __restrict__ direct, const float* __restrict__ h0,
           float* __restrict__ dh0, int n4, size_t step, Quant qin) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n4) return;
  const size_t o = (size_t)i * 4;
  float4 s = ld4s(via + o);
  for (int p = 1; p < nvia; ++p) {
    const float4 v = ld4s(via + (size_t)p * step + o);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  const float4 dir = ld4(direct + o), h = ld4(h0 + o);
  const float sv[4] = {s.x, s.y, s.z, s.w}, dv[4] = {dir.x, dir.y, dir.z, dir.w}, hv[4] = {h.x, h.y, h.z, h.w};
  float r[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) r[e] = dv[e] + sv[e] * (qin.enabled ? ste_mask<true>(hv[e], qin) : 1.0f);
  *reinterpret_cast<float4*>(dh0 + o) = make_float4(r[0], r[1], r[2], r[3]);
}

// v[i] = num / w_row_scale[i]  (row scale of the weight gradient product)
__global__ void inv_scale_kernel(const float* __restrict__ s, float* __restrict__ out, int n, float num) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = num / s[i];
}

bool codes_fit_int8(const Quant& q) { return q.enabled && q.qmin >= -128.f && q.qmax <= 127.f; }

// all plane pairs (i, j) with i + j <= 2, most significant first
int fill_pairs(int na, int nb, int* pa, int* pb) {
  int n = 0;
  for (int s = 0; s <= 2; ++s)
    for (int i = 0; i <= s; ++i) {
      const int j = s - i;
      if (i < na && j < nb) { pa[n] = i; pb[n] = j; ++n; }
    }
  return n;
}

struct Plan {
  int T, B, H;
  bool w_codes;          // weights given as int8 codes + row scales
  bool h_codes;          // hidden operand is integer codes (input quantiser on, range inside int8)
  bool i8;               // forward product int8 x int8
  int h_mode;            // forward operand form of h
  int w_planes;          // bf16 planes of W used by the bf16 products
  int tc_steps;          // time steps per weight-gradient chunk
  int via_splits;
  int dw_splits;
};

Plan make_plan(int T, int B, int H, bool w_codes, const Quant& qin) {
  Plan p;
  p.T = T; p.B = B; p.H = H;
  p.w_codes = w_codes;
  p.h_codes = codes_fit_int8(qin);
  p.i8 = p.w_codes && p.h_codes;
  p.h_mode = p.h_codes ? (p.i8 ? 0 : 1) : 2;
  p.w_planes = w_codes ? 1 : 3;
  int tcs = cdiv(8192, B);
  if (tcs > T) tcs = T;
  if (tcs < 1) tcs = 1;
  p.tc_steps = tcs;
  // backward product [B,3H] x [3H,H]: split the contraction until the grid covers the GPU
  TcGemm g;
  memset(&g, 0, sizeof(g));
  g.kind = TC_KIND_BF16; g.K = 3 * H;
  const int tiles = cdiv(B, 128) * cdiv(H, 256);
  int want = cdiv(132, tiles);
  if (want > 12) want = 12;
  p.via_splits = tc_gemm_splits(g, want);
  // weight gradient [3H, rows] x [rows, H] per chunk: 3H/128 * H/256 tiles
  const int wt = cdiv(3 * H, 128) * cdiv(H, 256);
  g.K = tcs * B;
  p.dw_splits = tc_gemm_splits(g, wt >= 120 ? 1 : cdiv(280, wt));
  return p;
}

size_t w_planes_bytes(const Plan& p) { return align_up((size_t)p.w_planes * 3 * p.H * p.H * 2, 256); }
size_t h_op_elem_bytes(int mode) { return mode == 0 ? 1 : 2; }
int h_op_planes(int mode) { return mode == 2 ? 3 : 1; }

}  // namespace

bool tc_dense_path(int B, int H) {
  const size_t slice = (size_t)3 * ((H + 15) / 16) * H * sizeof(float);
  return slice > (size_t)200 * 1024 && B >= 128 && H % 32 == 0;
}

static size_t fwd_scratch(int T, int B, int H, bool w_codes, const Quant& qin) {
  const Plan p = make_plan(T, B, H, w_codes, qin);
  size_t n = 0;
  if (!p.i8) n += w_planes_bytes(p);                                           // bf16 planes / codes of W
  n += align_up((size_t)2 * h_op_planes(p.h_mode) * B * H * h_op_elem_bytes(p.h_mode), 256);   // op(h), two steps
  n += align_up((size_t)B * 3 * H * sizeof(float), 256);                       // gh
  return n;
}

static size_t bwd_scratch(int T, int B, int H, bool w_codes, const Quant& qin) {
  const Plan p = make_plan(T, B, H, w_codes, qin);
  const size_t rows = (size_t)p.tc_steps * B;
  const int hm = p.h_codes ? 1 : 2;
  size_t n = w_planes_bytes(p);
  n += align_up((size_t)3 * rows * 3 * H * 2, 256);                            // op(dgh) of one chunk
  n += align_up((size_t)h_op_planes(hm) * rows * H * 2, 256);                  // op(h) of one chunk
  n += align_up((size_t)p.via_splits * B * H * sizeof(float), 256);            // via partials
  n += align_up((size_t)B * H * sizeof(float), 256);                           // direct
  n += align_up((size_t)p.dw_splits * 3 * H * H * sizeof(float), 256);         // dW partial accumulators
  n += align_up((size_t)3 * H * sizeof(float), 256);                           // row scale of the dW product
  n += bias_grads_scratch_bytes(T, B, H);
  return n;
}

// The hidden-state quantiser is not part of the shape, so the query covers both operand forms.
static Quant probe_quant(bool on) {
  Quant q;
  q.scale = 1.f; q.inv_scale = 1.f; q.qmin = on ? -127.f : 0.f; q.qmax = on ? 127.f : 0.f; q.enabled = on ? 1 : 0;
  return q;
}
size_t tc_dense_fwd_scratch_bytes(int T, int B, int H, bool w_codes) {
  const size_t a = fwd_scratch(T, B, H, w_codes, probe_quant(true)), b = fwd_scratch(T, B, H, w_codes, probe_quant(false));
  return a > b ? a : b;
}
size_t tc_dense_bwd_scratch_bytes(int T, int B, int H, bool w_codes) {
  const size_t a = bwd_scratch(T, B, H, w_codes, probe_quant(true)), b = bwd_scratch(T, B, H, w_codes, probe_quant(false));
  return a > b ? a : b;
}

// W operand for the bf16 products: planes of the fp32 weights, or the int8 codes as bf16
static int prepare_w_bf16(const TcWeights& w, int H, __nv_bfloat16* dst, cudaStream_t st) {
  const size_t n = (size_t)3 * H * H;
  if (w.codes != nullptr) {
    codes_to_bf16_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(w.codes, dst, n / 4);
    note_launch();
    return check_launch("codes_to_bf16_kernel");
  }
  return launch_split_planes(w.W, dst, n, n, 3, nullptr, 0, st);
}

int launch_tc_dense_forward(const float* gi, const float* h0, const TcWeights& w, const float* bh, float* out,
                            float* save, void* scratch, int T, int B, int H, Quant qin, Quant qout, cudaStream_t st) {
  const Plan p = make_plan(T, B, H, w.codes != nullptr, qin);
  char* ws = static_cast<char*>(scratch);
  __nv_bfloat16* wop = nullptr;
  if (!p.i8) {
    wop = reinterpret_cast<__nv_bfloat16*>(ws);
    ws += w_planes_bytes(p);
    int rc = prepare_w_bf16(w, H, wop, st);
    if (rc) return rc;
  }
  const int hp = h_op_planes(p.h_mode);
  const size_t heb = h_op_elem_bytes(p.h_mode);
  const size_t op_bytes = (size_t)hp * B * H * heb;
  char* op[2] = {ws, ws + op_bytes};
  ws += align_up(2 * op_bytes, 256);
  float* gh = reinterpret_cast<float*>(ws);

  const int n4 = B * (H / 4);
  h0_operand_kernel<<<cdiv(n4, 256), 256, 0, st>>>(h0, op[0], (size_t)B * H, p.h_mode, n4, qin);
  note_launch();
  int rc = check_launch("h0_operand_kernel");
  if (rc) return rc;

  if (p.i8) {
    // both operands are integer codes: one fused kernel per step (product + gates + next codes)
    FusedFwd f;
    rc = f.init(w.codes, reinterpret_cast<signed char*>(op[0]), reinterpret_cast<signed char*>(op[1]), gi, h0, out, save,
                T, B, H);
    if (rc) return rc;
    for (int t = 0; t < T; ++t) {
      rc = f.step(t, t & 1, w.row_scale, bh, (t + 1 < T) ? reinterpret_cast<signed char*>(op[(t + 1) & 1]) : nullptr,
                  qin.scale, qin, qout, st);
      if (rc) return rc;
    }
    return check_launch("tc_fwd_step_kernel");
  }

  TcGemm g;
  memset(&g, 0, sizeof(g));
  g.kind = p.i8 ? TC_KIND_I8 : TC_KIND_BF16;
  g.M = B; g.N = 3 * H; g.K = H;
  g.B = p.i8 ? static_cast<const void*>(w.codes) : static_cast<const void*>(wop);
  g.a_planes = hp; g.b_planes = p.i8 ? 1 : p.w_planes;
  g.lda = H; g.ldb = H; g.a_plane_stride = (long long)B * H; g.b_plane_stride = (long long)3 * H * H;
  g.npairs = fill_pairs(g.a_planes, g.b_planes, g.pa, g.pb);
  g.split_k = 1;
  g.alpha = p.h_codes ? qin.scale : 1.0f;
  g.col_scale = w.row_scale; g.bias = bh;
  g.C = gh; g.ldc = 3 * H; g.split_stride = 0;
  // narrow tiles when 256-wide ones leave most SMs idle
  const int t256 = cdiv(B, 128) * cdiv(3 * H, 256);
  g.tile_n = t256 >= 120 ? 256 : (2 * t256 >= 120 ? 128 : 64);
  if (2 * (g.a_planes * 16384 + g.b_planes * g.tile_n * 128) > TC_SMEM_BUDGET) g.tile_n = 128;

  FwdStepArgs a;
  memset(&a, 0, sizeof(a));
  a.gi = gi; a.gh = gh; a.save = save; a.T = T; a.B = B; a.H = H; a.qin = qin; a.qout = qout;
  a.op_plane_stride = (size_t)B * H; a.op_mode = p.h_mode;
  for (int t = 0; t < T; ++t) {
    g.A = op[t & 1];
    rc = launch_tc_gemm(g, st);
    if (rc) return rc;
    a.t = t;
    a.h_prev = (t == 0) ? h0 : out + (size_t)(t - 1) * B * H;
    a.out_t = out + (size_t)t * B * H;
    a.op_next = (t + 1 < T) ? op[(t + 1) & 1] : nullptr;
    launch_pdl(gate_fwd_kernel, dim3(cdiv(n4, 256)), dim3(256), 0, st, a);
    note_launch();
  }
  return check_launch("gate_fwd_kernel");
}

int launch_tc_dense_backward(const float* h0, const TcWeights& w, const float* out, const float* S, const float* dout,
                             float* dgi, float* dh0, float* dW, float* dbh, void* scratch, int T, int B, int H,
                             Quant qin, Quant qout, cudaStream_t st) {
  const Plan p = make_plan(T, B, H, w.codes != nullptr, qin);
  const size_t rows = (size_t)p.tc_steps * B;
  const int hm = p.h_codes ? 1 : 2;
  const int hpl = h_op_planes(hm);
  char* ws = static_cast<char*>(scratch);
  __nv_bfloat16* wop = reinterpret_cast<__nv_bfloat16*>(ws); ws += w_planes_bytes(p);
  __nv_bfloat16* dgh_op = reinterpret_cast<__nv_bfloat16*>(ws); ws += align_up((size_t)3 * rows * 3 * H * 2, 256);
  __nv_bfloat16* h_op = reinterpret_cast<__nv_bfloat16*>(ws); ws += align_up((size_t)hpl * rows * H * 2, 256);
  float* via = reinterpret_cast<float*>(ws); ws += align_up((size_t)p.via_splits * B * H * sizeof(float), 256);
  float* direct = reinterpret_cast<float*>(ws); ws += align_up((size_t)B * H * sizeof(float), 256);
  float* dw_part = reinterpret_cast<float*>(ws); ws += align_up((size_t)p.dw_splits * 3 * H * H * sizeof(float), 256);
  float* dw_scale = reinterpret_cast<float*>(ws); ws += align_up((size_t)3 * H * sizeof(float), 256);
  float* bias_part = reinterpret_cast<float*>(ws);

  int rc = prepare_w_bf16(w, H, wop, st);
  if (rc) return rc;
  const float h_scale = p.h_codes ? qin.scale : 1.0f;
  if (w.row_scale != nullptr) {
    inv_scale_kernel<<<cdiv(3 * H, 256), 256, 0, st>>>(w.row_scale, dw_scale, 3 * H, h_scale);
    note_launch();
  }

  // via[B,H] = op(dgh_t)[B,3H] . W[3H,H]   (W rows are the contraction index: MN-major B operand)
  TcGemm gv;
  memset(&gv, 0, sizeof(gv));
  gv.kind = TC_KIND_BF16;
  gv.M = B; gv.N = H; gv.K = 3 * H;
  gv.B = wop; gv.a_planes = 3; gv.b_planes = p.w_planes; gv.a_mn = 0; gv.b_mn = 1;
  gv.lda = 3 * H; gv.ldb = H; gv.a_plane_stride = (long long)rows * 3 * H; gv.b_plane_stride = (long long)3 * H * H;
  gv.npairs = fill_pairs(3, p.w_planes, gv.pa, gv.pb);
  gv.split_k = p.via_splits; gv.tile_n = 256;
  if (2 * (3 * 16384 + p.w_planes * 256 * 128) > TC_SMEM_BUDGET) gv.tile_n = 128;
  gv.alpha = 1.0f; gv.C = via; gv.ldc = H; gv.split_stride = (long long)B * H;

  // dW[3H,H] (+)= op(dgh)^T[3H,rows] . op(h)[rows,H] over one chunk of time steps
  TcGemm gw;
  memset(&gw, 0, sizeof(gw));
  gw.kind = TC_KIND_BF16;
  gw.M = 3 * H; gw.N = H;
  gw.A = dgh_op; gw.B = h_op; gw.a_planes = 3; gw.b_planes = hpl; gw.a_mn = 1; gw.b_mn = 1;
  gw.lda = 3 * H; gw.ldb = H; gw.a_plane_stride = (long long)rows * 3 * H; gw.b_plane_stride = (long long)rows * H;
  // Weight gradients are held to 1e-4 of their largest entry: the two leading planes of each fp32
  // operand (16 mantissa bits) and the cross products down to 2^-16 are enough (error about 1e-5 of
  // a term, averaged over rows * B terms); the chain product above keeps all three planes.
  gw.npairs = 0;
  for (int s2 = 0; s2 <= 1; ++s2)
    for (int i = 0; i <= s2; ++i) {
      const int j = s2 - i;
      if (j < hpl) { gw.pa[gw.npairs] = i; gw.pb[gw.npairs] = j; ++gw.npairs; }
    }
  gw.tile_n = 256;
  if (2 * (3 * 16384 + hpl * 256 * 128) > TC_SMEM_BUDGET) gw.tile_n = 128;
  gw.alpha = (w.row_scale != nullptr) ? 1.0f : h_scale;
  gw.row_scale = (w.row_scale != nullptr) ? dw_scale : nullptr;
  float* dw_dst = (p.dw_splits > 1) ? dw_part : dW;
  gw.C = dw_dst; gw.ldc = H; gw.split_stride = (long long)3 * H * H;

  BwdStepArgs a;
  memset(&a, 0, sizeof(a));
  a.S = S; a.dout = dout; a.direct = direct; a.dgi = dgi; a.nvia = p.via_splits;
  a.dgh_op = dgh_op; a.dgh_plane_stride = rows * 3 * H; a.w_row_scale = w.row_scale;
  a.h_op = h_op; a.h_plane_stride = rows * H; a.h_mode = hm;
  a.T = T; a.B = B; a.H = H; a.qin = qin; a.qout = qout;
  const int n4 = B * (H / 4);
  bool first_chunk = true;
  for (int t = T - 1; t >= 0; --t) {
    const int slot = t % p.tc_steps;
    a.t = t; a.row0 = slot * B;
    a.via = (t == T - 1) ? nullptr : via;
    a.h_t = out + (size_t)t * B * H;
    a.h_prev = (t == 0) ? h0 : out + (size_t)(t - 1) * B * H;
    launch_pdl(gate_bwd_kernel, dim3(cdiv(n4, 256)), dim3(256), 0, st, a);
    note_launch();
    gv.A = dgh_op + (size_t)slot * B * 3 * H;
    rc = launch_tc_gemm(gv, st);
    if (rc) return rc;
    if (slot == 0) {
      // the chunk [t, t + nsteps) is complete: its rows are contiguous from slot 0
      const int nsteps = ((t + p.tc_steps <= T) ? p.tc_steps : T - t);
      gw.K = nsteps * B;
      gw.split_k = tc_gemm_splits(gw, p.dw_splits);
      gw.accumulate = first_chunk ? 0 : 1;
      if (gw.split_k != p.dw_splits && first_chunk && p.dw_splits > 1) {
        // a short first chunk may use fewer K slices than the accumulators that are summed at the end
        cudaMemsetAsync(dw_part, 0, (size_t)p.dw_splits * 3 * H * H * sizeof(float), st);
        gw.accumulate = 1;
      }
      rc = launch_tc_gemm(gw, st);
      if (rc) return rc;
      first_chunk = false;
    }
  }
  dh0_kernel<<<cdiv(n4, 256), 256, 0, st>>>(via, p.via_splits, direct, h0, dh0, n4, (size_t)B * H, qin);
  note_launch();
  rc = check_launch("dh0_kernel");
  if (rc) return rc;
  if (p.dw_splits > 1) launch_reduce_partials(dw_part, p.dw_splits, (size_t)3 * H * H, (size_t)3 * H * H, dW, st);
  return launch_bias_grads(dgi, S, bias_part, dbh, T, B, H, st);
}


// ---- weight gradient of the dense cluster path on the tensor cores ----------------------------------
// dW[3H,H] = dgh^T[3H, T*B] . fq_in(h_prev)[T*B, H] with every operand known (the serial scan has
// finished): one pass writes the bf16 operand planes of dgh (dgh_n = dgi_n * r) and of h_{t-1},
// one GEMM with both operands MN-major contracts over the T*B rows.
struct WgOperandArgs {
  const float* dgi;        // [T*B][3H]
  const float* r;          // [T*B][H]
  const float* h0;         // [B][H]
  const float* out;        // [T][B][H]
  __nv_bfloat16* dgh_op;   // [2 planes][T*B][3H]
  __nv_bfloat16* h_op;     // [1 plane of codes | 2 planes][T*B][H]
  size_t rows;             // T*B
  int B, H, h_codes;
  Quant qin;
};

__global__ void __launch_bounds__(256)
wgrad_operands_kernel(const WgOperandArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int H4 = a.H >> 2;
  const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= a.rows * H4) return;
  const size_t row = idx / H4;
  const int u = (int)(idx - row * H4) * 4;
  const int H = a.H;
  const float* d = a.dgi + row * 3 * H + u;
  const float4 dr = ld4s(d), dz = ld4s(d + H), dn = ld4s(d + 2 * H);
  const float4 r4 = ld4s(a.r + row * H + u);
  const float4 hp = (row < (size_t)a.B) ? ld4(a.h0 + row * H + u) : ld4(a.out + (row - a.B) * H + u);
  float vr[4] = {dr.x, dr.y, dr.z, dr.w}, vz[4] = {dz.x, dz.y, dz.z, dz.w};
  float vn[4] = {dn.x * r4.x, dn.y * r4.y, dn.z * r4.z, dn.w * r4.w};
  const size_t dps = a.rows * 3 * H;
  __nv_bfloat16* dp = a.dgh_op + row * 3 * H + u;
  store_planes4(dp, dps, 2, vr);
  store_planes4(dp + H, dps, 2, vz);
  store_planes4(dp + 2 * H, dps, 2, vn);
  const float hv[4] = {hp.x, hp.y, hp.z, hp.w};
  if (a.h_codes) {
    store_h_operand(a.h_op, row * H + u, 0, 1, hv, a.qin);
  } else {
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = a.qin.enabled ? fake_quant<true>(hv[e], a.qin) : hv[e];
    store_planes4(a.h_op + row * H + u, a.rows * H, 2, v);
  }
}

bool tc_weight_grads_applies(int T, int B, int H) {
  return H % 8 == 0 && H >= 128 && (size_t)T * B >= 1024 && (size_t)T * B * 3 * H < ((size_t)1 << 31);
}

static TcGemm wgrad_gemm(int T, int B, int H, bool h_codes) {
  TcGemm g;
  memset(&g, 0, sizeof(g));
  const long long rows = (long long)T * B;
  g.kind = TC_KIND_BF16;
  g.M = 3 * H; g.N = H; g.K = (int)rows;
  g.a_planes = 2; g.b_planes = h_codes ? 1 : 2; g.a_mn = 1; g.b_mn = 1;
  g.lda = 3 * H; g.ldb = H; g.a_plane_stride = rows * 3 * H; g.b_plane_stride = rows * H;
  // two leading planes per fp32 operand and the cross products down to 2^-16: about 5e-6 of a term
  g.npairs = 0;
  for (int s2 = 0; s2 <= 1; ++s2)
    for (int i = 0; i <= s2; ++i) {
      const int j = s2 - i;
      if (j < g.b_planes) { g.pa[g.npairs] = i; g.pb[g.npairs] = j; ++g.npairs; }
    }
  // wide tiles: one k-block of the two A planes then feeds 256 columns (measured at c1: 31 K cycles
  // per CTA with 256-wide tiles and 4 K slices against 42 K with 128-wide ones)
  g.tile_n = g.N >= 256 ? 256 : 128;
  const int tiles = cdiv(g.M, 128) * cdiv(g.N, g.tile_n);
  // enough K slices to fill the SMs, at least 8 k-blocks each
  int want = tiles >= 148 ? 1 : cdiv(148, tiles);
  const int kb = cdiv(g.K, tc_gemm_kblock(g));
  if (want > kb / 8) want = kb / 8 > 0 ? kb / 8 : 1;
  g.split_k = tc_gemm_splits(g, want);
  g.ldc = H; g.split_stride = (long long)3 * H * H;
  g.alpha = 1.0f;
  return g;
}

size_t tc_weight_grads_scratch_bytes(int T, int B, int H, bool h_codes) {
  const size_t rows = (size_t)T * B;
  const TcGemm g = wgrad_gemm(T, B, H, h_codes);
  size_t n = align_up(2 * rows * 3 * H * 2, 256) + align_up((size_t)g.b_planes * rows * H * 2, 256);
  if (g.split_k > 1) n += align_up((size_t)g.split_k * 3 * H * H * sizeof(float), 256);
  return n;
}

int launch_tc_weight_grads(const float* dgi, const float* S, const float* h0, const float* out, Quant qin, float* dW,
                           void* scratch, int T, int B, int H, cudaStream_t st) {
  const bool h_codes = codes_fit_int8(qin);
  const size_t rows = (size_t)T * B;
  TcGemm g = wgrad_gemm(T, B, H, h_codes);
  char* ws = static_cast<char*>(scratch);
  __nv_bfloat16* dgh_op = reinterpret_cast<__nv_bfloat16*>(ws); ws += align_up(2 * rows * 3 * H * 2, 256);
  __nv_bfloat16* h_op = reinterpret_cast<__nv_bfloat16*>(ws); ws += align_up((size_t)g.b_planes * rows * H * 2, 256);
  float* part = reinterpret_cast<float*>(ws);

  WgOperandArgs a;
  memset(&a, 0, sizeof(a));
  a.dgi = dgi; a.r = S; a.h0 = h0; a.out = out; a.dgh_op = dgh_op; a.h_op = h_op;
  a.rows = rows; a.B = B; a.H = H; a.h_codes = h_codes ? 1 : 0; a.qin = qin;
  const size_t n4 = rows * (H / 4);
  launch_pdl(wgrad_operands_kernel, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, st, a);
  note_launch();
  int rc = check_launch("wgrad_operands_kernel");
  if (rc) return rc;
  g.A = dgh_op; g.B = h_op;
  g.alpha = h_codes ? qin.scale : 1.0f;
  g.C = g.split_k > 1 ? part : dW;
  rc = launch_tc_gemm(g, st);
  if (rc) return rc;
  if (g.split_k > 1) launch_reduce_partials(part, g.split_k, (size_t)3 * H * H, (size_t)3 * H * H, dW, st);
  return check_launch("weight gradient product");
}

}  // namespace tc
}  // namespace b200gru
