// Shared device helpers of the GRU scan kernels (sm_100a).
//
// Arithmetic contract (matches the reference's PyTorch path, gates ordered r,z,n):
//   fq(x; s,qmin,qmax) = clamp(rint(x / s), qmin, qmax) * s      true division, half-to-even
//   r = sigmoid(gi_r + gh_r)   z = sigmoid(gi_z + gh_z)   n = tanh(gi_n + r * gh_n)
//   h_raw = (1 - z) * n + z * h_prev
// The translation units are compiled with -fmad=false so the elementwise gate
// math rounds after every operation, as the eager reference does; dot products
// call fmaf() explicitly.
#pragma once

#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/b200gru.h"

namespace b200gru {

// Debug aid, compiled in only with -DB200GRU_PHASE_TIMING: thread 0 of CTA (0,0) adds the
// clock64() distance between consecutive marks of a step to g_phase_cycles[slot].
#ifdef B200GRU_PHASE_TIMING
static __device__ unsigned long long g_phase_cycles[16];   // one copy per translation unit
#define PHASE_DECL long long ph_last = 0; const bool ph_on = (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0)
#define PHASE_START() do { if (ph_on) ph_last = clock64(); } while (0)
#define PHASE_MARK(slot) do { if (ph_on) { long long ph_now = clock64(); \
    atomicAdd(&g_phase_cycles[slot], (unsigned long long)(ph_now - ph_last)); ph_last = ph_now; } } while (0)
#define B200GRU_DEFINE_PHASE_READER(name)                                                   \
  extern "C" void name(unsigned long long* out16, int reset) {                                \
    cudaDeviceSynchronize();                                                                  \
    cudaMemcpyFromSymbol(out16, b200gru::g_phase_cycles, sizeof(unsigned long long) * 16);    \
    if (reset) {                                                                              \
      unsigned long long z[16] = {0};                                                         \
      cudaMemcpyToSymbol(b200gru::g_phase_cycles, z, sizeof(z));                              \
    }                                                                                         \
  }
#else
#define B200GRU_DEFINE_PHASE_READER(name)
#define PHASE_DECL
#define PHASE_START()
#define PHASE_MARK(slot)
#endif

struct Quant {
  float scale;
  float inv_scale;   // RN(1 / scale), used by the exact division below
  float qmin;
  float qmax;
  int enabled;
};

// Correctly rounded float reciprocal of s: among the double-rounded candidate and its two
// neighbours pick the one whose product with s is closest to 1 (products of two floats are
// exact in double).
__host__ inline float exact_reciprocal(float s) {
  const float y = (float)(1.0 / (double)s);
  const float cand[3] = {y, nextafterf(y, 0.f), nextafterf(y, 2.f * y)};
  float best = y;
  double err = fabs(1.0 - (double)y * (double)s);
  for (int i = 1; i < 3; ++i) {
    const double e = fabs(1.0 - (double)cand[i] * (double)s);
    if (e < err) { err = e; best = cand[i]; }
  }
  return best;
}

__host__ inline Quant make_quant(const b200gru_quant* q) {
  Quant r;
  if (q == nullptr || !q->enabled) {
    r.scale = 1.f; r.inv_scale = 1.f; r.qmin = 0.f; r.qmax = 0.f; r.enabled = 0;
  } else {
    r.scale = q->scale; r.inv_scale = exact_reciprocal(q->scale);
    r.qmin = (float)q->qmin; r.qmax = (float)q->qmax; r.enabled = 1;
  }
  return r;
}

// 1 / (1 + e^-x): the reciprocal of a float is correctly rounded by rcp.rn, which is what the
// IEEE division 1.0f / y returns.
// e^-x through ex2.approx (relative error about |x| * 6e-8 + 2 ulp): the sigmoid then stays within
// 2e-7 of the exact value, far inside the 1e-5 parity bar, at a third of expf's instructions.
__device__ __forceinline__ float sigmoidf_acc(float x) {
  return __frcp_rn(1.0f + __expf(-x));
}

// x / s, correctly rounded (bit-identical to IEEE division), for the fixed divisor s of a
// quantizer: one multiply by RN(1/s) and one FMA-exact residual correction (Markstein).  The
// generic division routine costs about four times as many instructions.  If x * (1/s)
// overflows, the quotient is that infinity.
__device__ __forceinline__ float div_by_scale(float x, const Quant& q) {
  const float q0 = x * q.inv_scale;
  const float r = fmaf(-q0, q.scale, x);
  const float q1 = fmaf(r, q.inv_scale, q0);
  return (fabsf(q0) < 3.0e38f) ? q1 : q0;
}

// Unclamped integer code of x (as float), rint(x / s), saturated two codes outside [qmin, qmax]:
// the saturation changes neither the clamped code nor whether the code lies inside the range,
// and it keeps the value small enough for round-to-nearest-even by adding and subtracting
// 1.5 * 2^23 (two FADDs instead of a conversion instruction on the slow pipe).
__device__ __forceinline__ float fq_code(float x, const Quant& q) {
  float c = div_by_scale(x, q);
  c = fminf(fmaxf(c, q.qmin - 2.0f), q.qmax + 2.0f);
  const float magic = 12582912.0f;
  return (c + magic) - magic;
}

template <bool ON>
__device__ __forceinline__ float fake_quant(float x, const Quant& q) {
  if (!ON) return x;
  float c = fq_code(x, q);
  c = fminf(fmaxf(c, q.qmin), q.qmax);
  return c * q.scale;
}

// Straight-through mask: 1 where the rounded, unclamped code lies in [qmin, qmax].
template <bool ON>
__device__ __forceinline__ float ste_mask(float x, const Quant& q) {
  if (!ON) return 1.0f;
  float c = fq_code(x, q);
  return (c >= q.qmin && c <= q.qmax) ? 1.0f : 0.0f;
}

struct GateOut {
  float r, z, n, h_raw;
};

// ghr/ghz/ghn already contain the hidden bias.
__device__ __forceinline__ GateOut gru_gates(float gir, float giz, float gin,
                                             float ghr, float ghz, float ghn, float h_prev) {
  GateOut g;
  g.r = sigmoidf_acc(gir + ghr);
  g.z = sigmoidf_acc(giz + ghz);
  g.n = tanhf(gin + g.r * ghn);
  g.h_raw = (1.0f - g.z) * g.n + g.z * h_prev;
  return g;
}

struct GateGrad {
  float dgr, dgz, dgn, dghn, dh_direct;
};

// dh already carries the fq_out mask.
__device__ __forceinline__ GateGrad gru_gate_grads(float dh, float r, float z, float n,
                                                   float ghn, float h_prev) {
  GateGrad g;
  float dn = dh * (1.0f - z);
  float dz = dh * (h_prev - n);
  g.dh_direct = dh * z;
  g.dgn = dn * (1.0f - n * n);
  float dr = g.dgn * ghn;
  g.dghn = g.dgn * r;
  g.dgz = dz * z * (1.0f - z);
  g.dgr = dr * r * (1.0f - r);
  return g;
}

// ---- small host utilities --------------------------------------------------

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
__host__ __device__ inline int cdiv(int a, int b) { return (a + b - 1) / b; }

// Health flag of the diagonal kernels' bounded waits (diag_scan.cu); -1 on CUDA error.
int diag_read_status(int reset);
int bfly_read_status(int reset);     // same for the staged butterfly kernels (butterfly_scan2.cu)
namespace tc {
int tc_read_status(int reset);       // tensor-core GEMM core (tc_gemm.cu)
int tc_step_read_status(int reset);  // fused tensor-core step (tc_step.cu)
}  // namespace tc

// Test hook (b200gru_test_select_kernels): slot 0 != 0 -> butterfly launches use the register /
// global-twiddle kernels on every shape; slot 1 != 0 -> the diagonal forward uses the register-ring
// kernel on every shape.  Defaults 0: the dispatch is by shape only.
int test_kernel_choice(int slot);

// Launch bookkeeping shared by all translation units (defined in api.cu).
void note_launch(int n = 1);
int check_launch(const char* what);
// Once per (device, kernel): raise the kernel's dynamic shared-memory limit to the device's opt-in
// maximum (less the kernel's static shared memory).  Returns 0, or B200GRU_UNSUPPORTED when `bytes`
// exceeds that (or the call failed).
int allow_dynamic_smem(const void* kernel, size_t bytes);

// Deterministic reduction of `nparts` partial vectors of length n, `row_stride` floats apart:
// dst[i] = src[0*row_stride + i] + src[1*row_stride + i] + ... (fixed order).
void launch_reduce_partials(const float* src, int nparts, size_t row_stride, size_t n, float* dst,
                            cudaStream_t st);

// ---- programmatic dependent launch ---------------------------------------------------------------
// The per-step kernels of a scan form a chain in one stream; each is launched with the
// programmatic-stream-serialization attribute, lets its successor be scheduled as soon as every CTA
// of it has started (launch_dependents) and waits for its predecessor's completion and memory
// flush (wait) only after its own prologue -- barrier initialisation, tensor-memory allocation and
// loads of operands no kernel of the chain writes.  Both instructions do nothing in a kernel that
// was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- host side ---------------------------------------------------------------------------------
#ifndef B200GRU_NO_PDL
#define B200GRU_PDL_ALLOWED 1
#else
#define B200GRU_PDL_ALLOWED 0
#endif
// Launch with the programmatic-stream-serialization attribute (the kernel must call pdl_wait()
// before it touches anything an earlier kernel of the stream produces or still reads).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = B200GRU_PDL_ALLOWED;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}


}  // namespace b200gru
