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
#include <stdint.h>

#include "../../include/b200gru.h"

namespace b200gru {

struct Quant {
  float scale;
  float qmin;
  float qmax;
  int enabled;
};

__host__ inline Quant make_quant(const b200gru_quant* q) {
  Quant r;
  if (q == nullptr || !q->enabled) {
    r.scale = 1.f; r.qmin = 0.f; r.qmax = 0.f; r.enabled = 0;
  } else {
    r.scale = q->scale; r.qmin = (float)q->qmin; r.qmax = (float)q->qmax; r.enabled = 1;
  }
  return r;
}

__device__ __forceinline__ float sigmoidf_acc(float x) {
  return 1.0f / (1.0f + expf(-x));
}

// Unclamped integer code of x (as float): rint(x / s).
__device__ __forceinline__ float fq_code(float x, const Quant& q) {
  return rintf(__fdiv_rn(x, q.scale));
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

// Launch bookkeeping shared by all translation units (defined in api.cu).
void note_launch(int n = 1);
int check_launch(const char* what);

// Deterministic reduction of `nparts` partial vectors of length n, `row_stride` floats apart:
// dst[i] = src[0*row_stride + i] + src[1*row_stride + i] + ... (fixed order).
void launch_reduce_partials(const float* src, int nparts, size_t row_stride, size_t n, float* dst,
                            cudaStream_t st);

}  // namespace b200gru
