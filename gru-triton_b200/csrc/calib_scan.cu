// Calibration scan: the forward recurrence with the hidden-state quantisers in OBSERVING mode.
//
// While a layer is being calibrated (src/gru_qat/gru_layer.py:308-339 of the reference, which
// drops to its Python per-step loop for this), each hidden quantiser is in "min_max" mode
// (src/gru_qat/quantizers.py:95-156): every call fake-quantises its argument with a scale taken
// from that argument's own range, s = max(|min x|, |max x|, 1e-8) / qmax, and folds (min x, max x)
// into running statistics -- the first call sets them, later calls blend with momentum 0.99.
// quant_h_in sees h_{t-1}, quant_h_out sees h_raw_t, once per time step each.  Both ranges are
// reductions over the whole [B, H] tensor, so a step is a short sequence of launches:
//
//   hq      = fq(h_{t-1}; s_in)                     s_in from the range of h_{t-1} (previous launch)
//   z, n    = gates of ONE scan step on hq          (the kind's own kernel, T = 1, no quantiser)
//   h_raw   = (1 - z) n + z h_{t-1}                 + block partial min/max
//   observe : running range of quant_h_out, s_out   (one small kernel, fixed-order reduction)
//   h_t     = fq(h_raw; s_out) -> out[t]            + block partial min/max
//   observe : running range of quant_h_in, s_in     for the next step
//
// Everything stays on the device: the scales live in a small device array, the running ranges in
// the caller's tensors; nothing synchronises with the host.

#include <cstring>

#include "common.cuh"

namespace b200gru {

namespace {

constexpr int CS_THREADS = 256;
constexpr int CS_MAX_BLOCKS = 1024;

struct Range {
  float lo, hi;
};

__device__ __forceinline__ Range block_range(float lo, float hi) {
  __shared__ float slo[CS_THREADS / 32], shi[CS_THREADS / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
  }
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { slo[w] = lo; shi[w] = hi; }
  __syncthreads();
  Range r;
  r.lo = slo[0]; r.hi = shi[0];
#pragma unroll
  for (int i = 1; i < CS_THREADS / 32; ++i) { r.lo = fminf(r.lo, slo[i]); r.hi = fmaxf(r.hi, shi[i]); }
  return r;
}

__device__ __forceinline__ float fq_dyn(float x, float s, float qmin, float qmax) {
  return fminf(fmaxf(rintf(__fdiv_rn(x, s)), qmin), qmax) * s;
}

// partial[2*b], partial[2*b+1] = min, max of x over this block's grid-stride share
__global__ void __launch_bounds__(CS_THREADS)
range_kernel(const float* __restrict__ x, size_t n, float* __restrict__ partial) {
  float lo = INFINITY, hi = -INFINITY;
  for (size_t i = (size_t)blockIdx.x * CS_THREADS + threadIdx.x; i < n; i += (size_t)gridDim.x * CS_THREADS) {
    const float v = x[i];
    lo = fminf(lo, v); hi = fmaxf(hi, v);
  }
  const Range r = block_range(lo, hi);
  if (threadIdx.x == 0) { partial[2 * blockIdx.x] = r.lo; partial[2 * blockIdx.x + 1] = r.hi; }
}

// One observer call: global range from the block partials (fixed order), running statistics
// (first call: the range itself; later: momentum blend), and the dynamic scale of this call.
__global__ void observe_kernel(const float* __restrict__ partial, int nblocks, float* rmin, float* rmax,
                               int initialized, float momentum, float one_minus, float qmax, float* scale_slot) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float lo = partial[0], hi = partial[1];
  for (int b = 1; b < nblocks; ++b) { lo = fminf(lo, partial[2 * b]); hi = fmaxf(hi, partial[2 * b + 1]); }
  if (initialized) {
    *rmin = momentum * *rmin + one_minus * lo;       // two products and a sum, as the eager reference rounds
    *rmax = momentum * *rmax + one_minus * hi;
  } else {
    *rmin = lo; *rmax = hi;
  }
  *scale_slot = __fdiv_rn(fmaxf(fmaxf(fabsf(hi), fabsf(lo)), 1e-8f), qmax);
}

// y = fq(x; *scale)  (+ block partial range of y when partial != NULL)
__global__ void __launch_bounds__(CS_THREADS)
fq_dyn_kernel(const float* __restrict__ x, size_t n, const float* __restrict__ scale, float qmin, float qmax,
              float* __restrict__ y, float* __restrict__ partial) {
  const float s = *scale;
  float lo = INFINITY, hi = -INFINITY;
  for (size_t i = (size_t)blockIdx.x * CS_THREADS + threadIdx.x; i < n; i += (size_t)gridDim.x * CS_THREADS) {
    const float v = fq_dyn(x[i], s, qmin, qmax);
    y[i] = v;
    lo = fminf(lo, v); hi = fmaxf(hi, v);
  }
  if (partial != nullptr) {
    const Range r = block_range(lo, hi);
    if (threadIdx.x == 0) { partial[2 * blockIdx.x] = r.lo; partial[2 * blockIdx.x + 1] = r.hi; }
  }
}

// h_raw = (1 - z) n + z h_prev  + block partial range
__global__ void __launch_bounds__(CS_THREADS)
blend_kernel(const float* __restrict__ z, const float* __restrict__ nn, const float* __restrict__ h_prev, size_t n,
             float* __restrict__ h_raw, float* __restrict__ partial) {
  float lo = INFINITY, hi = -INFINITY;
  for (size_t i = (size_t)blockIdx.x * CS_THREADS + threadIdx.x; i < n; i += (size_t)gridDim.x * CS_THREADS) {
    const float v = (1.0f - z[i]) * nn[i] + z[i] * h_prev[i];
    h_raw[i] = v;
    lo = fminf(lo, v); hi = fmaxf(hi, v);
  }
  const Range r = block_range(lo, hi);
  if (threadIdx.x == 0) { partial[2 * blockIdx.x] = r.lo; partial[2 * blockIdx.x + 1] = r.hi; }
}

// Diagonal hidden weights: the whole observing step is elementwise, gh_g = w_g * hq + b_g.
__global__ void __launch_bounds__(CS_THREADS)
diag_blend_kernel(const float* __restrict__ gi_t, const float* __restrict__ hq, const float* __restrict__ h_prev,
                  const float* __restrict__ Wd, const float* __restrict__ bh, int B, int H,
                  float* __restrict__ h_raw, float* __restrict__ partial) {
  float lo = INFINITY, hi = -INFINITY;
  const size_t n = (size_t)B * H;
  for (size_t i = (size_t)blockIdx.x * CS_THREADS + threadIdx.x; i < n; i += (size_t)gridDim.x * CS_THREADS) {
    const size_t b = i / H;
    const int u = (int)(i - b * H);
    const float* g = gi_t + b * 3 * H + u;
    const float q = hq[i];
    const GateOut go = gru_gates(g[0], g[H], g[2 * H], Wd[u] * q + bh[u], Wd[H + u] * q + bh[H + u],
                                 Wd[2 * H + u] * q + bh[2 * H + u], h_prev[i]);
    h_raw[i] = go.h_raw;
    lo = fminf(lo, go.h_raw); hi = fmaxf(hi, go.h_raw);
  }
  const Range r = block_range(lo, hi);
  if (threadIdx.x == 0) { partial[2 * blockIdx.x] = r.lo; partial[2 * blockIdx.x + 1] = r.hi; }
}

int grid_for(size_t n) {
  const size_t b = (n + CS_THREADS - 1) / CS_THREADS;
  return (int)(b < (size_t)CS_MAX_BLOCKS ? (b ? b : 1) : CS_MAX_BLOCKS);
}

}  // namespace

size_t calib_scan_scratch_bytes(int B, int H) {
  // hq, h_raw, save[4][1][B][H], partials, two scale slots
  return align_up((size_t)6 * B * H * sizeof(float), 256) + align_up((size_t)2 * CS_MAX_BLOCKS * sizeof(float), 256) + 256;
}

}  // namespace b200gru

using namespace b200gru;

extern "C" {

size_t b200gru_calibration_workspace_bytes(const b200gru_shape* shape) {
  if (shape == nullptr || shape->T <= 0 || shape->B <= 0 || shape->H <= 0) return (size_t)-1;
  b200gru_shape one = *shape;
  one.T = 1;
  const size_t inner = b200gru_workspace_bytes(&one, 0);
  if (inner == (size_t)-1) return inner;
  return align_up(inner, 256) + calib_scan_scratch_bytes(shape->B, shape->H);
}

int b200gru_calibration_scan(const b200gru_shape* shape, const float* gi, const float* h0, const float* W,
                             const float* bh, int qmax, double momentum, float* in_min, float* in_max,
                             int in_initialized, float* out_min, float* out_max, int out_initialized, float* out,
                             void* workspace, size_t workspace_bytes, void* stream) {
  if (!shape || !gi || !h0 || !W || !bh || !in_min || !in_max || !out_min || !out_max || !out)
    return B200GRU_INVALID_ARGUMENT;
  if (qmax < 1 || !(momentum >= 0.0 && momentum <= 1.0)) return B200GRU_INVALID_ARGUMENT;
  // the reference blends with Python scalars: momentum and (1 - momentum) are each rounded to fp32
  const float mom = (float)momentum, one_minus = (float)(1.0 - momentum);
  const size_t need = b200gru_calibration_workspace_bytes(shape);
  if (need == (size_t)-1) return B200GRU_INVALID_ARGUMENT;
  if (workspace == nullptr || workspace_bytes < need) return B200GRU_WORKSPACE_TOO_SMALL;
  const int T = shape->T, B = shape->B, H = shape->H;
  b200gru_shape one = *shape;
  one.T = 1;
  const size_t inner = align_up(b200gru_workspace_bytes(&one, 0), 256);
  char* ws = static_cast<char*>(workspace);
  void* inner_ws = inner ? static_cast<void*>(ws) : nullptr;
  ws += inner;
  const size_t n = (size_t)B * H;
  float* hq = reinterpret_cast<float*>(ws);
  float* h_raw = hq + n;
  float* save = h_raw + n;                      // r, z, n, gh_n of one step
  ws += align_up(6 * n * sizeof(float), 256);
  float* partial = reinterpret_cast<float*>(ws);
  ws += align_up((size_t)2 * CS_MAX_BLOCKS * sizeof(float), 256);
  float* scales = reinterpret_cast<float*>(ws);  // [0] = s_in, [1] = s_out
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n);
  const float q = (float)qmax;
  const bool diagonal = shape->kind == B200GRU_DIAGONAL;
  // the diagonal kind has no `save` output; its step is elementwise and has its own kernel

  // quant_h_in's first observation: h0
  range_kernel<<<grid, CS_THREADS, 0, st>>>(h0, n, partial);
  observe_kernel<<<1, 32, 0, st>>>(partial, grid, in_min, in_max, in_initialized, mom, one_minus, q, scales);
  note_launch(2);
  for (int t = 0; t < T; ++t) {
    const float* h_prev = (t == 0) ? h0 : out + (size_t)(t - 1) * n;
    float* out_t = out + (size_t)t * n;
    fq_dyn_kernel<<<grid, CS_THREADS, 0, st>>>(h_prev, n, scales, -q, q, hq, nullptr);
    note_launch();
    // one step of the kind's own kernel on hq, no quantiser: its z and n depend on hq only through
    // the hidden product, which is what the observing step needs
    if (diagonal) {
      diag_blend_kernel<<<grid, CS_THREADS, 0, st>>>(gi + (size_t)t * B * 3 * H, hq, h_prev, W, bh, B, H, h_raw, partial);
    } else {
      const int rc = b200gru_scan_forward(&one, gi + (size_t)t * B * 3 * H, hq, W, bh, nullptr, nullptr, out_t, save,
                                          inner_ws, inner, stream);
      if (rc) return rc;
      blend_kernel<<<grid, CS_THREADS, 0, st>>>(save + n, save + 2 * n, h_prev, n, h_raw, partial);
    }
    observe_kernel<<<1, 32, 0, st>>>(partial, grid, out_min, out_max, (out_initialized || t > 0) ? 1 : 0, mom, one_minus,
                                     q, scales + 1);
    fq_dyn_kernel<<<grid, CS_THREADS, 0, st>>>(h_raw, n, scales + 1, -q, q, out_t, partial);
    note_launch(3);
    if (t + 1 < T) {
      observe_kernel<<<1, 32, 0, st>>>(partial, grid, in_min, in_max, 1, mom, one_minus, q, scales);
      note_launch();
    }
  }
  return check_launch("calibration scan");
}

}  // extern "C"
