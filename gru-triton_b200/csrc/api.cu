// C ABI of the library: argument checks, workspace carving, kernel dispatch.
// Nothing here allocates or synchronises; all work is enqueued on the caller's stream.

#include <atomic>
#include <map>
#include <mutex>
#include <utility>
#include <cstdio>
#include <cstring>

#include "block_scan.cuh"
#include "butterfly_scan.cuh"
#include "tc_scan.cuh"

namespace b200gru {

// diag_scan.cu
size_t diag_bwd_workspace_bytes(int T, int B, int H);
int diag_forward(const float* gi, const float* h0, const float* W, const float* bh, float* out, int T, int B,
                 int H, Quant qi, Quant qo, cudaStream_t st);
int diag_backward(const float* gi, const float* h0, const float* W, const float* bh, const float* out,
                  const float* dout, float* dgi, float* dh0, float* dW, float* dbh, void* workspace, int T,
                  int B, int H, Quant qi, Quant qo, cudaStream_t st);

static std::atomic<unsigned long long> g_launches{0};
static std::atomic<int> g_test_choice[2] = {{0}, {0}};

int test_kernel_choice(int slot) { return (slot >= 0 && slot < 2) ? g_test_choice[slot].load(std::memory_order_relaxed) : 0; }
static thread_local char g_last_error[256] = {0};

void note_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return B200GRU_OK;
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
  return B200GRU_LAUNCH_FAILURE;
}

int allow_dynamic_smem(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> limit;      // opt-in bytes granted, -1 = failed
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  auto key = std::make_pair(dev, kernel);
  auto it = limit.find(key);
  if (it == limit.end()) {
    int optin = 0;
    cudaFuncAttributes fa;
    cudaError_t e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, kernel);
    if (e == cudaSuccess) {
      optin -= (int)fa.sharedSizeBytes;               // the opt-in limit covers static + dynamic
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
    }
    if (e != cudaSuccess) { cudaGetLastError(); optin = -1; }
    it = limit.emplace(key, optin).first;
  }
  return (it->second >= 0 && bytes <= (size_t)it->second) ? B200GRU_OK : B200GRU_UNSUPPORTED;
}

__global__ void reduce_partials_kernel(const float* __restrict__ src, int nparts, size_t row_stride, size_t n,
                                       float* __restrict__ dst) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = src[i];
  for (int p = 1; p < nparts; ++p) s += src[(size_t)p * row_stride + i];
  dst[i] = s;
}

void launch_reduce_partials(const float* src, int nparts, size_t row_stride, size_t n, float* dst,
                            cudaStream_t st) {
  const unsigned grid = (unsigned)((n + 255) / 256);
  launch_pdl(reduce_partials_kernel, dim3(grid), dim3(256), 0, st, src, nparts, row_stride, n, dst);
  note_launch();
}

// ---------------------------------------------------------------------------

struct Dims {
  int kind, T, B, H, nb, Hb, logn, Hpad, nstages;
  long long gate_stride, block_stride;
  size_t w_elems;
};

static bool parse_shape(const b200gru_shape* s, Dims* d) {
  if (s == nullptr) return false;
  if (s->T <= 0 || s->B <= 0 || s->H <= 0) return false;
  if ((long long)s->T * s->B > 0x7fffffffLL / 4) return false;     // flattened row index stays in int
  d->kind = s->kind; d->T = s->T; d->B = s->B; d->H = s->H;
  d->nb = 1; d->Hb = s->H; d->logn = 0; d->Hpad = s->H; d->nstages = 0;
  switch (s->kind) {
    case B200GRU_DENSE:
      d->gate_stride = (long long)s->H * s->H; d->block_stride = 0;
      d->w_elems = (size_t)3 * s->H * s->H;
      return true;
    case B200GRU_DIAGONAL:
      d->gate_stride = s->H; d->block_stride = 0; d->w_elems = (size_t)3 * s->H;
      return true;
    case B200GRU_MONARCH:
      if (s->nblocks <= 0 || s->H % s->nblocks != 0) return false;
      d->nb = s->nblocks; d->Hb = s->H / s->nblocks;
      d->gate_stride = (long long)d->nb * d->Hb * d->Hb; d->block_stride = (long long)d->Hb * d->Hb;
      d->w_elems = (size_t)3 * d->nb * d->Hb * d->Hb;
      return true;
    case B200GRU_BUTTERFLY:
      if (s->nblocks <= 0 || s->log2_hpad <= 0 || s->log2_hpad > 20) return false;
      d->logn = s->log2_hpad; d->Hpad = 1 << s->log2_hpad;
      if (d->Hpad < s->H) return false;
      d->nb = s->nblocks; d->nstages = s->nblocks * s->log2_hpad;
      d->w_elems = (size_t)3 * d->nstages * (d->Hpad / 2) * 4;
      return true;
    default:
      return false;
  }
}

static size_t s_bytes(const Dims& d) { return align_up((size_t)4 * d.T * d.B * d.H * sizeof(float), 256); }

static size_t wt_bytes(const Dims& d) {
  return align_up((size_t)3 * d.nb * d.Hb * transposed_row_bound(d.Hb) * sizeof(float), 256);
}
static size_t tc_max(size_t a, size_t b) { return a > b ? a : b; }
static bool step_path(const Dims& d) { return d.kind == B200GRU_DENSE && tc::tc_dense_path(d.B, d.H); }
// dense problems on the cluster kernels whose weight gradient is one tensor-core product
static bool tc_wgrad_path(const Dims& d) {
  return d.kind == B200GRU_DENSE && !step_path(d) && tc::tc_weight_grads_applies(d.T, d.B, d.H);
}

// backward: 0 forward, 1 backward that recomputes the gates, 2 backward that is given `save`
static size_t workspace_bytes(const Dims& d, int backward) {
  const size_t s_need = (backward == 2) ? 0 : s_bytes(d);
  switch (d.kind) {
    case B200GRU_DENSE:
    case B200GRU_MONARCH:
      if (step_path(d))          // tensor-core path: its own scratch (weights as fp32 values)
        return backward ? s_need + tc_max(tc::tc_dense_bwd_scratch_bytes(d.T, d.B, d.H, false),
                                          tc::tc_dense_bwd_scratch_bytes(d.T, d.B, d.H, true))
                        : tc_max(tc::tc_dense_fwd_scratch_bytes(d.T, d.B, d.H, false),
                                 tc::tc_dense_fwd_scratch_bytes(d.T, d.B, d.H, true));
      if (!backward) return wt_bytes(d);
      if (tc_wgrad_path(d))
        return s_need + align_up(bias_grads_scratch_bytes(d.T, d.B, d.H), 256) +
               tc_max(tc::tc_weight_grads_scratch_bytes(d.T, d.B, d.H, false),
                      tc::tc_weight_grads_scratch_bytes(d.T, d.B, d.H, true));
      return s_need + weight_grads_scratch_bytes(d.T, d.B, d.H, d.nb, d.Hb);
    case B200GRU_DIAGONAL:
      return backward ? diag_bwd_workspace_bytes(d.T, d.B, d.H) : 0;
    case B200GRU_BUTTERFLY: {
      const size_t twp = align_up(d.w_elems * sizeof(float), 256);      // twiddles in pass order
      if (!backward) return twp;
      const size_t w = bfly_wgrad_scratch_bytes(d.T, d.B, d.H, d.Hpad, d.nstages);
      if (w == (size_t)-1) return (size_t)-1;
      return s_need + w + align_up(bias_grads_scratch_bytes(d.T, d.B, d.H), 256) + twp;
    }
  }
  return (size_t)-1;
}

static int fill_bfly(const Dims& d, BflyArgs* a) {
  memset(a, 0, sizeof(*a));
  a->T = d.T; a->B = d.B; a->H = d.H; a->Hpad = d.Hpad; a->logn = d.logn; a->nstages = d.nstages;
  a->h0_rows = d.B;
  a->npasses = build_bfly_passes(d.logn, d.nb, a->passes, BFLY_MAX_PASSES);
  return a->npasses > 0 ? 0 : B200GRU_UNSUPPORTED;
}

}  // namespace b200gru

using namespace b200gru;

extern "C" {

size_t b200gru_workspace_bytes(const b200gru_shape* shape, int backward) {
  Dims d;
  if (!parse_shape(shape, &d)) return (size_t)-1;
  return workspace_bytes(d, backward);
}

size_t b200gru_save_bytes(const b200gru_shape* shape) {
  Dims d;
  if (!parse_shape(shape, &d)) return (size_t)-1;
  if (d.kind == B200GRU_DIAGONAL) return 0;      // recompute is free for the elementwise kind
  return (size_t)4 * d.T * d.B * d.H * sizeof(float);
}

// codes / scales: optional int8 form of a dense W (W then holds codes * scales)
static int scan_forward_impl(const b200gru_shape* shape, const float* gi, const float* h0, const float* W,
                             const signed char* codes, const float* scales,
                             const float* bh, const b200gru_quant* q_in, const b200gru_quant* q_out, float* out,
                             float* save, void* workspace, size_t workspace_bytes_, void* stream) {
  Dims d;
  if (!parse_shape(shape, &d)) return B200GRU_INVALID_ARGUMENT;
  if (!gi || !h0 || !W || !bh || !out) return B200GRU_INVALID_ARGUMENT;
  if (q_in && q_in->enabled && !(q_in->scale > 0.f)) return B200GRU_INVALID_ARGUMENT;
  if (q_out && q_out->enabled && !(q_out->scale > 0.f)) return B200GRU_INVALID_ARGUMENT;
  const size_t need = workspace_bytes(d, 0);
  if (need == (size_t)-1) return B200GRU_UNSUPPORTED;
  if (need > 0 && (workspace == nullptr || workspace_bytes_ < need)) return B200GRU_WORKSPACE_TOO_SMALL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Quant qi = make_quant(q_in), qo = make_quant(q_out);

  switch (d.kind) {
    case B200GRU_DIAGONAL:
      return diag_forward(gi, h0, W, bh, out, d.T, d.B, d.H, qi, qo, st);
    case B200GRU_DENSE:
    case B200GRU_MONARCH: {
      if (step_path(d)) {
        const tc::TcWeights w = {W, codes, scales};
        return tc::launch_tc_dense_forward(gi, h0, w, bh, out, save, workspace, d.T, d.B, d.H, qi, qo, st);
      }
      BlockScanConfig cfg;
      if (!choose_block_config(true, d.B, d.Hb, d.nb, &cfg)) return B200GRU_UNSUPPORTED;
      BlockScanArgs a;
      memset(&a, 0, sizeof(a));
      a.gi = gi; a.h0 = h0; a.W = W; a.bh = bh; a.out = out; a.save = save;
      a.T = d.T; a.B = d.B; a.H = d.H; a.nb = d.nb; a.Hb = d.Hb;
      a.w_gate_stride = d.gate_stride; a.w_block_stride = d.block_stride;
      a.qin = qi; a.qout = qo;
      if (!cfg.w_in_smem) {
        float* Wt = static_cast<float*>(workspace);
        int rc = launch_transpose_weights(W, Wt, d.nb, d.Hb, cfg.Hb4 + 4, d.gate_stride, d.block_stride, st);
        if (rc) return rc;
        a.Wt = Wt;
      }
      return launch_block_scan(true, cfg, a, d.nb, st);
    }
    case B200GRU_BUTTERFLY: {
      BflyArgs a;
      int rc = fill_bfly(d, &a);
      if (rc) return rc;
      a.gi = gi; a.h0 = h0; a.h0_tail = h0; a.tw = W; a.bh = bh; a.out = out; a.save = save;
      a.qin = qi; a.qout = qo;
      float* twp = static_cast<float*>(workspace);
      rc = bfly2_permute_twiddles(a, twp, st);
      if (rc) return rc;
      a.twp = twp;
      return bfly_launch_forward(a, st);
    }
  }
  return B200GRU_INVALID_ARGUMENT;
}

int b200gru_scan_forward(const b200gru_shape* shape, const float* gi, const float* h0, const float* W,
                         const float* bh, const b200gru_quant* q_in, const b200gru_quant* q_out, float* out,
                         float* save, void* workspace, size_t workspace_bytes_, void* stream) {
  return scan_forward_impl(shape, gi, h0, W, nullptr, nullptr, bh, q_in, q_out, out, save, workspace, workspace_bytes_,
                           stream);
}

static int scan_backward_impl(const b200gru_shape* shape, const float* gi, const float* h0, const float* W,
                              const signed char* codes, const float* scales,
                              const float* bh, const float* out, const float* dout, const float* save,
                              const b200gru_quant* q_in, const b200gru_quant* q_out, float* dgi, float* dh0,
                              float* dW, float* dbh, void* workspace, size_t workspace_bytes_, void* stream) {
  Dims d;
  if (!parse_shape(shape, &d)) return B200GRU_INVALID_ARGUMENT;
  if (!gi || !h0 || !W || !bh || !out || !dout || !dgi || !dh0 || !dW || !dbh) return B200GRU_INVALID_ARGUMENT;
  if (q_in && q_in->enabled && !(q_in->scale > 0.f)) return B200GRU_INVALID_ARGUMENT;
  if (q_out && q_out->enabled && !(q_out->scale > 0.f)) return B200GRU_INVALID_ARGUMENT;
  const size_t need = workspace_bytes(d, save != nullptr ? 2 : 1);
  if (need == (size_t)-1) return B200GRU_UNSUPPORTED;
  if (need > 0 && (workspace == nullptr || workspace_bytes_ < need)) return B200GRU_WORKSPACE_TOO_SMALL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Quant qi = make_quant(q_in), qo = make_quant(q_out);
  char* ws = static_cast<char*>(workspace);
  const size_t s_off = (save != nullptr) ? 0 : s_bytes(d);     // the gate buffer leads the workspace when needed

  switch (d.kind) {
    case B200GRU_DIAGONAL:
      return diag_backward(gi, h0, W, bh, out, dout, dgi, dh0, dW, dbh, workspace, d.T, d.B, d.H, qi, qo, st);
    case B200GRU_DENSE:
    case B200GRU_MONARCH: {
      float* S_ws = reinterpret_cast<float*>(ws);
      float* scratch = reinterpret_cast<float*>(ws + s_off);
      BlockGemmArgs g;
      memset(&g, 0, sizeof(g));
      g.gi = gi; g.h0 = h0; g.out = out; g.W = W; g.bh = bh; g.dgi = dgi;
      g.dW = dW; g.dbh = dbh; g.partial = scratch;
      g.T = d.T; g.B = d.B; g.H = d.H; g.nb = d.nb; g.Hb = d.Hb;
      g.w_gate_stride = d.gate_stride; g.w_block_stride = d.block_stride; g.qin = qi;
      g.out_on_qin_grid = (qi.enabled && qo.enabled && qi.scale == qo.scale && qi.qmin == qo.qmin &&
                           qi.qmax == qo.qmax) ? 1 : 0;
      const float* S = save;
      if (S == nullptr) {
        g.S = S_ws;
        int rc = launch_recompute_gates(g, st);
        if (rc) return rc;
        S = S_ws;
      }
      if (step_path(d)) {
        const tc::TcWeights w = {W, codes, scales};
        return tc::launch_tc_dense_backward(h0, w, out, S, dout, dgi, dh0, dW, dbh, ws + s_off, d.T, d.B, d.H, qi, qo,
                                            st);
      }
      BlockScanConfig cfg;
      if (!choose_block_config(false, d.B, d.Hb, d.nb, &cfg)) return B200GRU_UNSUPPORTED;
      BlockScanArgs a;
      memset(&a, 0, sizeof(a));
      a.gi = gi; a.h0 = h0; a.W = W; a.bh = bh; a.out = const_cast<float*>(out); a.S = S; a.dout = dout;
      a.dgi = dgi; a.dh0 = dh0;
      a.T = d.T; a.B = d.B; a.H = d.H; a.nb = d.nb; a.Hb = d.Hb;
      a.w_gate_stride = d.gate_stride; a.w_block_stride = d.block_stride;
      a.qin = qi; a.qout = qo;
      int rc = launch_block_scan(false, cfg, a, d.nb, st);
      if (rc) return rc;
      if (tc_wgrad_path(d)) {
        // off-chain products on the tensor cores: bias sums first (their scratch leads), then dW
        char* sc = ws + s_off;
        rc = launch_bias_grads(dgi, S, reinterpret_cast<float*>(sc), dbh, d.T, d.B, d.H, st);
        if (rc) return rc;
        sc += align_up(bias_grads_scratch_bytes(d.T, d.B, d.H), 256);
        return tc::launch_tc_weight_grads(dgi, S, h0, out, qi, dW, sc, d.T, d.B, d.H, st);
      }
      g.S = const_cast<float*>(S);
      return launch_weight_grads(g, st);
    }
    case B200GRU_BUTTERFLY: {
      float* S_ws = reinterpret_cast<float*>(ws);
      const size_t wg = bfly_wgrad_scratch_bytes(d.T, d.B, d.H, d.Hpad, d.nstages);
      float* part_w = reinterpret_cast<float*>(ws + s_off);
      float* part_b = reinterpret_cast<float*>(ws + s_off + wg);
      float* twp = reinterpret_cast<float*>(ws + s_off + wg + align_up(bias_grads_scratch_bytes(d.T, d.B, d.H), 256));
      BflyArgs a;
      int rc = fill_bfly(d, &a);
      if (rc) return rc;
      a.tw = W; a.bh = bh; a.qin = qi; a.qout = qo;
      rc = bfly2_permute_twiddles(a, twp, st);
      if (rc) return rc;
      a.twp = twp;
      const float* S = save;
      if (S == nullptr) {
        // gate recompute: the forward kernel, teacher-forced over all T*B rows (T = 1)
        BflyArgs p = a;
        p.T = 1; p.B = d.T * d.B; p.h0_rows = d.B;
        p.gi = gi; p.h0 = h0; p.h0_tail = out; p.out = nullptr; p.save = S_ws;
        rc = bfly_launch_forward(p, st);
        if (rc) return rc;
        S = S_ws;
      }
      a.gi = gi; a.h0 = h0; a.S = S; a.dout = dout; a.out_c = out; a.dgi = dgi; a.dh0 = dh0;
      rc = bfly_launch_backward(a, st);
      if (rc) return rc;
      a.dgi_c = dgi;
      rc = bfly_launch_wgrad(a, part_w, dW, st);
      if (rc) return rc;
      return launch_bias_grads(dgi, S, part_b, dbh, d.T, d.B, d.H, st);
    }
  }
  return B200GRU_INVALID_ARGUMENT;
}

int b200gru_scan_backward(const b200gru_shape* shape, const float* gi, const float* h0, const float* W,
                          const float* bh, const float* out, const float* dout, const float* save,
                          const b200gru_quant* q_in, const b200gru_quant* q_out, float* dgi, float* dh0,
                          float* dW, float* dbh, void* workspace, size_t workspace_bytes_, void* stream) {
  return scan_backward_impl(shape, gi, h0, W, nullptr, nullptr, bh, out, dout, save, q_in, q_out, dgi, dh0, dW, dbh,
                            workspace, workspace_bytes_, stream);
}

// ---- per-kind conveniences ---------------------------------------------------

static b200gru_shape mk_shape(int kind, int T, int B, int H, int nblocks, int log2_hpad) {
  b200gru_shape s;
  s.kind = kind; s.T = T; s.B = B; s.H = H; s.nblocks = nblocks; s.log2_hpad = log2_hpad;
  return s;
}

int b200gru_dense_forward(const float* gi, const float* h0, const float* Wh_cat, const float* bh_cat, int T,
                          int B, int H, const b200gru_quant* q_in, const b200gru_quant* q_out, float* out,
                          float* save, void* workspace, size_t workspace_bytes_, void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_DENSE, T, B, H, 1, 0);
  return b200gru_scan_forward(&s, gi, h0, Wh_cat, bh_cat, q_in, q_out, out, save, workspace, workspace_bytes_, stream);
}

int b200gru_dense_backward(const float* gi, const float* h0, const float* Wh_cat, const float* bh_cat,
                           const float* out, const float* dout, const float* save, int T, int B, int H,
                           const b200gru_quant* q_in, const b200gru_quant* q_out, float* dgi, float* dh0,
                           float* dWh, float* dbh, void* workspace, size_t workspace_bytes_, void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_DENSE, T, B, H, 1, 0);
  return b200gru_scan_backward(&s, gi, h0, Wh_cat, bh_cat, out, dout, save, q_in, q_out, dgi, dh0, dWh, dbh,
                               workspace, workspace_bytes_, stream);
}

int b200gru_diagonal_forward(const float* gi, const float* h0, const float* Wh_diag, const float* bh_cat, int T,
                             int B, int H, const b200gru_quant* q_in, const b200gru_quant* q_out, float* out,
                             void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_DIAGONAL, T, B, H, 1, 0);
  return b200gru_scan_forward(&s, gi, h0, Wh_diag, bh_cat, q_in, q_out, out, nullptr, nullptr, 0, stream);
}

int b200gru_diagonal_backward(const float* gi, const float* h0, const float* Wh_diag, const float* bh_cat,
                              const float* out, const float* dout, int T, int B, int H,
                              const b200gru_quant* q_in, const b200gru_quant* q_out, float* dgi, float* dh0,
                              float* dWh_diag, float* dbh, void* workspace, size_t workspace_bytes_,
                              void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_DIAGONAL, T, B, H, 1, 0);
  return b200gru_scan_backward(&s, gi, h0, Wh_diag, bh_cat, out, dout, nullptr, q_in, q_out, dgi, dh0, dWh_diag,
                               dbh, workspace, workspace_bytes_, stream);
}

int b200gru_monarch_forward(const float* gi, const float* h0, const float* Wh_struct, const float* bh_cat, int T,
                            int B, int H, int nblocks, const b200gru_quant* q_in, const b200gru_quant* q_out,
                            float* out, float* save, void* workspace, size_t workspace_bytes_, void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_MONARCH, T, B, H, nblocks, 0);
  return b200gru_scan_forward(&s, gi, h0, Wh_struct, bh_cat, q_in, q_out, out, save, workspace, workspace_bytes_,
                              stream);
}

int b200gru_monarch_backward(const float* gi, const float* h0, const float* Wh_struct, const float* bh_cat,
                             const float* out, const float* dout, const float* save, int T, int B, int H,
                             int nblocks, const b200gru_quant* q_in, const b200gru_quant* q_out, float* dgi,
                             float* dh0, float* dWh_struct, float* dbh, void* workspace, size_t workspace_bytes_,
                             void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_MONARCH, T, B, H, nblocks, 0);
  return b200gru_scan_backward(&s, gi, h0, Wh_struct, bh_cat, out, dout, save, q_in, q_out, dgi, dh0, dWh_struct,
                               dbh, workspace, workspace_bytes_, stream);
}

int b200gru_butterfly_forward(const float* gi, const float* h0, const float* twiddles, const float* bh_cat, int T,
                              int B, int H, int nblocks, int log2_hpad, const b200gru_quant* q_in,
                              const b200gru_quant* q_out, float* out, float* save, void* workspace,
                              size_t workspace_bytes_, void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_BUTTERFLY, T, B, H, nblocks, log2_hpad);
  return b200gru_scan_forward(&s, gi, h0, twiddles, bh_cat, q_in, q_out, out, save, workspace, workspace_bytes_,
                              stream);
}

int b200gru_butterfly_backward(const float* gi, const float* h0, const float* twiddles, const float* bh_cat,
                               const float* out, const float* dout, const float* save, int T, int B, int H,
                               int nblocks, int log2_hpad, const b200gru_quant* q_in, const b200gru_quant* q_out,
                               float* dgi, float* dh0, float* dtwiddles, float* dbh, void* workspace,
                               size_t workspace_bytes_, void* stream) {
  const b200gru_shape s = mk_shape(B200GRU_BUTTERFLY, T, B, H, nblocks, log2_hpad);
  return b200gru_scan_backward(&s, gi, h0, twiddles, bh_cat, out, dout, save, q_in, q_out, dgi, dh0, dtwiddles,
                               dbh, workspace, workspace_bytes_, stream);
}

int b200gru_quantize_rows(const float* W, int rows, int cols, int bits, signed char* codes, float* scales, float* Wq,
                          void* stream) {
  return tc::launch_quantize_rows(W, rows, cols, bits, codes, scales, Wq, static_cast<cudaStream_t>(stream));
}

int b200gru_quantize_rows_backward(const float* W, const float* dWq, int rows, int cols, int bits, float* dW,
                                   void* stream) {
  return tc::launch_quantize_rows_backward(W, dWq, rows, cols, bits, dW, static_cast<cudaStream_t>(stream));
}

size_t b200gru_column_sums_workspace_bytes(size_t rows, int cols) {
  return cols > 0 ? tc::column_sums_scratch_bytes(rows, cols) : 0;
}

int b200gru_column_sums(const float* src, size_t rows, int cols, float* dst, void* workspace, size_t workspace_bytes_,
                        void* stream) {
  if (cols <= 0 || workspace_bytes_ < tc::column_sums_scratch_bytes(rows, cols)) return B200GRU_WORKSPACE_TOO_SMALL;
  return tc::launch_column_sums(src, rows, cols, dst, static_cast<float*>(workspace), static_cast<cudaStream_t>(stream));
}

int b200gru_dense_q8_forward(const float* gi, const float* h0, const float* Wq, const signed char* codes,
                             const float* scales, const float* bh_cat, int T, int B, int H,
                             const b200gru_quant* q_in, const b200gru_quant* q_out, float* out, float* save,
                             void* workspace, size_t workspace_bytes_, void* stream) {
  if (!codes || !scales) return B200GRU_INVALID_ARGUMENT;
  const b200gru_shape s = mk_shape(B200GRU_DENSE, T, B, H, 1, 0);
  return scan_forward_impl(&s, gi, h0, Wq, codes, scales, bh_cat, q_in, q_out, out, save, workspace, workspace_bytes_,
                           stream);
}

int b200gru_dense_q8_backward(const float* gi, const float* h0, const float* Wq, const signed char* codes,
                              const float* scales, const float* bh_cat, const float* out, const float* dout,
                              const float* save, int T, int B, int H, const b200gru_quant* q_in,
                              const b200gru_quant* q_out, float* dgi, float* dh0, float* dWq, float* dbh,
                              void* workspace, size_t workspace_bytes_, void* stream) {
  if (!codes || !scales) return B200GRU_INVALID_ARGUMENT;
  const b200gru_shape s = mk_shape(B200GRU_DENSE, T, B, H, 1, 0);
  return scan_backward_impl(&s, gi, h0, Wq, codes, scales, bh_cat, out, dout, save, q_in, q_out, dgi, dh0, dWq, dbh,
                            workspace, workspace_bytes_, stream);
}

void b200gru_test_select_kernels(int butterfly_register_kernels, int diagonal_register_ring) {
  g_test_choice[0].store(butterfly_register_kernels, std::memory_order_relaxed);
  g_test_choice[1].store(diagonal_register_ring, std::memory_order_relaxed);
}

unsigned long long b200gru_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* b200gru_strerror(int status) {
  switch (status) {
    case B200GRU_OK: return "ok";
    case B200GRU_INVALID_ARGUMENT: return "invalid argument";
    case B200GRU_UNSUPPORTED: return "shape not supported by this build or device";
    case B200GRU_LAUNCH_FAILURE: return "kernel launch failed";
    case B200GRU_WORKSPACE_TOO_SMALL: return "workspace too small";
    case B200GRU_SCRATCH_EXCEEDED:
      return "problem needs more scratch than the library's built-in buffer (B200GRU_NOALLOC_SCRATCH_BYTES)";
    default: return "unknown status";
  }
}

const char* b200gru_last_cuda_error(void) { return g_last_error; }

int b200gru_version(void) { return 100; }

}  // extern "C"
