// Tensor-core GEMM core (tcgen05 + tensor memory + TMA), sm_100a.
//
//   C[M,N] = alpha * row_scale[m] * col_scale[n] * sum_p  A_{pa[p]}[M,K] . B_{pb[p]}[N,K]^T  + bias[n]
//
// A and B are given as up to three "planes" of the same shape.  Planes carry an fp32 operand split
// into bf16 terms (hi + mid + lo, 8 mantissa bits each, so three planes hold an fp32 value exactly)
// or, for operands that lie on an int8 grid, a single exact plane of integer codes; the list of
// plane pairs (pa[p], pb[p]) says which cross products are accumulated.  Accumulation is fp32 in
// tensor memory (bf16 planes) or exact int32 (int8 planes).  Each operand is either K-major
// (rows of K contiguous elements) or MN-major (rows of M / N contiguous elements, one row per k),
// so x.W^T, dgh.W and dgh^T.h all run without a transposed copy.
//
// One CTA computes one 128 x BN tile of C for one slice of K (split_k slices write separate
// partial matrices; the caller reduces them in a fixed order).  Warp 0 loads tiles by TMA into a
// ring of shared-memory stages (a stage = one k-block of every plane), warp 1 issues tcgen05.mma
// for every plane pair of a stage and commits the stage back to the loader, warps 2-5 read the
// accumulator from tensor memory (32 lanes each), scale and store.
//
// Stands in for the reference's tl.dot tiles (src/gru_qat/triton_kernels/scan.py:153-155, 521-616)
// and its F.linear input projection (src/gru_qat/gru_layer.py:251-253).

#include <mutex>
#include <type_traits>
#include <set>
#include <utility>

#include "tc_common.cuh"
#include "tc_gemm.cuh"

namespace b200gru {
namespace tc {

__device__ int g_tc_status;

namespace {

constexpr int BM = 128;
constexpr int STAGE_ROW_BYTES = 128;         // one swizzle row: 64 bf16 or 128 int8 along the contiguous axis
constexpr int MN_BK = 64;                    // k rows per stage of an MN-major bf16 operand
constexpr int EPI_WARPS = 8;
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;

struct GemmParams {
  int M, N;
  int kb_total, kb_per_split;                // k-blocks (of 128 bytes of K, or 64 k rows)
  int a_planes, b_planes, npairs;
  int pa[TC_MAX_PAIRS], pb[TC_MAX_PAIRS];
  int stages;
  int chunk_kb;                              // k-blocks summed in tensor memory before a drain
  int accumulate;
  unsigned ab_format;                        // kind::f16 operand format: 0 = fp16, 1 = bf16
  int staged_store;                          // the result tile leaves through the operand ring, whole rows per warp
  float alpha;
  const float* row_scale;
  const float* col_scale;
  const float* bias;
  float* C;
  long long ldc, split_stride;
};

template <bool I8, bool A_MN, bool B_MN, int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  static_assert(!(I8 && (A_MN || B_MN)), "int8 operands are K-major here");
  constexpr int ES = I8 ? 1 : 2;                        // element size
  constexpr int KE = STAGE_ROW_BYTES / ES;              // K elements per k-block of a K-major operand
  constexpr int BK = (A_MN || B_MN) ? MN_BK : KE;       // K elements per stage
  static_assert(!(A_MN != B_MN) || KE == MN_BK, "mixed majors need equal k-block sizes");
  constexpr int UMMA_K = 32 / ES;                       // K of one tcgen05.mma
  constexpr int A_PLANE_BYTES = BM * BK * ES;           // 16 KB
  constexpr int B_PLANE_BYTES = BN * BK * ES;
  const uint32_t IDESC = umma_idesc(I8, A_MN, B_MN, BM, BN, p.ab_format);
  constexpr int NC = BN / 2;                            // accumulator columns per epilogue thread
  typedef typename std::conditional<I8, int, float>::type AccT;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bar_full[TC_MAX_STAGES], bar_empty[TC_MAX_STAGES];
  __shared__ __align__(8) unsigned long long bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int dead;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(p.kb_total, kb_begin + p.kb_per_split);
  const int nkb = max(0, kb_end - kb_begin);
  const int nchunks = (nkb + p.chunk_kb - 1) / p.chunk_kb;
  const int stage_bytes = p.a_planes * A_PLANE_BYTES + p.b_planes * B_PLANE_BYTES;
  int* status = &g_tc_status;
  pdl_launch_dependents();
#ifdef B200GRU_PHASE_TIMING
  const long long gm_t0 = clock64();
#define GM_MARK(cond, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (cond)) \
    atomicAdd(&g_phase_cycles[slot], (unsigned long long)(clock64() - gm_t0)); } while (0)
#else
#define GM_MARK(cond, slot)
#endif

  if (threadIdx.x == 0) {
    dead = (*reinterpret_cast<volatile int*>(status) != 0) ? 1 : 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), EPI_WARPS);
    }
    mbar_fence_init();
    tma_prefetch_map(&tmA);
    tma_prefetch_map(&tmB);
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), 2 * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_base_slot;
  volatile int* deadp = &dead;
  pdl_wait();          // the operands (and, when accumulating, C) may come from the previous kernel of the stream
  GM_MARK(threadIdx.x == 0, 0);      // prologue done

  if (warp == 0) {
    if (lane == 0 && !*deadp) {
      // ---- loader: one k-block of every plane per stage
      for (int i = 0; i < nkb; ++i) {
        const int s = i % p.stages, round = i / p.stages;
        if (round > 0 && !mbar_wait(smem_u32(&bar_empty[s]), (round - 1) & 1, deadp, status)) break;
        const uint32_t full = smem_u32(&bar_full[s]);
        mbar_expect_tx(full, (uint32_t)stage_bytes);
        unsigned char* st = smem + (size_t)s * stage_bytes;
        const int kb = kb_begin + i;
        for (int pl = 0; pl < p.a_planes; ++pl) {
          const uint32_t dst = smem_u32(st + pl * A_PLANE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(dst + c * (MN_BK * 128), &tmA, m0 + c * 64, kb * MN_BK, pl, full);
          } else {
            tma_load_3d(dst, &tmA, kb * KE, m0, pl, full);
          }
        }
        unsigned char* sb = st + p.a_planes * A_PLANE_BYTES;
        for (int pl = 0; pl < p.b_planes; ++pl) {
          const uint32_t dst = smem_u32(sb + pl * B_PLANE_BYTES);
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(dst + c * (MN_BK * 128), &tmB, n0 + c * 64, kb * MN_BK, pl, full);
          } else {
            tma_load_3d(dst, &tmB, kb * KE, n0, pl, full);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && !*deadp) {
      // ---- issuer.  The fp32 accumulator of the tensor core truncates, so its error grows with
      // the number of accumulation steps; a chunk of chunk_kb k-blocks is summed in tensor
      // memory from zero, then handed to the epilogue warps, which keep the running total in
      // registers with round-to-nearest adds.  Two accumulator buffers alternate.
      bool alive = true;
      for (int c = 0; c < nchunks && alive; ++c) {
        const int buf = c & 1;
        if (c >= 2 && !mbar_wait(smem_u32(&bar_acc_empty[buf]), ((c >> 1) - 1) & 1, deadp, status)) break;
        tc_fence_after();
        const uint32_t tacc = tmem_acc + (uint32_t)(buf * BN);
        const int i_end = min(nkb, (c + 1) * p.chunk_kb);
        for (int i = c * p.chunk_kb; i < i_end; ++i) {
          const int s = i % p.stages, round = i / p.stages;
          if (!mbar_wait(smem_u32(&bar_full[s]), round & 1, deadp, status)) { alive = false; break; }
          tc_fence_after();
          GM_MARK(i == 0, 1);          // first stage landed
          GM_MARK(i == nkb - 1, 2);    // last stage landed
          const uint32_t sa = smem_u32(smem + (size_t)s * stage_bytes);
          const uint32_t sb = sa + p.a_planes * A_PLANE_BYTES;
          for (int q = 0; q < p.npairs; ++q) {
            const uint32_t pa = sa + p.pa[q] * A_PLANE_BYTES, pb = sb + p.pb[q] * B_PLANE_BYTES;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              const uint64_t da = A_MN ? umma_smem_desc(pa + kk * UMMA_K * 128, MN_BK * 128, 1024)
                                       : umma_smem_desc(pa + kk * 32, 16, 1024);
              const uint64_t db = B_MN ? umma_smem_desc(pb + kk * UMMA_K * 128, MN_BK * 128, 1024)
                                       : umma_smem_desc(pb + kk * 32, 16, 1024);
              umma<I8>(tacc, da, db, IDESC, (i > c * p.chunk_kb || q > 0 || kk > 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&bar_empty[s]));          // the stage is free once these MMAs have read it
        }
        if (alive) umma_commit(smem_u32(&bar_acc_full[buf]));   // this chunk's sum is complete
      }
    }
  } else {
    // ---- epilogue: warp w reads tensor-memory lanes [32 * (w % 4), +32); the two warps of a lane
    // quarter take one half of the tile's columns each; thread = one row x NC columns
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int m = m0 + q * 32 + lane;
    const int cbase = half * NC;
    AccT acc[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) acc[j] = (AccT)0;
    bool ok = true;
    for (int c = 0; c < nchunks; ++c) {
      const int buf = c & 1;
      if (ok) ok = mbar_wait(smem_u32(&bar_acc_full[buf]), (c >> 1) & 1, deadp, status);
      ok = __all_sync(0xffffffffu, ok);                  // tcgen05.ld below is warp-collective
      if (!ok) break;
      tc_fence_after();
      const uint32_t tsrc = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + cbase);
#pragma unroll
      for (int c0 = 0; c0 < NC; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tsrc + (uint32_t)c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (I8) acc[c0 + j] += (AccT)(int)v[j];
          else acc[c0 + j] += (AccT)__uint_as_float(v[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
    }
    GM_MARK(threadIdx.x == 64, 3);    // all chunks drained
    if (p.staged_store) {
      // Coalesced stores.  A thread holds one row of the tile, so its own stores would scatter 16
      // bytes into each of 32 rows per instruction (a quarter of a cache line each: the LSU queues
      // them for longer than the whole main loop of a short product).  The operand ring is free
      // once the last chunk has been committed: the tile goes through it, row-major with a
      // 4-float pad, and every warp then writes whole rows, 512 contiguous bytes per instruction.
      constexpr int LDS = BN + 4;
      float* tile = reinterpret_cast<float*>(smem);
      const int r = q * 32 + lane;
      if (ok) {
#pragma unroll
        for (int j = 0; j < NC; j += 4)
          *reinterpret_cast<float4*>(tile + r * LDS + cbase + j) =
              make_float4((float)acc[j], (float)acc[j + 1], (float)acc[j + 2], (float)acc[j + 3]);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
      const int ew = warp - 2;                                   // 0..7
      constexpr int NH = BN >= 128 ? BN / 128 : 1;               // 128-column spans of the tile
      float cs[NH][4], bs[NH][4];
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        const int n = n0 + h * 128 + lane * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          cs[h][e] = (p.col_scale != nullptr && n + e < p.N) ? __ldg(p.col_scale + n + e) : 1.0f;
          bs[h][e] = (p.bias != nullptr && n + e < p.N) ? __ldg(p.bias + n + e) : 0.0f;
        }
      }
      if (ok) {
        constexpr int RPW = BM / EPI_WARPS;                        // rows per warp
        float rsv[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) {                            // all row scales in flight at once
          const int mm = m0 + ew + i * EPI_WARPS;
          rsv[i] = p.alpha * ((p.row_scale != nullptr && mm < p.M) ? __ldg(p.row_scale + mm) : 1.0f);
        }
#pragma unroll 4
        for (int i = 0; i < RPW; ++i) {
          const int rr = ew + i * EPI_WARPS;
          const int mm = m0 + rr;
          if (mm < p.M) {
            const float rs = rsv[i];
            float* crow = p.C + (size_t)blockIdx.z * p.split_stride + (size_t)mm * p.ldc;
#pragma unroll
            for (int h = 0; h < NH; ++h) {
              const int c = h * 128 + lane * 4;
              const int n = n0 + c;
              if (c < BN && n < p.N) {
                const float4 v = *reinterpret_cast<const float4*>(tile + rr * LDS + c);
                float o[4] = {v.x * rs, v.y * rs, v.z * rs, v.w * rs};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  if (p.col_scale != nullptr) o[e] = o[e] * cs[h][e];
                  if (p.bias != nullptr) o[e] = o[e] + bs[h][e];
                }
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(crow + n);
                  o[0] += old.x; o[1] += old.y; o[2] += old.z; o[3] += old.w;
                }
                *reinterpret_cast<float4*>(crow + n) = make_float4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
      }
    } else if (m < p.M) {
      const float rs = p.alpha * (p.row_scale != nullptr ? p.row_scale[m] : 1.0f);
      float* crow = p.C + (size_t)blockIdx.z * p.split_stride + (size_t)m * p.ldc;
#pragma unroll
      for (int j = 0; j < NC; j += 4) {
        const int n = n0 + cbase + j;
        if (n < p.N) {                                    // N % 4 == 0: whole float4 in range
          float o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float r = (float)acc[j + e] * rs;
            if (p.col_scale != nullptr) r = r * __ldg(p.col_scale + n + e);
            if (p.bias != nullptr) r = r + __ldg(p.bias + n + e);
            o[e] = r;
          }
          if (p.accumulate) {
            const float4 old = *reinterpret_cast<const float4*>(crow + n);
            o[0] += old.x; o[1] += old.y; o[2] += old.z; o[3] += old.w;
          }
          *reinterpret_cast<float4*>(crow + n) = make_float4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }

  // ---- teardown: a CTA that gave up may still have tile copies in flight; let them land
  if (warp == 0 && lane == 0 && *deadp) {
    const long long start = clock64();
    while (clock64() - start < (1ll << 18)) {
    }
  }
  GM_MARK(threadIdx.x == 64, 4);      // stores issued
  tc_fence_before();
  __syncthreads();
  GM_MARK(threadIdx.x == 0, 5);       // all warps done
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_acc, 2 * BN);
  }
}

// ---- fp32 -> bf16 planes ------------------------------------------------------------------------
// dst[pl][i] = pl-th bf16 term of src[i] * scale[i % ncols] (scale optional): hi = RN(x),
// mid = RN(x - hi), lo = RN(x - hi - mid); the residuals are exact in fp32.
__global__ void __launch_bounds__(256)
split_planes_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n4, size_t plane_stride,
                    int planes, const float* __restrict__ col_scale, int ncols) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 v = __ldcs(reinterpret_cast<const float4*>(src) + i);
  float x[4] = {v.x, v.y, v.z, v.w};
  if (col_scale != nullptr) {
    const int c = (int)((i * 4) % (size_t)ncols);
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = x[e] * col_scale[c + e];
  }
  for (int pl = 0; pl < planes; ++pl) {
    __nv_bfloat16 h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      h[e] = __float2bfloat16_rn(x[e]);
      x[e] = x[e] - __bfloat162float(h[e]);
    }
    uint2 o;
    o.x = (uint32_t)__bfloat16_as_ushort(h[0]) | ((uint32_t)__bfloat16_as_ushort(h[1]) << 16);
    o.y = (uint32_t)__bfloat16_as_ushort(h[2]) | ((uint32_t)__bfloat16_as_ushort(h[3]) << 16);
    *reinterpret_cast<uint2*>(dst + (size_t)pl * plane_stride + i * 4) = o;
  }
}

// Two fp16 planes of every row of src[rows][cols], scaled by a power of two of the row's own:
// s_r = 2^(15 - e) with max|row| = m * 2^e, m in [0.5, 1), so the largest scaled element lies in
// [2^14, 2^15).  hi = RN16(x * s), lo = RN16(x * s - hi) (the difference is exact in fp32), and
// inv_scale[r] = 1 / s_r exactly.  hi + lo carries 22 significant bits of every element that is
// not below 2^-17 of its row's largest; smaller ones keep an absolute error of 2^-40 of it.
// One warp per row; the second read of the row hits L1.
__global__ void __launch_bounds__(256)
split_rows_f16_kernel(const float* __restrict__ src, __half* __restrict__ dst, int rows, int cols, size_t plane_stride,
                      float* __restrict__ inv_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float4* s4 = reinterpret_cast<const float4*>(src + (size_t)row * cols);
  const int c4 = cols >> 2;
  float mx = 0.f;
  for (int i = lane; i < c4; i += 32) {
    const float4 v = s4[i];
    mx = fmaxf(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))), mx);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  int e = 0;
  float s = 1.0f, inv = 1.0f;
  if (mx > 0.f && mx < 3.0e38f) {
    frexpf(mx, &e);
    e = max(-110, min(110, e));               // both 2^(15-e) and 2^(e-15) stay normal
    s = ldexpf(1.0f, 15 - e);
    inv = ldexpf(1.0f, e - 15);
  }
  if (lane == 0) inv_scale[row] = inv;
  __half* d = dst + (size_t)row * cols;
  for (int i = lane; i < c4; i += 32) {
    const float4 v = s4[i];
    const float x[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
    __half hi[4], lo[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      hi[k] = __float2half_rn(x[k]);
      lo[k] = __float2half_rn(x[k] - __half2float(hi[k]));
    }
    uint2 a, b;
    a.x = (uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[1]) << 16);
    a.y = (uint32_t)__half_as_ushort(hi[2]) | ((uint32_t)__half_as_ushort(hi[3]) << 16);
    b.x = (uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[1]) << 16);
    b.y = (uint32_t)__half_as_ushort(lo[2]) | ((uint32_t)__half_as_ushort(lo[3]) << 16);
    *reinterpret_cast<uint2*>(d + i * 4) = a;
    *reinterpret_cast<uint2*>(d + plane_stride + i * 4) = b;
  }
}

// Test probe of the bounded waits: one CTA arms an mbarrier for bytes that nothing ever sends and
// waits on it with a budget of about a millisecond; the wait gives up, sets the health word and
// the kernel returns normally.
__global__ void wait_timeout_probe_kernel(long long budget_cycles) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x != 0) return;
  mbar_init(smem_u32(&bar), 1);
  mbar_fence_init();
  mbar_expect_tx(smem_u32(&bar), 16);
  const long long start = clock64();
  bool ok = false;
  while (clock64() - start < budget_cycles) {
    if (mbar_try_wait(smem_u32(&bar), 0)) { ok = true; break; }
  }
  if (!ok) atomicExch(&g_tc_status, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encoder() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Opt in to the large dynamic shared memory once per (device, kernel).
int prepare(const void* kernel) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return B200GRU_LAUNCH_FAILURE;
  std::lock_guard<std::mutex> lk(mu);
  const auto key = std::make_pair(dev, kernel);
  if (done.count(key) == 0) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BUDGET + 1024) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(tc_gemm_kernel)");
    done.insert(key);
  }
  return B200GRU_OK;
}

template <bool I8, bool A_MN, bool B_MN, int BN>
int launch_variant(const TcGemm& g, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, dim3 grid,
                   int smem, cudaStream_t st) {
  auto kernel = tc_gemm_kernel<I8, A_MN, B_MN, BN>;
  int rc = prepare(reinterpret_cast<const void*>(kernel));
  if (rc) return rc;
  launch_pdl(kernel, grid, dim3(GEMM_THREADS), (size_t)smem, st, ta, tb, p);
  note_launch();
  return check_launch("tc_gemm_kernel");
}

template <bool I8, bool A_MN, bool B_MN>
int launch_bn(const TcGemm& g, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, dim3 grid, int smem,
              int bn, cudaStream_t st) {
  switch (bn) {
    case 64: return launch_variant<I8, A_MN, B_MN, 64>(g, ta, tb, p, grid, smem, st);
    case 128: return launch_variant<I8, A_MN, B_MN, 128>(g, ta, tb, p, grid, smem, st);
    case 256: return launch_variant<I8, A_MN, B_MN, 256>(g, ta, tb, p, grid, smem, st);
  }
  return B200GRU_INVALID_ARGUMENT;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int make_tensor_map_3d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, unsigned long long d0,
                       unsigned long long d1, unsigned long long d2, unsigned long long stride1_bytes,
                       unsigned long long stride2_bytes, unsigned box0, unsigned box1) {
  EncodeTiledFn fn = encoder();
  if (fn == nullptr) return B200GRU_UNSUPPORTED;
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, dtype, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200GRU_OK : B200GRU_INVALID_ARGUMENT;
}

int launch_wait_timeout_probe(cudaStream_t st) {
  wait_timeout_probe_kernel<<<1, 32, 0, st>>>(1ll << 21);
  note_launch();
  return check_launch("wait_timeout_probe_kernel");
}

int tc_read_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int));
  }
  return v;
}

int tc_gemm_tile_n(const TcGemm& g) {
  if (g.tile_n == 64 || g.tile_n == 128 || g.tile_n == 256) return g.tile_n;
  // Fewest waves over the 148 SMs, weighted by a tile's cost (a fixed part for the A operand and
  // the pipeline fill plus a part proportional to the tile width); the ring needs two stages.
  const int splits = g.split_k < 1 ? 1 : g.split_k;
  int best = 0;
  long long best_cost = 0;
  for (int bn = 256; bn >= 64; bn >>= 1) {
    const int stage = g.a_planes * 16384 + g.b_planes * bn * 128;
    if (2 * stage > TC_SMEM_BUDGET) continue;
    const long long tiles = (long long)cdiv(g.M, BM) * cdiv(g.N, bn) * splits;
    const long long cost = ((tiles + 147) / 148) * (128 + bn);
    if (best == 0 || cost < best_cost) { best = bn; best_cost = cost; }
  }
  return best;
}

int launch_tc_gemm(const TcGemm& g, cudaStream_t st) {
  const bool i8 = g.kind == TC_KIND_I8;
  const int es = i8 ? 1 : 2;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.A == nullptr || g.B == nullptr || g.C == nullptr) return B200GRU_INVALID_ARGUMENT;
  if (g.a_planes < 1 || g.a_planes > 3 || g.b_planes < 1 || g.b_planes > 3) return B200GRU_INVALID_ARGUMENT;
  if (g.npairs < 1 || g.npairs > TC_MAX_PAIRS) return B200GRU_INVALID_ARGUMENT;
  for (int q = 0; q < g.npairs; ++q)
    if (g.pa[q] < 0 || g.pa[q] >= g.a_planes || g.pb[q] < 0 || g.pb[q] >= g.b_planes) return B200GRU_INVALID_ARGUMENT;
  if (i8 && (g.a_mn || g.b_mn)) return B200GRU_UNSUPPORTED;
  if ((g.N & 3) || (g.ldc & 3) || !aligned16(g.C) || !aligned16(g.A) || !aligned16(g.B)) return B200GRU_INVALID_ARGUMENT;
  if (((g.lda * es) & 15) || ((g.ldb * es) & 15) || ((g.a_plane_stride * es) & 15) || ((g.b_plane_stride * es) & 15))
    return B200GRU_INVALID_ARGUMENT;
  const int bn = tc_gemm_tile_n(g);
  if (bn == 0) return B200GRU_UNSUPPORTED;
  const int ke = 128 / es;
  const int bk = tc_gemm_kblock(g);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = g.M; p.N = g.N;
  p.kb_total = cdiv(g.K, bk);
  const int split = g.split_k < 1 ? 1 : g.split_k;
  p.kb_per_split = cdiv(p.kb_total, split);
  const int nsplit = cdiv(p.kb_total, p.kb_per_split);
  if (nsplit != split) return B200GRU_INVALID_ARGUMENT;       // the caller sizes C by tc_gemm_splits()
  p.a_planes = g.a_planes; p.b_planes = g.b_planes; p.npairs = g.npairs;
  for (int q = 0; q < g.npairs; ++q) { p.pa[q] = g.pa[q]; p.pb[q] = g.pb[q]; }
  const int stage = g.a_planes * BM * 128 + g.b_planes * bn * 128;
  p.stages = TC_SMEM_BUDGET / stage;
  if (p.stages > TC_MAX_STAGES) p.stages = TC_MAX_STAGES;
  if (p.stages < 2) return B200GRU_UNSUPPORTED;
  if (g.chunk_kb > 0) p.chunk_kb = g.chunk_kb;
  else if (i8) p.chunk_kb = p.kb_per_split;                   // int32 accumulation is exact
  else p.chunk_kb = (32 / (4 * g.npairs)) > 0 ? 32 / (4 * g.npairs) : 1;   // at most 32 accumulation steps per chunk
  p.accumulate = g.accumulate;
  p.ab_format = (g.kind == TC_KIND_F16) ? 0u : 1u;
  p.staged_store = ((size_t)p.stages * stage >= (size_t)BM * (bn + 4) * sizeof(float)) ? 1 : 0;
  p.alpha = g.alpha; p.row_scale = g.row_scale; p.col_scale = g.col_scale; p.bias = g.bias;
  p.C = g.C; p.ldc = g.ldc; p.split_stride = g.split_stride;

  const CUtensorMapDataType dt = i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                    : (g.kind == TC_KIND_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                             : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  alignas(64) CUtensorMap ta, tb;
  int rc;
  // K-major: dims {K, rows, planes}, box {128 bytes of K, tile rows}.  MN-major: dims {rows(M|N), K, planes},
  // box {64 elements, 64 k rows}.
  const unsigned long long a_pl = g.a_planes > 1 ? (unsigned long long)g.a_plane_stride * es
                                                 : (unsigned long long)(g.a_mn ? g.K : g.M) * g.lda * es;
  const unsigned long long b_pl = g.b_planes > 1 ? (unsigned long long)g.b_plane_stride * es
                                                 : (unsigned long long)(g.b_mn ? g.K : g.N) * g.ldb * es;
  if (g.a_mn) rc = make_tensor_map_3d(&ta, dt, g.A, g.M, g.K, g.a_planes, (unsigned long long)g.lda * es, a_pl, 64, MN_BK);
  else rc = make_tensor_map_3d(&ta, dt, g.A, g.K, g.M, g.a_planes, (unsigned long long)g.lda * es, a_pl, ke, BM);
  if (rc) return rc;
  if (g.b_mn) rc = make_tensor_map_3d(&tb, dt, g.B, g.N, g.K, g.b_planes, (unsigned long long)g.ldb * es, b_pl, 64, MN_BK);
  else rc = make_tensor_map_3d(&tb, dt, g.B, g.K, g.N, g.b_planes, (unsigned long long)g.ldb * es, b_pl, ke, bn);
  if (rc) return rc;

  const dim3 grid(cdiv(g.N, bn), cdiv(g.M, BM), split);
  if (grid.y > 65535u || grid.z > 65535u) return B200GRU_UNSUPPORTED;
  const int smem = p.stages * stage + 1024;
  if (i8) return launch_bn<true, false, false>(g, ta, tb, p, grid, smem, bn, st);
  if (!g.a_mn && !g.b_mn) return launch_bn<false, false, false>(g, ta, tb, p, grid, smem, bn, st);
  if (!g.a_mn && g.b_mn) return launch_bn<false, false, true>(g, ta, tb, p, grid, smem, bn, st);
  if (g.a_mn && !g.b_mn) return launch_bn<false, true, false>(g, ta, tb, p, grid, smem, bn, st);
  return launch_bn<false, true, true>(g, ta, tb, p, grid, smem, bn, st);
}

int tc_gemm_kblock(const TcGemm& g) { return (g.kind == TC_KIND_I8) ? 128 : 64; }

int tc_gemm_splits(const TcGemm& g, int want) {
  const int kb = cdiv(g.K, tc_gemm_kblock(g));
  if (want < 1) want = 1;
  if (want > kb) want = kb;
  const int per = cdiv(kb, want);
  return cdiv(kb, per);
}

int launch_split_planes(const float* src, void* dst, size_t n, size_t plane_stride, int planes,
                        const float* col_scale, int ncols, cudaStream_t st) {
  if (src == nullptr || dst == nullptr || (n & 3) || planes < 1 || planes > 3) return B200GRU_INVALID_ARGUMENT;
  if (col_scale != nullptr && (ncols <= 0 || (ncols & 3))) return B200GRU_INVALID_ARGUMENT;
  if (!aligned16(src) || (reinterpret_cast<uintptr_t>(dst) & 7u) || (plane_stride & 3)) return B200GRU_INVALID_ARGUMENT;
  const size_t n4 = n / 4;
  if (n4 == 0) return B200GRU_OK;
  launch_pdl(split_planes_kernel, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, st, src,
             static_cast<__nv_bfloat16*>(dst), n4, plane_stride, planes, col_scale, ncols);
  note_launch();
  return check_launch("split_planes_kernel");
}

int launch_split_rows_f16(const float* src, void* dst, int rows, int cols, size_t plane_stride, float* inv_scale,
                          cudaStream_t st) {
  if (src == nullptr || dst == nullptr || inv_scale == nullptr || rows < 0 || cols <= 0 || (cols & 3) ||
      (plane_stride & 3))
    return B200GRU_INVALID_ARGUMENT;
  if (!aligned16(src) || (reinterpret_cast<uintptr_t>(dst) & 7u)) return B200GRU_INVALID_ARGUMENT;
  if (rows == 0) return B200GRU_OK;
  launch_pdl(split_rows_f16_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, st, src, static_cast<__half*>(dst),
             rows, cols, plane_stride, inv_scale);
  note_launch();
  return check_launch("split_rows_f16_kernel");
}

}  // namespace tc
}  // namespace b200gru

B200GRU_DEFINE_PHASE_READER(b200gru_debug_phase_cycles_gemm)
