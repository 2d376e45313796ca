// Fused forward step of the dense QAT scan on the tensor cores (sm_100a).
//
// When weights and hidden state are both int8 codes, one kernel does a whole time step:
//
//   acc[b, (g,u)] = sum_k codes_h[b,k] * codes_W[(g,u),k]        tcgen05.mma kind::i8, int32, exact
//   gh = acc * (s_h * s_row[(g,u)]) + bh ;  r, z, n gates ;  h_t = fq_out((1-z) n + z h_{t-1})
//   out[t], save[r,z,n,gh_n], and the int8 codes of fq_in(h_t) for the next step
//
// CTA tile = 128 batch rows x 32 hidden units x 3 gates: the B operand of the MMA is the three
// 32-row slabs W[g*H + u0 .. +32, :] stacked to N = 96, so that the r, z and n pre-activations of
// one (row, unit) sit in the same tensor-memory lane and the gate math needs no exchange between
// threads.  Warp 0 loads k-blocks by TMA (the weight slabs of the first stages before the
// programmatic-dependency wait: they do not depend on the previous step), warp 1 issues the
// MMAs, warps 2-9 prefetch gi[t] and h_{t-1} for their (row, 16 units), then read the accumulator
// and run the gate epilogue.  One launch per step; the stream order is the recurrence.
//
// Reference: the per-step body of gru_scan_fwd_persistent_kernel
// (src/gru_qat/triton_kernels/scan.py:120-184), with tl.dot replaced by an exact integer product.

#include <cstring>
#include <mutex>
#include <set>
#include <utility>

#include "tc_common.cuh"
#include "tc_step.cuh"

namespace b200gru {
namespace tc {

__device__ int g_tc_step_status;

namespace {

constexpr int FS_BM = 128;          // batch rows per CTA
constexpr int FS_UNITS = 32;        // hidden units per CTA
constexpr int FS_BN = 3 * FS_UNITS; // MMA N
constexpr int FS_KB = 128;          // int8 elements of K per stage
constexpr int FS_A_BYTES = FS_BM * FS_KB;            // 16 KB
constexpr int FS_B_SLAB = FS_UNITS * FS_KB;          // 4 KB per gate
constexpr int FS_STAGE = FS_A_BYTES + 3 * FS_B_SLAB; // 28 KB
constexpr int FS_STAGES = 4;                         // ring; also holds the five 16 KB output tiles afterwards
constexpr int FS_TILE = FS_BM * FS_UNITS * 4;        // one fp32 [128 rows][32 units] tile: 16 KB
constexpr int FS_SMEM = FS_STAGES * FS_STAGE + 4 * FS_TILE + 1024;   // ring + gi(3) + h_prev(1) + alignment
constexpr int FS_EPI_WARPS = 8;
constexpr int FS_THREADS = 64 + 32 * FS_EPI_WARPS;
static_assert(FS_STAGES * FS_STAGE >= 5 * FS_TILE, "output staging reuses the operand ring");

struct FusedFwdArgs {
  const float* col_scale;  // [3H] row scales of the weight codes
  const float* bh;       // [3H]
  signed char* codes_next;   // [B][H] or NULL
  int t, T, B, H;
  int nkb;
  int has_save;
  float alpha;           // scale of the hidden codes
  Quant qin, qout;
};

// fp32 tile [128 rows][32 floats] written by TMA with the 128-byte swizzle: 16-byte chunk c of row r
// sits at chunk position c ^ (r & 7).  A thread that owns row r touches chunks without bank conflicts.
__device__ __forceinline__ float4* tile_chunk(unsigned char* tile, int r, int c) {
  return reinterpret_cast<float4*>(tile + r * 128 + ((c ^ (r & 7)) << 4));
}

__global__ void __launch_bounds__(FS_THREADS, 1)
tc_fwd_step_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmGi, const __grid_constant__ CUtensorMap tmPrev,
                   const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmSave,
                   const FusedFwdArgs a) {
  constexpr uint32_t IDESC = umma_idesc(true, false, false, FS_BM, FS_BN);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* io = smem + FS_STAGES * FS_STAGE;        // gi_r, gi_z, gi_n, h_prev tiles
  __shared__ __align__(8) unsigned long long bar_full[FS_STAGES], bar_empty[FS_STAGES], bar_acc, bar_io;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int dead;
  __shared__ float s_scale[FS_BN], s_bias[FS_BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int u0 = blockIdx.x * FS_UNITS, m0 = blockIdx.y * FS_BM;
  const int H = a.H;
  int* status = &g_tc_step_status;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    dead = (*reinterpret_cast<volatile int*>(status) != 0) ? 1 : 0;
    for (int s = 0; s < FS_STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_acc), 1);
    mbar_init(smem_u32(&bar_io), 1);
    mbar_fence_init();
    tma_prefetch_map(&tmA);
    tma_prefetch_map(&tmB);
    tma_prefetch_map(&tmGi);
    tma_prefetch_map(&tmPrev);
  }
  if (threadIdx.x >= 64 && threadIdx.x < 64 + FS_BN) {
    const int c = threadIdx.x - 64, g = c / FS_UNITS, j = c - g * FS_UNITS;
    s_scale[c] = a.alpha * a.col_scale[g * H + u0 + j];
    s_bias[c] = a.bh[g * H + u0 + j];
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_base_slot;
  volatile int* deadp = &dead;

  if (warp == 0) {
    if (lane == 0 && !*deadp) {
      // Nothing the previous step's kernel writes: gi[t] and the weight slabs of the first ring
      // round go in flight before the wait for that kernel.
      const uint32_t iob = smem_u32(&bar_io);
      mbar_expect_tx(iob, 4 * FS_TILE);
#pragma unroll
      for (int g = 0; g < 3; ++g) tma_load_3d(smem_u32(io + g * FS_TILE), &tmGi, g * H + u0, m0, a.t, iob);
      const int first = a.nkb < FS_STAGES ? a.nkb : FS_STAGES;
      for (int i = 0; i < first; ++i) {
        const uint32_t full = smem_u32(&bar_full[i]);
        mbar_expect_tx(full, FS_STAGE);
        unsigned char* st = smem + (size_t)i * FS_STAGE;
#pragma unroll
        for (int g = 0; g < 3; ++g)
          tma_load_3d(smem_u32(st + FS_A_BYTES + g * FS_B_SLAB), &tmB, i * FS_KB, g * H + u0, 0, full);
      }
      pdl_wait();
      // h_{t-1} and its integer codes come from the previous step
      tma_load_3d(smem_u32(io + 3 * FS_TILE), &tmPrev, u0, m0, a.t > 0 ? a.t - 1 : 0, iob);
      for (int i = 0; i < first; ++i)
        tma_load_3d(smem_u32(smem + (size_t)i * FS_STAGE), &tmA, i * FS_KB, m0, 0, smem_u32(&bar_full[i]));
      for (int i = first; i < a.nkb; ++i) {
        const int s = i % FS_STAGES, round = i / FS_STAGES;
        if (round > 0 && !mbar_wait(smem_u32(&bar_empty[s]), (round - 1) & 1, deadp, status)) break;
        const uint32_t full = smem_u32(&bar_full[s]);
        mbar_expect_tx(full, FS_STAGE);
        unsigned char* st = smem + (size_t)s * FS_STAGE;
#pragma unroll
        for (int g = 0; g < 3; ++g)
          tma_load_3d(smem_u32(st + FS_A_BYTES + g * FS_B_SLAB), &tmB, i * FS_KB, g * H + u0, 0, full);
        tma_load_3d(smem_u32(st), &tmA, i * FS_KB, m0, 0, full);
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0 && !*deadp) {
      bool alive = true;
      for (int i = 0; i < a.nkb && alive; ++i) {
        const int s = i % FS_STAGES, round = i / FS_STAGES;
        if (!mbar_wait(smem_u32(&bar_full[s]), round & 1, deadp, status)) { alive = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)s * FS_STAGE);
        const uint32_t sb = sa + FS_A_BYTES;
#pragma unroll
        for (int kk = 0; kk < FS_KB / 32; ++kk)
          umma<true>(tmem_acc, umma_smem_desc(sa + kk * 32, 16, 1024), umma_smem_desc(sb + kk * 32, 16, 1024), IDESC,
                     (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(smem_u32(&bar_empty[s]));
      }
      if (alive) umma_commit(smem_u32(&bar_acc));
    }
  } else {
    pdl_wait();
    // ---- epilogue: thread = (batch row, 16 units)
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int r = q * 32 + lane;                    // row inside the tile
    const int b = m0 + r;
    const int ub = half * 16;                       // first unit of this thread inside the CTA's 32
    bool ok = mbar_wait(smem_u32(&bar_io), 0, deadp, status);
    if (ok) ok = mbar_wait(smem_u32(&bar_acc), 0, deadp, status);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    uint32_t ar[16], az[16], an[16];
    if (ok) {
      const uint32_t tsrc = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)ub;
      tmem_ld16(tsrc, ar);
      tmem_ld16(tsrc + FS_UNITS, az);
      tmem_ld16(tsrc + 2 * FS_UNITS, an);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) { ar[j] = 0u; az[j] = 0u; an[j] = 0u; }
    }
    // every MMA has completed (bar_acc): the operand ring is free and takes the output tiles
    unsigned char* stage_out = smem;                // out, r, z, n, gh_n: five 16 KB tiles
    uint32_t cw[4];
#pragma unroll
    for (int j4 = 0; j4 < 16; j4 += 4) {
      const int c = (ub + j4) >> 2;                 // 16-byte chunk of the row
      const float4 vr = *tile_chunk(io, r, c);
      const float4 vz = *tile_chunk(io + FS_TILE, r, c);
      const float4 vn = *tile_chunk(io + 2 * FS_TILE, r, c);
      const float4 vh = *tile_chunk(io + 3 * FS_TILE, r, c);
      const float gir[4] = {vr.x, vr.y, vr.z, vr.w}, giz[4] = {vz.x, vz.y, vz.z, vz.w};
      const float gin[4] = {vn.x, vn.y, vn.z, vn.w}, hp[4] = {vh.x, vh.y, vh.z, vh.w};
      float hn[4], rr[4], zz[4], nn[4], gg[4];
      uint32_t packed = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j4 + e, cc = ub + j;
        const float ghr = (float)(int)ar[j] * s_scale[cc] + s_bias[cc];
        const float ghz = (float)(int)az[j] * s_scale[FS_UNITS + cc] + s_bias[FS_UNITS + cc];
        const float ghn = (float)(int)an[j] * s_scale[2 * FS_UNITS + cc] + s_bias[2 * FS_UNITS + cc];
        const GateOut go = gru_gates(gir[e], giz[e], gin[e], ghr, ghz, ghn, hp[e]);
        rr[e] = go.r; zz[e] = go.z; nn[e] = go.n; gg[e] = ghn;
        hn[e] = a.qout.enabled ? fake_quant<true>(go.h_raw, a.qout) : go.h_raw;
        const float code = fminf(fmaxf(fq_code(hn[e], a.qin), a.qin.qmin), a.qin.qmax);
        packed |= ((uint32_t)(int)code & 0xffu) << (8 * e);
      }
      cw[j4 >> 2] = packed;
      *tile_chunk(stage_out, r, c) = make_float4(hn[0], hn[1], hn[2], hn[3]);
      if (a.has_save) {
        *tile_chunk(stage_out + FS_TILE, r, c) = make_float4(rr[0], rr[1], rr[2], rr[3]);
        *tile_chunk(stage_out + 2 * FS_TILE, r, c) = make_float4(zz[0], zz[1], zz[2], zz[3]);
        *tile_chunk(stage_out + 3 * FS_TILE, r, c) = make_float4(nn[0], nn[1], nn[2], nn[3]);
        *tile_chunk(stage_out + 4 * FS_TILE, r, c) = make_float4(gg[0], gg[1], gg[2], gg[3]);
      }
    }
    if (a.codes_next != nullptr && b < a.B)
      *reinterpret_cast<uint4*>(a.codes_next + (size_t)b * H + u0 + ub) = make_uint4(cw[0], cw[1], cw[2], cw[3]);
    // hand the tiles to the TMA engine: all epilogue threads' writes first, then one thread stores
    fence_async_smem();
    asm volatile("bar.sync 1, %0;" ::"n"(32 * FS_EPI_WARPS) : "memory");
    if (warp == 2 && lane == 0 && ok) {
      tma_store_3d(&tmOut, u0, m0, a.t, smem_u32(stage_out));
      if (a.has_save) {
#pragma unroll
        for (int k = 0; k < 4; ++k) tma_store_3d(&tmSave, u0, m0, k * a.T + a.t, smem_u32(stage_out + (k + 1) * FS_TILE));
      }
      tma_store_commit_and_wait();
    }
  }

  if (warp == 0 && lane == 0 && *deadp) {        // a CTA that gave up: let tile copies in flight land
    const long long start = clock64();
    while (clock64() - start < (1ll << 18)) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_acc, 128);
  }
}

int prepare_once(const void* kernel, int smem) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return B200GRU_LAUNCH_FAILURE;
  std::lock_guard<std::mutex> lk(mu);
  const auto key = std::make_pair(dev, kernel);
  if (done.count(key) == 0) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return check_launch("cudaFuncSetAttribute(tc_fwd_step_kernel)");
    done.insert(key);
  }
  return B200GRU_OK;
}

}  // namespace

int tc_step_read_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_step_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_tc_step_status, &z, sizeof(int));
  }
  return v;
}

int FusedFwd::init(const signed char* w_codes, signed char* h_codes0, signed char* h_codes1, const float* gi,
                   const float* h0, float* out, float* save, int T_, int B_, int H_) {
  T = T_; B = B_; H = H_;
  const unsigned long long uH = H, uB = B, uT = T;
  int rc = make_tensor_map_3d(&mapW, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_codes, uH, 3 * uH, 1, uH, 3 * uH * uH, FS_KB, FS_UNITS);
  if (rc) return rc;
  signed char* bufs[2] = {h_codes0, h_codes1};
  for (int i = 0; i < 2; ++i) {
    rc = make_tensor_map_3d(&mapH[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, bufs[i], uH, uB, 1, uH, uB * uH, FS_KB, FS_BM);
    if (rc) return rc;
  }
  // fp32 tiles of [128 rows][32 units]: gi[T][B][3H], h0[B][H], out[T][B][H], save[4T][B][H]
  rc = make_tensor_map_3d(&mapGi, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, gi, 3 * uH, uB, uT, 3 * uH * 4, uB * 3 * uH * 4, FS_UNITS, FS_BM);
  if (rc) return rc;
  rc = make_tensor_map_3d(&mapH0, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, h0, uH, uB, 1, uH * 4, uB * uH * 4, FS_UNITS, FS_BM);
  if (rc) return rc;
  rc = make_tensor_map_3d(&mapOut, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, out, uH, uB, uT, uH * 4, uB * uH * 4, FS_UNITS, FS_BM);
  if (rc) return rc;
  has_save = save != nullptr;
  rc = make_tensor_map_3d(&mapSave, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, has_save ? save : out, uH, uB, has_save ? 4 * uT : uT,
                          uH * 4, uB * uH * 4, FS_UNITS, FS_BM);
  if (rc) return rc;
  nkb = cdiv(H, FS_KB);
  return prepare_once(reinterpret_cast<const void*>(tc_fwd_step_kernel), FS_SMEM);
}

int FusedFwd::step(int t, int src, const float* col_scale, const float* bh, signed char* codes_next, float alpha,
                   Quant qin, Quant qout, cudaStream_t st) const {
  FusedFwdArgs a;
  memset(&a, 0, sizeof(a));
  a.col_scale = col_scale; a.bh = bh; a.codes_next = codes_next; a.t = t; a.T = T; a.B = B; a.H = H; a.nkb = nkb;
  a.has_save = has_save ? 1 : 0; a.alpha = alpha; a.qin = qin; a.qout = qout;
  const dim3 grid(H / FS_UNITS, cdiv(B, FS_BM));
  launch_pdl(tc_fwd_step_kernel, grid, dim3(FS_THREADS), (size_t)FS_SMEM, st, mapH[src], mapW, mapGi,
             t == 0 ? mapH0 : mapOut, mapOut, mapSave, a);
  note_launch();
  return B200GRU_OK;
}

}  // namespace tc
}  // namespace b200gru
