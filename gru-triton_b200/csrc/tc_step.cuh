// Host interface of the fused tensor-core forward step (tc_step.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200gru {
namespace tc {

// One scan's worth of launch state for the int8 x int8 forward step: tensor maps of the weight
// codes [3H,H], of the two alternating hidden-code buffers [B,H] and of the fp32 tensors the gate
// epilogue reads and writes by TMA tiles (gi, h0, out, save), all encoded once per scan.
struct FusedFwd {
  alignas(64) CUtensorMap mapW;
  alignas(64) CUtensorMap mapH[2];
  alignas(64) CUtensorMap mapGi, mapH0, mapOut, mapSave;
  int T, B, H, nkb;
  bool has_save;

  // gi, h0, out 16-byte aligned, H % 32 == 0; save may be NULL.
  int init(const signed char* w_codes, signed char* h_codes0, signed char* h_codes1, const float* gi, const float* h0,
           float* out, float* save, int T, int B, int H);
  // Step t: reads hidden codes from buffer `src` and h_{t-1} from out[t-1] (h0 at t = 0), writes
  // out[t], save (optional) and the codes of h_t into codes_next (NULL at the last step).
  int step(int t, int src, const float* col_scale, const float* bh, signed char* codes_next, float alpha, Quant qin,
           Quant qout, cudaStream_t st) const;
};

}  // namespace tc
}  // namespace b200gru
