// Host interface of the fused tensor-core forward step (tc_step.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200gru {
namespace tc {

// One scan's worth of launch state for the int8 x int8 forward step: tensor maps of the weight
// codes [3H,H] and of the two alternating hidden-code buffers [B,H], encoded once per scan.
struct FusedFwd {
  alignas(64) CUtensorMap mapW;
  alignas(64) CUtensorMap mapH[2];
  int B, H, nkb, stages, smem;

  int init(const signed char* w_codes, signed char* h_codes0, signed char* h_codes1, int B, int H);
  // Step t: reads hidden codes from buffer `src`, writes out_t, save (optional) and the codes of
  // h_t into codes_next (NULL at the last step).  alpha = scale of the hidden codes.
  int step(int t, int T, int src, const float* gi, const float* h_prev, const float* col_scale, const float* bh,
           float* out_t, float* save, signed char* codes_next, float alpha, Quant qin, Quant qout,
           cudaStream_t st) const;
};

}  // namespace tc
}  // namespace b200gru
