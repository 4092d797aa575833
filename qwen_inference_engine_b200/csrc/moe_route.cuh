// moe_route.cuh -- the choice of a sigmoid router with a correction and group-limited top-k for ONE row, by one warp
// (ditenex.h: RouteRider, the rider of the norm in front of a mixture of experts, rmsnorm_f32.cu).
#pragma once
#include "common.cuh"

namespace qie {

// the largest value, the lowest index among equals; every lane returns the winner
__device__ __forceinline__ int warp_argmax_first(const float* v, int count, int lane) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int e = lane; e < count; e += 32) {
    const float x = v[e];
    if (bi == 0x7fffffff || x > bv) bv = x, bi = e;  // ascending e within a lane
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) bv = ov, bi = oi;
  }
  return bi;
}

// floats of scratch the warp needs: choice scores [experts] | plain scores [experts] | group scores [groups] | kept marks [groups]
__host__ __device__ inline size_t route_scratch_floats(int experts, int groups) { return (size_t)2 * experts + 2 * (size_t)groups; }

// z: the row's router logits (any memory the warp can read); scratch: route_scratch_floats() floats of shared memory
__device__ __forceinline__ void route_sigmoid_row(const float* z, float* scratch, int experts, int top, int groups, int keep,
                                                  const bf16* __restrict__ correction, float scale, int* __restrict__ top_idx,
                                                  float* __restrict__ top_w, int lane) {
  float* c = scratch;
  float* s = c + experts;
  float* gs = s + experts;
  float* kept = gs + groups;
  for (int e = lane; e < experts; e += 32) {
    const float v = 1.0f / (1.0f + expf(-z[e]));
    s[e] = v;
    c[e] = v + (correction ? bf2f(correction[e]) : 0.f);
  }
  __syncwarp();
  if (keep < groups) {
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {  // the two largest choice scores of the group
      float a = -INFINITY, b = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float x = c[e];
        if (x > a) b = a, a = x;
        else if (x > b) b = x;
      }
      gs[g] = per > 1 ? a + b : a;
      kept[g] = 0.f;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      const int bi = warp_argmax_first(gs, groups, lane);
      __syncwarp();
      if (lane == 0) gs[bi] = -INFINITY, kept[bi] = 1.f;
      __syncwarp();
    }
    // experts of the other groups drop out of the choice (not merely to zero: choice scores may be negative)
    for (int e = lane; e < experts; e += 32)
      if (kept[e / per] == 0.f) c[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    const int bi = warp_argmax_first(c, experts, lane);
    __syncwarp();
    if (lane == 0) {
      top_idx[k] = bi;
      top_w[k] = s[bi] * scale;
      c[bi] = -INFINITY;
    }
    __syncwarp();
  }
}

}  // namespace qie
