// moe.cu -- routing of a mixture-of-experts feed-forward (nogatar.h): softmax router with top-k choice and
// renormalised weights, the grouping of (row, choice) assignments by expert for the grouped expert GEMMs
// (launch_gemm_f32 with grp_off / row_idx), and the weighted combine with an optional gated shared expert.
// All of it fp32; a row's choice, weights and sums do not depend on the other rows of the launch (its slot in
// the grouped buffers does, the values stored there do not).
#include "launch.h"
#include "nogatar.h"

namespace qie {
namespace {

// one warp per row; shared memory: per warp `experts` scores
__global__ void moe_route_kernel(const float* __restrict__ z, int ldz, int experts, int top, int* __restrict__ top_idx,
                                 float* __restrict__ top_w, int n) {
  extern __shared__ float sc[];
  pdl_wait();
  pdl_trigger();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + w;
  if (r >= n) return;
  float* s = sc + (size_t)w * experts;
  const float* zr = z + (size_t)r * ldz;
  float mx = -INFINITY;
  for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, zr[e]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) {
    const float v = expf(zr[e] - mx);
    s[e] = v;
    sum += v;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  float chosen_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float bv = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = s[e];
      if (v > bv) {  // ascending e: the lowest index wins among equals
        bv = v;
        bi = e;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    const float score = bv / sum;
    if (lane == 0) {
      top_idx[(size_t)r * top + k] = bi;
      top_w[(size_t)r * top + k] = score;
      s[bi] = -2.f;
    }
    chosen_sum += score;
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = 1.0f / (chosen_sum + 1e-20f);
    for (int k = 0; k < top; ++k) top_w[(size_t)r * top + k] *= inv;
  }
}

// one CTA; warp w serves experts w, w + nw, ...: an ordered compaction of the assignments that chose the expert
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* top_idx, int n_assign, int top, int experts, int* grp_off,
                                                         int* __restrict__ perm_row, int* __restrict__ slot_of, int in_smem) {
  extern __shared__ int s_idx[];  // the assignments, when they fit (in_smem)
  pdl_wait();
  pdl_trigger();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (in_smem) {
    for (int i = threadIdx.x; i < n_assign; i += blockDim.x) s_idx[i] = top_idx[i];
    __syncthreads();
    top_idx = s_idx;
  }
  for (int e = w; e < experts; e += nw) {
    int cnt = 0;
    for (int i0 = 0; i0 < n_assign; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n_assign && top_idx[i] == e;
      cnt += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) grp_off[e + 1] = cnt;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    grp_off[0] = 0;
    for (int e = 0; e < experts; ++e) {
      run += grp_off[e + 1];
      grp_off[e + 1] = run;
    }
  }
  __syncthreads();
  for (int e = w; e < experts; e += nw) {
    int base = grp_off[e];
    for (int i0 = 0; i0 < n_assign; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n_assign && top_idx[i] == e;
      const unsigned b = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int s = base + __popc(b & ((1u << lane) - 1u));
        perm_row[s] = i / top;
        slot_of[i] = s;
      }
      base += __popc(b);
    }
  }
}

// The same grouping for many assignments: the 32 warps of one CTA each take a contiguous chunk; a step of 32 assignments
// finds, with one match, every lane's rank among the lanes of its expert.  Pass 1 counts per (warp, expert), a scan over
// (expert, warp) gives every warp its first slot per expert, pass 2 hands out the slots: ascending assignment order within
// an expert, exactly as the kernel above.  Shared memory: base [32][experts] ints.
__global__ void __launch_bounds__(1024) moe_group_chunked_kernel(const int* __restrict__ top_idx, int n_assign, int top, int experts,
                                                                 int* __restrict__ grp_off, int* __restrict__ perm_row, int* __restrict__ slot_of) {
  extern __shared__ int base[];  // [32][experts]
  pdl_wait();
  pdl_trigger();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = ((n_assign + 31) / 32 + 31) / 32 * 32;  // per warp, a multiple of 32
  const int i0 = w * chunk, i1 = min(n_assign, i0 + chunk);
  int* mine = base + w * experts;
  for (int e = lane; e < experts; e += 32) mine[e] = 0;
  __syncwarp();
  for (int s = i0; s < i1; s += 32) {
    const int i = s + lane;
    const bool on = i < i1;
    const int e = on ? top_idx[i] : -1 - lane;  // idle lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (on && (peers & ((1u << lane) - 1u)) == 0) mine[e] += __popc(peers);  // the first lane of each expert adds its count
    __syncwarp();
  }
  __syncthreads();
  // first slot of (expert, warp): experts in order, within an expert the warps in order
  if (w == 0) {
    int run = 0;
    for (int e0 = 0; e0 < experts; e0 += 32) {
      const int e = e0 + lane;
      int tot = 0;
      if (e < experts)
        for (int ww = 0; ww < 32; ++ww) tot += base[ww * experts + e];
      int inc = tot;  // inclusive scan over the 32 experts of this step
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      int first = run + inc - tot;
      if (e < experts) {
        grp_off[e] = first;
        for (int ww = 0; ww < 32; ++ww) {
          const int c = base[ww * experts + e];
          base[ww * experts + e] = first;
          first += c;
        }
      }
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) grp_off[experts] = run;
  }
  __syncthreads();
  for (int s = i0; s < i1; s += 32) {
    const int i = s + lane;
    const bool on = i < i1;
    const int e = on ? top_idx[i] : -1 - lane;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (on) {
      const int slot = mine[e] + __popc(peers & ((1u << lane) - 1u));
      perm_row[slot] = i / top;
      slot_of[i] = slot;
    }
    __syncwarp();
    if (on && (peers & ((1u << lane) - 1u)) == 0) mine[e] += __popc(peers);
    __syncwarp();
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ ye, const int* __restrict__ slot_of, const float* __restrict__ top_w, int top,
                                   const float* __restrict__ ys, const float* __restrict__ z, int ldz, int gate_col, float* __restrict__ y,
                                   int width) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  float sg = 0.f;
  if (ys) sg = 1.0f / (1.0f + expf(-z[(size_t)r * ldz + gate_col]));
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) a = fmaf(top_w[(size_t)r * top + k], ye[(size_t)slot_of[(size_t)r * top + k] * width + i], a);
    if (ys) a = fmaf(sg, ys[(size_t)r * width + i], a);
    y[(size_t)r * width + i] = a;
  }
}

}  // namespace

cudaError_t launch_moe_route(const float* z, int ldz, int experts, int top, int* top_idx, float* top_w, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  int warps = 8;
  while (warps > 1 && (size_t)warps * experts * sizeof(float) > 40 * 1024) warps /= 2;
  if ((size_t)warps * experts * sizeof(float) > 48 * 1024) return cudaErrorInvalidValue;
  return launch_k(moe_route_kernel, dim3((n + warps - 1) / warps), dim3(32 * warps), (size_t)warps * experts * sizeof(float), st, z, ldz, experts,
                  top, top_idx, top_w, n);
}

cudaError_t launch_moe_group(const int* top_idx, int n_assign, int top, int experts, int* grp_off, int* perm_row, int* slot_of, cudaStream_t st) {
  if (n_assign <= 0) return cudaSuccess;
  if (n_assign >= 1024 && experts <= 1024) {  // many assignments: chunks over the warps instead of a warp per expert over all of them
    const size_t smem = (size_t)32 * experts * sizeof(int);
    if (smem > 48 * 1024) {
      cudaError_t r = cudaFuncSetAttribute(moe_group_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
      if (r != cudaSuccess) return r;
    }
    return launch_k(moe_group_chunked_kernel, dim3(1), dim3(1024), smem, st, top_idx, n_assign, top, experts, grp_off, perm_row, slot_of);
  }
  int threads = 32 * experts;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  const size_t bytes = (size_t)n_assign * sizeof(int);
  const int in_smem = bytes <= 160 * 1024 ? 1 : 0;
  if (in_smem && bytes > 48 * 1024) {
    cudaError_t r = cudaFuncSetAttribute(moe_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (r != cudaSuccess) return r;
  }
  return launch_k(moe_group_kernel, dim3(1), dim3(threads), in_smem ? bytes : 0, st, top_idx, n_assign, top, experts, grp_off, perm_row, slot_of,
                  in_smem);
}

cudaError_t launch_moe_combine(const float* ye, const int* slot_of, const float* top_w, int top, const float* ys, const float* z, int ldz,
                               int gate_col, float* y, int width, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  return launch_k(moe_combine_kernel, dim3(n), dim3(256), 0, st, ye, slot_of, top_w, top, ys, z, ldz, gate_col, y, width);
}

}  // namespace qie
