// rmsnorm_f32.cu -- RMS norms of a model whose sublayers sit between two norms (ditenex.h): the output norm folded
// into the residual add together with the next sublayer's input norm, and the input norm of a mixer that reads a blend
// of each row with the row before it (token shift) with one carried row per sequence slot.  All fp32, one CTA per row,
// every reduction in a fixed order per row, so a row's result does not depend on the rows it shares a launch with.
#include "ditenex.h"
#include "launch.h"
#include "moe_route.cuh"

namespace qie {
namespace {

__device__ __forceinline__ float block_sum_r(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // red may still be read from the previous call
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__global__ void __launch_bounds__(256) rms_step_kernel(const RmsStep a) {
  extern __shared__ float row[];  // [width]
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, W = a.width;
  const bool add = a.y || a.y_bf || a.mix.ye;
  const int src = a.gather ? a.gather[r] : r;  // the add half is never combined with a gather
  float* xr = a.x + (size_t)src * W;
  float sq = 0.f;
  if (add) {
    float s = 0.f;
    if (a.y || a.y_bf) {
      const float* y = a.y + (size_t)r * W;
      const bf16* yb = a.y_bf + (size_t)r * W;
      for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = a.y_bf ? bf2f(yb[i]) : y[i];
        row[i] = v;
        s = fmaf(v, v, s);
      }
    } else {  // the chosen experts' outputs of this row, weighted, plus the shared expert (gated only when mix.z is given)
      const MoeMix& m = a.mix;
      const bool shared = m.ys || a.ys_bf;
      const float sg = shared ? (m.z ? 1.0f / (1.0f + expf(-m.z[(size_t)r * m.ldz + m.gate_col])) : 1.0f) : 0.f;
      for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < m.top; ++k) v = fmaf(m.top_w[(size_t)r * m.top + k], m.ye[(size_t)m.slot_of[(size_t)r * m.top + k] * W + i], v);
        if (shared) v = fmaf(sg, a.ys_bf ? bf2f(a.ys_bf[(size_t)r * W + i]) : m.ys[(size_t)r * W + i], v);
        row[i] = v;
        s = fmaf(v, v, s);
      }
    }
    const float rstd = 1.0f / sqrtf(block_sum_r(s, red) / (float)W + a.eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = xr[i] + a.mult * (row[i] * rstd * bf2f(a.w_out[i]));
      xr[i] = v;
      row[i] = v;
      sq = fmaf(v, v, sq);
    }
  } else if (a.h || a.h_bf) {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = xr[i];
      row[i] = v;
      sq = fmaf(v, v, sq);
    }
  }
  if (!a.h && !a.h_bf) return;
  const float rstd = 1.0f / sqrtf(block_sum_r(sq, red) / (float)W + a.eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = row[i] * rstd * bf2f(a.w_in[i]);
    if (a.h) a.h[(size_t)r * W + i] = v;
    if (a.h_bf) a.h_bf[(size_t)r * W + i] = f2bf(v);
    row[i] = v;
  }
  if (!a.route.w_router) return;
  // router logits of the row: a warp per expert, lanes stride the width (16-byte weight loads when the rows allow it)
  const RouteRider& rt = a.route;
  float* zl = row + W;  // [experts] logits, then the router's scratch
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool vec = W % 8 == 0 && (reinterpret_cast<uintptr_t>(rt.w_router) & 15) == 0;
  for (int e = warp; e < rt.experts; e += nw) {
    const bf16* wr = rt.w_router + (size_t)e * W;
    float acc = 0.f;
    if (vec) {
      for (int i = lane * 8; i < W; i += 256) {
        const uint4 p = *reinterpret_cast<const uint4*>(wr + i);
        const float* h = row + i;
        acc = fmaf(h[0], lo2f(p.x), acc), acc = fmaf(h[1], hi2f(p.x), acc), acc = fmaf(h[2], lo2f(p.y), acc), acc = fmaf(h[3], hi2f(p.y), acc);
        acc = fmaf(h[4], lo2f(p.z), acc), acc = fmaf(h[5], hi2f(p.z), acc), acc = fmaf(h[6], lo2f(p.w), acc), acc = fmaf(h[7], hi2f(p.w), acc);
      }
    } else {
      for (int i = lane; i < W; i += 32) acc = fmaf(row[i], bf2f(wr[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) zl[e] = acc;
  }
  __syncthreads();
  if (warp == 0)
    route_sigmoid_row(zl, zl + rt.experts, rt.experts, rt.top, rt.groups, rt.keep, rt.correction, rt.scale, rt.top_idx + (size_t)r * rt.top,
                      rt.top_w + (size_t)r * rt.top, lane);
}

// one CTA per row.  The CTA of a segment's first row also moves the segment's last normed row into the carried row:
// each thread reads the old carried elements it needs before it overwrites exactly those, and no other CTA touches them.
__global__ void __launch_bounds__(256) rms_shift_kernel(const RmsShiftArgs a) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, W = a.width;
  // the segment of this row: the last s with seg_start[s] <= r
  int lo = 0, hi = a.n_seg - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (a.seg_start[mid] <= r) lo = mid;
    else hi = mid - 1;
  }
  const int first = a.seg_start[lo], last = a.seg_start[lo + 1] - 1;
  const bool head = r == first;
  const float* xr = a.x + (size_t)r * W;
  const float* xp = head ? a.x + (size_t)last * W : xr - W;  // the other row this CTA norms: the one before, or (first row) the segment's last
  float s0 = 0.f, s1 = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = xr[i], u = xp[i];
    s0 = fmaf(v, v, s0);
    s1 = fmaf(u, u, s1);
  }
  const float r0 = 1.0f / sqrtf(block_sum_r(s0, red) / (float)W + a.eps);
  const float r1 = 1.0f / sqrtf(block_sum_r(s1, red) / (float)W + a.eps);
  float* carry = a.carry + (size_t)a.seg_slot[lo] * a.slot_stride;
  float* out = a.out + (size_t)r * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float w = bf2f(a.w[i]);
    const float h = xr[i] * r0 * w, o = xp[i] * r1 * w;
    const float before = head ? carry[i] : o;
    const float v = h + (before - h) * bf2f(a.mu[i]);
    if (a.out) out[i] = v;
    if (a.out_bf) a.out_bf[(size_t)r * W + i] = f2bf(v);
    if (head) carry[i] = o;
  }
}

}  // namespace

cudaError_t launch_rms_step(const RmsStep& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  const bool add = a.y || a.y_bf || a.mix.ye, read = a.h || a.h_bf;
  if ((add && (!a.w_out || a.gather)) || (read && !a.w_in) || (!add && !read)) return cudaErrorInvalidValue;
  size_t smem = (size_t)a.width * sizeof(float);
  if (a.route.w_router) {
    const RouteRider& rt = a.route;
    if (!read || a.gather || rt.experts <= 0 || rt.top <= 0 || rt.top > rt.experts || rt.groups <= 0 || rt.experts % rt.groups || rt.keep <= 0 ||
        rt.keep > rt.groups || !rt.top_idx || !rt.top_w)
      return cudaErrorInvalidValue;
    smem += ((size_t)rt.experts + route_scratch_floats(rt.experts, rt.groups)) * sizeof(float);
  }
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t r = cudaFuncSetAttribute(rms_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (r != cudaSuccess) return r;
  }
  return launch_k(rms_step_kernel, dim3(a.n), dim3(256), smem, st, a);
}

cudaError_t launch_rms_shift(const RmsShiftArgs& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  if (a.n_seg <= 0 || !a.seg_start || !a.seg_slot || !a.carry) return cudaErrorInvalidValue;
  return launch_k(rms_shift_kernel, dim3(a.n), dim3(256), 0, st, a);
}

}  // namespace qie
