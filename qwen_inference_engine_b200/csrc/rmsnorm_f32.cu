// rmsnorm_f32.cu -- RMS norms of a model whose sublayers sit between two norms (ditenex.h): the output norm folded
// into the residual add together with the next sublayer's input norm, and the input norm of a mixer that reads a blend
// of each row with the row before it (token shift) with one carried row per sequence slot; and the grouped RMS norm of a
// model of parallel blocks (dedunex.h): the residual add of the two sublayer outputs and the next block's norm in one kernel.
// All fp32, one CTA per row, every reduction in a fixed order per row, so a row's result does not depend on the rows it
// shares a launch with.
#include "dedunex.h"
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

// V consecutive elements per thread and step (V = 4: 16-byte fp32 and 8-byte bf16 accesses when the width and the
// pointers allow it; V = 1 otherwise)
template <int V>
struct Pack {
  float v[V];
};
template <int V>
__device__ __forceinline__ Pack<V> ld_f32(const float* p) {
  Pack<V> r;
  if constexpr (V == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    r.v[0] = t.x, r.v[1] = t.y, r.v[2] = t.z, r.v[3] = t.w;
  } else {
    r.v[0] = p[0];
  }
  return r;
}
template <int V>
__device__ __forceinline__ Pack<V> ld_bf16(const bf16* p) {
  Pack<V> r;
  if constexpr (V == 4) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    r.v[0] = lo2f(t.x), r.v[1] = hi2f(t.x), r.v[2] = lo2f(t.y), r.v[3] = hi2f(t.y);
  } else {
    r.v[0] = bf2f(p[0]);
  }
  return r;
}
template <int V>
__device__ __forceinline__ void st_f32(float* p, const Pack<V>& r) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else p[0] = r.v[0];
}
template <int V>
__device__ __forceinline__ void st_bf16(bf16* p, const Pack<V>& r) {
  if constexpr (V == 4) *reinterpret_cast<uint2*>(p) = make_uint2(pack2(f2bf(r.v[0]), f2bf(r.v[1])), pack2(f2bf(r.v[2]), f2bf(r.v[3])));
  else p[0] = f2bf(r.v[0]);
}

template <int V>
__global__ void __launch_bounds__(256) rms_step_kernel(const RmsStep a) {
  extern __shared__ __align__(16) float row[];  // [width]
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, W = a.width;
  const int t0 = threadIdx.x * V, step = blockDim.x * V;
  const bool add = a.y || a.y_bf || a.mix.ye;
  const int src = a.gather ? a.gather[r] : r;  // the add half is never combined with a gather
  float* xr = a.x + (size_t)src * W;
  float sq = 0.f;
  if (add) {
    float s = 0.f;
    if (a.y || a.y_bf) {
      for (int i = t0; i < W; i += step) {
        const Pack<V> p = a.y_bf ? ld_bf16<V>(a.y_bf + (size_t)r * W + i) : ld_f32<V>(a.y + (size_t)r * W + i);
        st_f32<V>(row + i, p);
#pragma unroll
        for (int u = 0; u < V; ++u) s = fmaf(p.v[u], p.v[u], s);
      }
    } else {  // the chosen experts' outputs of this row, weighted, plus the shared expert (gated only when mix.z is given)
      const MoeMix& m = a.mix;
      const bool shared = m.ys || a.ys_bf;
      const float sg = shared ? (m.z ? 1.0f / (1.0f + expf(-m.z[(size_t)r * m.ldz + m.gate_col])) : 1.0f) : 0.f;
      for (int i = t0; i < W; i += step) {
        Pack<V> p;
#pragma unroll
        for (int u = 0; u < V; ++u) p.v[u] = 0.f;
        for (int k = 0; k < m.top; ++k) {
          const float wk = m.top_w[(size_t)r * m.top + k];
          const Pack<V> e = ld_f32<V>(m.ye + (size_t)m.slot_of[(size_t)r * m.top + k] * W + i);
#pragma unroll
          for (int u = 0; u < V; ++u) p.v[u] = fmaf(wk, e.v[u], p.v[u]);
        }
        if (shared) {
          const Pack<V> e = a.ys_bf ? ld_bf16<V>(a.ys_bf + (size_t)r * W + i) : ld_f32<V>(m.ys + (size_t)r * W + i);
#pragma unroll
          for (int u = 0; u < V; ++u) p.v[u] = fmaf(sg, e.v[u], p.v[u]);
        }
        st_f32<V>(row + i, p);
#pragma unroll
        for (int u = 0; u < V; ++u) s = fmaf(p.v[u], p.v[u], s);
      }
    }
    const float rstd = 1.0f / sqrtf(block_sum_r(s, red) / (float)W + a.eps);
    for (int i = t0; i < W; i += step) {
      const Pack<V> y = ld_f32<V>(row + i), x = ld_f32<V>(xr + i), w = ld_bf16<V>(a.w_out + i);
      Pack<V> o;
#pragma unroll
      for (int u = 0; u < V; ++u) {
        o.v[u] = x.v[u] + a.mult * (y.v[u] * rstd * w.v[u]);
        sq = fmaf(o.v[u], o.v[u], sq);
      }
      st_f32<V>(xr + i, o);
      st_f32<V>(row + i, o);
    }
  } else if (a.h || a.h_bf) {
    for (int i = t0; i < W; i += step) {
      const Pack<V> x = ld_f32<V>(xr + i);
      st_f32<V>(row + i, x);
#pragma unroll
      for (int u = 0; u < V; ++u) sq = fmaf(x.v[u], x.v[u], sq);
    }
  }
  if (!a.h && !a.h_bf) return;
  const float rstd = 1.0f / sqrtf(block_sum_r(sq, red) / (float)W + a.eps);
  for (int i = t0; i < W; i += step) {
    const Pack<V> x = ld_f32<V>(row + i), w = ld_bf16<V>(a.w_in + i);
    Pack<V> o;
#pragma unroll
    for (int u = 0; u < V; ++u) o.v[u] = x.v[u] * rstd * w.v[u];
    if (a.h) st_f32<V>(a.h + (size_t)r * W + i, o);
    if (a.h_bf) st_bf16<V>(a.h_bf + (size_t)r * W + i, o);
    st_f32<V>(row + i, o);
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
template <int V>
__global__ void __launch_bounds__(256) rms_shift_kernel(const RmsShiftArgs a) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, W = a.width;
  const int t0 = threadIdx.x * V, step = blockDim.x * V;
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
  for (int i = t0; i < W; i += step) {
    const Pack<V> v = ld_f32<V>(xr + i), u = ld_f32<V>(xp + i);
#pragma unroll
    for (int k = 0; k < V; ++k) s0 = fmaf(v.v[k], v.v[k], s0), s1 = fmaf(u.v[k], u.v[k], s1);
  }
  const float r0 = 1.0f / sqrtf(block_sum_r(s0, red) / (float)W + a.eps);
  const float r1 = 1.0f / sqrtf(block_sum_r(s1, red) / (float)W + a.eps);
  float* carry = a.carry + (size_t)a.seg_slot[lo] * a.slot_stride;
  for (int i = t0; i < W; i += step) {
    const Pack<V> v = ld_f32<V>(xr + i), u = ld_f32<V>(xp + i), w = ld_bf16<V>(a.w + i), mu = ld_bf16<V>(a.mu + i);
    Pack<V> before, o, res;
    if (head) before = ld_f32<V>(carry + i);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float h = v.v[k] * r0 * w.v[k];
      o.v[k] = u.v[k] * r1 * w.v[k];
      const float b = head ? before.v[k] : o.v[k];
      res.v[k] = h + (b - h) * mu.v[k];
    }
    if (a.out) st_f32<V>(a.out + (size_t)r * W + i, res);
    if (a.out_bf) st_bf16<V>(a.out_bf + (size_t)r * W + i, res);
    if (head) st_f32<V>(carry + i, o);
  }
}


// The row lies in shared memory.  Each of the `groups` parts is normed by a team of warps: with fewer groups than warps a
// group gets blockDim / 32 / groups warps whose partial sums meet in shared memory in a fixed order, else a warp walks the
// groups warp, warp + nw, ...  scale[g] receives 1 / sqrt(mean + eps) of every group.
__device__ __forceinline__ void group_rstd(const float* row, int W, int groups, float eps, float* red, float* scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, gs = W / groups;
  if (groups >= nw) {
    for (int g = warp; g < groups; g += nw) {
      float s = 0.f;
      for (int i = lane; i < gs; i += 32) s = fmaf(row[g * gs + i], row[g * gs + i], s);
      s = warp_sum(s);
      if (lane == 0) scale[g] = 1.0f / sqrtf(s / (float)gs + eps);
    }
  } else {
    const int wpg = nw / groups, g = warp / wpg, k = warp % wpg;
    float s = 0.f;
    if (g < groups)
      for (int i = k * 32 + lane; i < gs; i += 32 * wpg) s = fmaf(row[g * gs + i], row[g * gs + i], s);
    s = warp_sum(s);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (threadIdx.x < groups) {
      float t = 0.f;
      for (int j = 0; j < wpg; ++j) t += red[threadIdx.x * wpg + j];
      scale[threadIdx.x] = 1.0f / sqrtf(t / (float)gs + eps);
    }
  }
  __syncthreads();
}

template <int V>
__global__ void __launch_bounds__(256) group_norm_step_kernel(const GroupNormStep a) {
  extern __shared__ __align__(16) float row[];  // [width], then [groups] scales
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, W = a.width, gs = W / a.groups;
  float* scale = row + W;
  const int t0 = threadIdx.x * V, step = blockDim.x * V;
  const int src = a.gather ? a.gather[r] : r;
  float* xr = a.x + (size_t)src * W;
  bool changed = false;
  if (a.ids) {  // the embedding row, normed
    const bf16* er = a.embed + (size_t)a.ids[r] * W;
    for (int i = t0; i < W; i += step) st_f32<V>(row + i, ld_bf16<V>(er + i));
    __syncthreads();
    group_rstd(row, W, a.groups, a.eps, red, scale);
    for (int i = t0; i < W; i += step) {
      Pack<V> v = ld_f32<V>(row + i);
      const Pack<V> w = ld_bf16<V>(a.w_pre + i);
#pragma unroll
      for (int u = 0; u < V; ++u) v.v[u] = v.v[u] * scale[(i + u) / gs] * w.v[u];
      st_f32<V>(row + i, v);
    }
    changed = true;
  } else {
    for (int i = t0; i < W; i += step) st_f32<V>(row + i, ld_f32<V>(xr + i));
  }
  // every thread touches only its own elements of the row until the norm below
  if (a.y1 || a.y1_bf || a.y2 || a.y2_bf) {
    for (int i = t0; i < W; i += step) {
      Pack<V> v = ld_f32<V>(row + i);
      if (a.y1 || a.y1_bf) {
        const Pack<V> y = a.y1_bf ? ld_bf16<V>(a.y1_bf + (size_t)src * W + i) : ld_f32<V>(a.y1 + (size_t)src * W + i);
        if (a.y2 || a.y2_bf) {
          const Pack<V> z = a.y2_bf ? ld_bf16<V>(a.y2_bf + (size_t)src * W + i) : ld_f32<V>(a.y2 + (size_t)src * W + i);
#pragma unroll
          for (int u = 0; u < V; ++u) v.v[u] += y.v[u] + z.v[u];
        } else {
#pragma unroll
          for (int u = 0; u < V; ++u) v.v[u] += y.v[u];
        }
      } else {
        const Pack<V> z = a.y2_bf ? ld_bf16<V>(a.y2_bf + (size_t)src * W + i) : ld_f32<V>(a.y2 + (size_t)src * W + i);
#pragma unroll
        for (int u = 0; u < V; ++u) v.v[u] += z.v[u];
      }
      st_f32<V>(row + i, v);
    }
    changed = true;
  }
  if (a.dump)
    for (int i = t0; i < W; i += step) st_f32<V>(a.dump + (size_t)r * W + i, ld_f32<V>(row + i));
  if (a.step) {
    for (int i = t0; i < W; i += step) {
      Pack<V> v = ld_f32<V>(row + i);
      const Pack<V> s = ld_bf16<V>(a.step + i);
#pragma unroll
      for (int u = 0; u < V; ++u) v.v[u] += s.v[u];
      st_f32<V>(row + i, v);
    }
    changed = true;
  }
  if (changed)
    for (int i = t0; i < W; i += step) st_f32<V>(xr + i, ld_f32<V>(row + i));
  if (!a.h && !a.h_bf) return;
  __syncthreads();
  group_rstd(row, W, a.groups, a.eps, red, scale);
  for (int i = t0; i < W; i += step) {
    const Pack<V> x = ld_f32<V>(row + i), w = ld_bf16<V>(a.w_in + i);
    Pack<V> o;
#pragma unroll
    for (int u = 0; u < V; ++u) o.v[u] = x.v[u] * scale[(i + u) / gs] * w.v[u];
    if (a.h) st_f32<V>(a.h + (size_t)r * W + i, o);
    if (a.h_bf) st_bf16<V>(a.h_bf + (size_t)r * W + i, o);
  }
}

}  // namespace

cudaError_t launch_group_norm_step(const GroupNormStep& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  const bool read = a.h || a.h_bf;
  if (a.width <= 0 || a.groups <= 0 || a.width % a.groups || (read && !a.w_in) || (a.ids && (!a.embed || !a.w_pre || a.gather))) return cudaErrorInvalidValue;
  const size_t smem = ((size_t)a.width + a.groups) * sizeof(float);
  auto al = [](const void* p, size_t b) { return (reinterpret_cast<uintptr_t>(p) & (b - 1)) == 0; };
  const bool vec = a.width % 4 == 0 && al(a.x, 16) && al(a.y1, 16) && al(a.y2, 16) && al(a.y1_bf, 8) && al(a.y2_bf, 8) && al(a.dump, 16) && al(a.h, 16) &&
                   al(a.h_bf, 8) && al(a.w_in, 8) && al(a.w_pre, 8) && al(a.step, 8) && al(a.embed, 8);
  auto* kern = vec ? group_norm_step_kernel<4> : group_norm_step_kernel<1>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t r = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (r != cudaSuccess) return r;
  }
  return launch_k(kern, dim3(a.n), dim3(256), smem, st, a);
}

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
  // 16-byte accesses when every row starts on a 16-byte boundary (cudaMalloc'd buffers, width a multiple of 4)
  auto al = [](const void* p, size_t b) { return (reinterpret_cast<uintptr_t>(p) & (b - 1)) == 0; };
  const bool vec = a.width % 4 == 0 && al(a.x, 16) && al(a.y, 16) && al(a.y_bf, 8) && al(a.ys_bf, 8) && al(a.mix.ye, 16) && al(a.mix.ys, 16) &&
                   al(a.h, 16) && al(a.h_bf, 8) && al(a.w_out, 8) && al(a.w_in, 8);
  auto* kern = vec ? rms_step_kernel<4> : rms_step_kernel<1>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t r = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (r != cudaSuccess) return r;
  }
  return launch_k(kern, dim3(a.n), dim3(256), smem, st, a);
}

cudaError_t launch_rms_shift(const RmsShiftArgs& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  if (a.n_seg <= 0 || !a.seg_start || !a.seg_slot || !a.carry) return cudaErrorInvalidValue;
  auto al = [](const void* p, size_t b) { return (reinterpret_cast<uintptr_t>(p) & (b - 1)) == 0; };
  const bool vec = a.width % 4 == 0 && a.slot_stride % 4 == 0 && al(a.x, 16) && al(a.out, 16) && al(a.out_bf, 8) && al(a.carry, 16) && al(a.w, 8) &&
                   al(a.mu, 8);
  return vec ? launch_k(rms_shift_kernel<4>, dim3(a.n), dim3(256), 0, st, a) : launch_k(rms_shift_kernel<1>, dim3(a.n), dim3(256), 0, st, a);
}

}  // namespace qie
