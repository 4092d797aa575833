// activations.cu -- elementwise activations of feed-forward layers on fp32 rows (ditenex.h): xIELU with its two learned
// numbers, the SiLU-gated product of a [gate | up] row, and the gated product with the activation as an argument over
// fp32 or bf16 rows (dedunex.h).
#include "dedunex.h"
#include "ditenex.h"
#include "launch.h"

namespace qie {
namespace {

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

__global__ void xielu_kernel(float* __restrict__ z, int ld, int cols, const bf16* __restrict__ pq) {
  pdl_wait();
  pdl_trigger();
  const float ap = softplus_f(bf2f(pq[0])), an = 0.5f + softplus_f(bf2f(pq[1]));
  float* row = z + (size_t)blockIdx.x * ld;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const float v = row[i];
    row[i] = v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v);
  }
}

__global__ void silu_glu_kernel(const float* gu, int ld, float* out, int ldo, int ff) {  // out may be gu (a thread reads its elements first)
  pdl_wait();
  pdl_trigger();
  const float* row = gu + (size_t)blockIdx.x * ld;
  float* o = out + (size_t)blockIdx.x * ldo;
  for (int i = threadIdx.x; i < ff; i += blockDim.x) {
    const float g = row[i];
    o[i] = g / (1.0f + expf(-g)) * row[ff + i];
  }
}

__global__ void xielu_bf16_kernel(bf16* __restrict__ z, int ld, int cols, const bf16* __restrict__ pq) {
  pdl_wait();
  pdl_trigger();
  const float ap = softplus_f(bf2f(pq[0])), an = 0.5f + softplus_f(bf2f(pq[1]));
  bf16* row = z + (size_t)blockIdx.x * ld;
  auto f = [&](float v) { return v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v); };
  if (cols % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0) {  // 8 elements per 16-byte access
    for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 8) {
      uint4 p = *reinterpret_cast<const uint4*>(row + i);
      p.x = pack2(f2bf(f(lo2f(p.x))), f2bf(f(hi2f(p.x)))), p.y = pack2(f2bf(f(lo2f(p.y))), f2bf(f(hi2f(p.y))));
      p.z = pack2(f2bf(f(lo2f(p.z))), f2bf(f(hi2f(p.z)))), p.w = pack2(f2bf(f(lo2f(p.w))), f2bf(f(hi2f(p.w))));
      *reinterpret_cast<uint4*>(row + i) = p;
    }
    return;
  }
  for (int i = threadIdx.x; i < cols; i += blockDim.x) row[i] = f2bf(f(bf2f(row[i])));
}

__global__ void silu_glu_bf16_kernel(const bf16* __restrict__ gu, int ld, bf16* __restrict__ out, int ldo, int ff) {
  pdl_wait();
  pdl_trigger();
  const bf16* row = gu + (size_t)blockIdx.x * ld;
  bf16* o = out + (size_t)blockIdx.x * ldo;
  auto f = [](float g, float u) { return g / (1.0f + expf(-g)) * u; };
  if (ff % 8 == 0 && ld % 8 == 0 && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(gu) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    for (int i = threadIdx.x * 8; i < ff; i += blockDim.x * 8) {
      const uint4 g = *reinterpret_cast<const uint4*>(row + i), u = *reinterpret_cast<const uint4*>(row + ff + i);
      uint4 p;
      p.x = pack2(f2bf(f(lo2f(g.x), lo2f(u.x))), f2bf(f(hi2f(g.x), hi2f(u.x)))), p.y = pack2(f2bf(f(lo2f(g.y), lo2f(u.y))), f2bf(f(hi2f(g.y), hi2f(u.y))));
      p.z = pack2(f2bf(f(lo2f(g.z), lo2f(u.z))), f2bf(f(hi2f(g.z), hi2f(u.z)))), p.w = pack2(f2bf(f(lo2f(g.w), lo2f(u.w))), f2bf(f(hi2f(g.w), hi2f(u.w))));
      *reinterpret_cast<uint4*>(o + i) = p;
    }
    return;
  }
  for (int i = threadIdx.x; i < ff; i += blockDim.x) o[i] = f2bf(f(bf2f(row[i]), bf2f(row[ff + i])));
}


__device__ __forceinline__ float gated_act_f(int act, float g, float u) {
  const float a = act == 1 ? 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) : g / (1.0f + expf(-g));
  return a * u;
}

// one CTA per row
__global__ void gated_act_kernel(const GatedAct a) {
  pdl_wait();
  pdl_trigger();
  const size_t r = blockIdx.x;
  if (a.g_bf) {
    const bf16* g = a.g_bf + r * a.ld_bf;
    const bf16* u = a.u_bf + r * a.ld_bf;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (a.out_bf && !a.out && a.ff % 8 == 0 && a.ld_bf % 8 == 0 && a.ldo_bf % 8 == 0 && al(a.g_bf) && al(a.u_bf) && al(a.out_bf)) {
      bf16* o = a.out_bf + r * a.ldo_bf;
      for (int i = threadIdx.x * 8; i < a.ff; i += blockDim.x * 8) {  // 8 elements per 16-byte access
        const uint4 gv = *reinterpret_cast<const uint4*>(g + i), uv = *reinterpret_cast<const uint4*>(u + i);
        uint4 p;
        p.x = pack2(f2bf(gated_act_f(a.act, lo2f(gv.x), lo2f(uv.x))), f2bf(gated_act_f(a.act, hi2f(gv.x), hi2f(uv.x))));
        p.y = pack2(f2bf(gated_act_f(a.act, lo2f(gv.y), lo2f(uv.y))), f2bf(gated_act_f(a.act, hi2f(gv.y), hi2f(uv.y))));
        p.z = pack2(f2bf(gated_act_f(a.act, lo2f(gv.z), lo2f(uv.z))), f2bf(gated_act_f(a.act, hi2f(gv.z), hi2f(uv.z))));
        p.w = pack2(f2bf(gated_act_f(a.act, lo2f(gv.w), lo2f(uv.w))), f2bf(gated_act_f(a.act, hi2f(gv.w), hi2f(uv.w))));
        *reinterpret_cast<uint4*>(o + i) = p;
      }
      return;
    }
    for (int i = threadIdx.x; i < a.ff; i += blockDim.x) {
      const float v = gated_act_f(a.act, bf2f(g[i]), bf2f(u[i]));
      if (a.out) a.out[r * a.ldo + i] = v;
      if (a.out_bf) a.out_bf[r * a.ldo_bf + i] = f2bf(v);
    }
    return;
  }
  const float* g = a.g + r * a.ld;
  const float* u = a.u + r * a.ld;
  for (int i = threadIdx.x; i < a.ff; i += blockDim.x) {
    const float v = gated_act_f(a.act, g[i], u[i]);
    if (a.out) a.out[r * a.ldo + i] = v;
    if (a.out_bf) a.out_bf[r * a.ldo_bf + i] = f2bf(v);
  }
}

}  // namespace

cudaError_t launch_gated_act(const GatedAct& a, cudaStream_t st) {
  if (a.n <= 0 || a.ff <= 0) return cudaSuccess;
  if (!(a.g && a.u) && !(a.g_bf && a.u_bf)) return cudaErrorInvalidValue;
  if ((!a.out && !a.out_bf) || a.act < 0 || a.act > 1) return cudaErrorInvalidValue;
  return launch_k(gated_act_kernel, dim3(a.n), dim3(256), 0, st, a);
}

cudaError_t launch_xielu_bf16(bf16* z, int ld, int cols, const bf16* pq, int n, cudaStream_t st) {
  if (n <= 0 || cols <= 0) return cudaSuccess;
  return launch_k(xielu_bf16_kernel, dim3(n), dim3(256), 0, st, z, ld, cols, pq);
}

cudaError_t launch_silu_glu_bf16(const bf16* gu, int ld, bf16* out, int ldo, int ff, int n, cudaStream_t st) {
  if (n <= 0 || ff <= 0) return cudaSuccess;
  return launch_k(silu_glu_bf16_kernel, dim3(n), dim3(256), 0, st, gu, ld, out, ldo, ff);
}

cudaError_t launch_xielu(float* z, int ld, int cols, const bf16* pq, int n, cudaStream_t st) {
  if (n <= 0 || cols <= 0) return cudaSuccess;
  return launch_k(xielu_kernel, dim3(n), dim3(256), 0, st, z, ld, cols, pq);
}

cudaError_t launch_silu_glu(const float* gu, int ld, float* out, int ldo, int ff, int n, cudaStream_t st) {
  if (n <= 0 || ff <= 0) return cudaSuccess;
  return launch_k(silu_glu_kernel, dim3(n), dim3(256), 0, st, gu, ld, out, ldo, ff);
}

}  // namespace qie
