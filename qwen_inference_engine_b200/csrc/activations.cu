// activations.cu -- elementwise activations of feed-forward layers on fp32 rows (ditenex.h): xIELU with its two learned
// numbers, and the SiLU-gated product of a [gate | up] row.
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

}  // namespace

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
