// ops_f32.cu -- operators of models whose residual stream, norms and reductions are fp32 (nogatar.h): scaled
// embedding gather, output LayerNorm folded into the residual add, a general fp32-accumulate GEMM (batched,
// grouped, gathered) and the logit soft cap.  Every reduction has a fixed order per row, so a row's result does
// not depend on the rows it shares a launch with.
#include "launch.h"
#include "dedunex.h"
#include "nogatar.h"

namespace qie {
namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  // fixed tree: warp shuffles, then warp 0 over the per-warp partials
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // red may still be read from the previous call
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__global__ void embed_scale_kernel(float* __restrict__ x, const bf16* __restrict__ table, const int* __restrict__ ids, int width,
                                   float scale) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const bf16* src = table + (size_t)ids[r] * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)r * width + i] = bf2f(src[i]) * scale;
}

__global__ void layernorm_f32_kernel(const float* __restrict__ y, const bf16* __restrict__ w, float* out, const float* res,
                                     const int* __restrict__ gather, int width, float eps, float mult, const MoeMix mix) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  float s = 0.f;
  if (y) {
    const float* src = y + (size_t)(gather ? gather[r] : r) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float v = src[i];
      row[i] = v;
      s += v;
    }
  } else {  // the experts' outputs of this row, weighted, plus the gated shared expert
    const float sg = mix.ys ? 1.0f / (1.0f + expf(-mix.z[(size_t)r * mix.ldz + mix.gate_col])) : 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float a = 0.f;
      for (int k = 0; k < mix.top; ++k)
        a = fmaf(mix.top_w[(size_t)r * mix.top + k], mix.ye[(size_t)mix.slot_of[(size_t)r * mix.top + k] * width + i], a);
      if (mix.ys) a = fmaf(sg, mix.ys[(size_t)r * width + i], a);
      row[i] = a;
      s += a;
    }
  }
  const float mean = block_sum(s, red) / (float)width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = row[i] - mean;
    q += d * d;
  }
  const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = (row[i] - mean) * rstd * bf2f(w[i]);
    const size_t o = (size_t)r * width + i;
    out[o] = res ? res[o] + mult * v : mult * v;
  }
}

constexpr int GT = 64, GK = 16;  // output tile, k step
constexpr int GEMV_MAX_ROWS = 16;  // up to this many rows (per launch, over all groups) the warp-per-column kernels run

__global__ void __launch_bounds__(256) gemm_f32_kernel(const GemmF32 g) {
  __shared__ float As[GK][GT + 4];
  __shared__ float Ws[GK][GT + 4];
  __shared__ int src_row[GT];
  pdl_wait();
  pdl_trigger();
  const int z = blockIdx.z;
  int row_base = 0, Mz = g.M;
  if (g.grp_off) {
    row_base = g.grp_off[z];
    Mz = g.grp_off[z + 1] - row_base;
  }
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  if (m0 >= Mz) return;
  const int tid = threadIdx.x;
  if (tid < GT) {
    const int m = m0 + tid;
    int s = -1;
    if (m < Mz) s = g.row_idx ? g.row_idx[row_base + m] : row_base + m;
    src_row[tid] = s;
  }
  __syncthreads();
  const float* A = g.A + (size_t)z * g.a_batch;
  const bf16* W = g.W + (size_t)z * g.w_batch;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < g.K; k0 += GK) {
    // A tile: 64 rows x 16 k, k fastest
    for (int i = tid; i < GT * GK; i += 256) {
      const int mm = i / GK, kk = i % GK;
      const int s = src_row[mm];
      float a = 0.f;
      if (s >= 0 && k0 + kk < g.K) {
        a = A[(size_t)s * g.lda + k0 + kk];
        if (g.round_a) a = bf2f(f2bf(a));
      }
      As[kk][mm] = a;
    }
    if (!g.w_trans) {
      for (int i = tid; i < GT * GK; i += 256) {
        const int nn = i / GK, kk = i % GK;
        float b = 0.f;
        if (n0 + nn < g.N && k0 + kk < g.K) b = bf2f(W[(size_t)(n0 + nn) * g.ldw + k0 + kk]);
        Ws[kk][nn] = b;
      }
    } else {
      for (int i = tid; i < GT * GK; i += 256) {
        const int kk = i / GT, nn = i % GT;
        float b = 0.f;
        if (n0 + nn < g.N && k0 + kk < g.K) b = bf2f(W[(size_t)(k0 + kk) * g.ldw + n0 + nn]);
        Ws[kk][nn] = b;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* C = g.C + (size_t)z * g.c_batch;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= Mz) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (g.bias) v += bf2f(g.bias[(size_t)z * g.bias_batch + n]);
      if (g.act == 1) {
        v = fmaxf(v, 0.f);
        v = v * v;
      }
      if (g.round_c) v = bf2f(f2bf(v));
      C[(size_t)(row_base + m) * g.ldc + n] = v;
    }
  }
}


// The same tile on tensor cores for bf16 operands (round_a): A is rounded to bf16 while it is staged, the products run
// as mma.sync m16n8k16 with fp32 accumulators, k ascending.  8 warps: warp w owns rows (w % 4) * 16 .. + 16 and columns
// (w / 4) * 32 .. + 32 of the 64 x 64 tile.  Rows of 32 k-elements are padded to 40 so that the 32-bit fragment loads
// of a warp fall into 32 different banks.
constexpr int MK = 32, MKP = 40;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(256) gemm_bf16_mma_kernel(const GemmF32 g) {
  __shared__ __align__(16) bf16 As[GT][MKP];
  __shared__ __align__(16) bf16 Ws[GT][MKP];
  __shared__ int src_row[GT];
  pdl_wait();
  pdl_trigger();
  const int z = blockIdx.z;
  int row_base = 0, Mz = g.M;
  if (g.grp_off) {
    row_base = g.grp_off[z];
    Mz = g.grp_off[z + 1] - row_base;
  }
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  if (m0 >= Mz) return;
  const int tid = threadIdx.x;
  if (tid < GT) {
    const int m = m0 + tid;
    src_row[tid] = m < Mz ? (g.row_idx ? g.row_idx[row_base + m] : row_base + m) : -1;
  }
  __syncthreads();
  const float* A = g.A + (size_t)z * g.a_batch;
  const bf16* W = g.W + (size_t)z * g.w_batch;
  const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int wm = (warp & 3) * 16, wn = (warp >> 2) * 32;
  float acc[4][4] = {};
  // staging: a thread moves 8 consecutive k of one row with 16-byte loads when the operands allow it
  const bool a_vec = g.lda % 4 == 0 && g.a_batch % 4 == 0 && (reinterpret_cast<uintptr_t>(g.A) & 15) == 0;
  const bool w_vec = !g.w_trans && g.ldw % 8 == 0 && g.w_batch % 8 == 0 && (reinterpret_cast<uintptr_t>(g.W) & 15) == 0;
  const int srow = tid >> 2, sk = (tid & 3) * 8;
  for (int k0 = 0; k0 < g.K; k0 += MK) {
    const bool full = k0 + MK <= g.K;
    if (a_vec && full) {
      const int s = src_row[srow];
      uint4 pk = make_uint4(0, 0, 0, 0);
      if (s >= 0) {
        const float4 v0 = *reinterpret_cast<const float4*>(A + (size_t)s * g.lda + k0 + sk);
        const float4 v1 = *reinterpret_cast<const float4*>(A + (size_t)s * g.lda + k0 + sk + 4);
        pk.x = pack2(f2bf(v0.x), f2bf(v0.y)), pk.y = pack2(f2bf(v0.z), f2bf(v0.w));
        pk.z = pack2(f2bf(v1.x), f2bf(v1.y)), pk.w = pack2(f2bf(v1.z), f2bf(v1.w));
      }
      *reinterpret_cast<uint4*>(&As[srow][sk]) = pk;
    } else {
      for (int i = tid; i < GT * MK; i += 256) {
        const int mm = i / MK, kk = i % MK;
        const int s = src_row[mm];
        As[mm][kk] = f2bf(s >= 0 && k0 + kk < g.K ? A[(size_t)s * g.lda + k0 + kk] : 0.f);
      }
    }
    if (w_vec && full) {
      uint4 pk = make_uint4(0, 0, 0, 0);
      if (n0 + srow < g.N) pk = *reinterpret_cast<const uint4*>(W + (size_t)(n0 + srow) * g.ldw + k0 + sk);
      *reinterpret_cast<uint4*>(&Ws[srow][sk]) = pk;
    } else if (!g.w_trans) {
      for (int i = tid; i < GT * MK; i += 256) {
        const int nn = i / MK, kk = i % MK;
        Ws[nn][kk] = n0 + nn < g.N && k0 + kk < g.K ? W[(size_t)(n0 + nn) * g.ldw + k0 + kk] : f2bf(0.f);
      }
    } else {
      for (int i = tid; i < GT * MK; i += 256) {
        const int kk = i / GT, nn = i % GT;
        Ws[nn][kk] = n0 + nn < g.N && k0 + kk < g.K ? W[(size_t)(k0 + kk) * g.ldw + n0 + nn] : f2bf(0.f);
      }
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < MK; ks += 16) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(&As[wm + gq][ks + 2 * tq]);
      a[1] = *reinterpret_cast<const uint32_t*>(&As[wm + gq + 8][ks + 2 * tq]);
      a[2] = *reinterpret_cast<const uint32_t*>(&As[wm + gq][ks + 2 * tq + 8]);
      a[3] = *reinterpret_cast<const uint32_t*>(&As[wm + gq + 8][ks + 2 * tq + 8]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t b[2];
        b[0] = *reinterpret_cast<const uint32_t*>(&Ws[wn + j * 8 + gq][ks + 2 * tq]);
        b[1] = *reinterpret_cast<const uint32_t*>(&Ws[wn + j * 8 + gq][ks + 2 * tq + 8]);
        mma_bf16_16816(acc[j], a, b);
      }
    }
    __syncthreads();
  }
  float* C = g.C + (size_t)z * g.c_batch;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int m = m0 + wm + gq + (u >> 1) * 8, n = n0 + wn + j * 8 + 2 * tq + (u & 1);
      if (m >= Mz || n >= g.N) continue;
      float v = acc[j][u];
      if (g.bias) v += bf2f(g.bias[(size_t)z * g.bias_batch + n]);
      if (g.act == 1) {
        v = fmaxf(v, 0.f);
        v = v * v;
      }
      if (g.round_c) v = bf2f(f2bf(v));
      C[(size_t)(row_base + m) * g.ldc + n] = v;
    }
  }
}

// Few output columns, many rows (router logits, gate pre-activations): the weights go to shared memory once per CTA,
// transposed to [k][NP] fp32 (NP = columns rounded up to 4), a warp per row reads its row once (k lane-strided) and
// keeps all columns' partial sums, fed by 16-byte shared-memory loads; then a shuffle tree.  The k order per output
// is fixed.  K is walked in chunks of SKINNY_KC.
constexpr int SKINNY_N = 64;  // widest case; instantiated for <= 32 columns (16 rows per CTA, k chunks of 1024) and <= 64 (8 rows, 512)
template <int SKINNY_N, int SKINNY_ROWS, int SKINNY_KC>
__global__ void __launch_bounds__(256) gemm_skinny_f32_kernel(const GemmF32 g) {
  extern __shared__ float4 s_w4[];
  float* s_w = reinterpret_cast<float*>(s_w4);
  pdl_wait();
  pdl_trigger();
  const int NP = (g.N + 3) & ~3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_base = blockIdx.x * SKINNY_ROWS;
  float acc[SKINNY_ROWS / 8][SKINNY_N];
#pragma unroll
  for (int r = 0; r < SKINNY_ROWS / 8; ++r)
#pragma unroll
    for (int n = 0; n < SKINNY_N; ++n) acc[r][n] = 0.f;
  for (int k0 = 0; k0 < g.K; k0 += SKINNY_KC) {
    const int kc = min(SKINNY_KC, g.K - k0);
    __syncthreads();
    if (g.ldw % 8 == 0 && kc % 8 == 0 && k0 % 8 == 0 && (reinterpret_cast<uintptr_t>(g.W) & 15) == 0) {
      const int kv = kc / 8;  // 16-byte pieces per weight row
      for (int i = threadIdx.x; i < NP * kv; i += 256) {
        const int n = i / kv, k = (i % kv) * 8;
        uint4 wv = make_uint4(0, 0, 0, 0);
        if (n < g.N) wv = *reinterpret_cast<const uint4*>(g.W + (size_t)n * g.ldw + k0 + k);
        const float wf[8] = {lo2f(wv.x), hi2f(wv.x), lo2f(wv.y), hi2f(wv.y), lo2f(wv.z), hi2f(wv.z), lo2f(wv.w), hi2f(wv.w)};
#pragma unroll
        for (int u = 0; u < 8; ++u) s_w[(k + u) * NP + n] = wf[u];
      }
    } else {
      for (int i = threadIdx.x; i < NP * kc; i += 256) {
        const int n = i / kc, k = i % kc;  // k fastest: coalesced weight reads
        s_w[k * NP + n] = n < g.N ? bf2f(g.W[(size_t)n * g.ldw + k0 + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < SKINNY_ROWS / 8; ++r) {
      const int m = m_base + warp + 8 * r;
      if (m >= g.M) continue;
      const float* a = g.A + (size_t)m * g.lda + k0;
#pragma unroll 4
      for (int k = lane; k < kc; k += 32) {
        float av = a[k];
        if (g.round_a) av = bf2f(f2bf(av));
        const float4* w4 = reinterpret_cast<const float4*>(s_w + (size_t)k * NP);
#pragma unroll
        for (int j = 0; j < SKINNY_N / 4; ++j) {
          if (j * 4 < NP) {
            const float4 wv = w4[j];
            acc[r][4 * j] = fmaf(av, wv.x, acc[r][4 * j]);
            acc[r][4 * j + 1] = fmaf(av, wv.y, acc[r][4 * j + 1]);
            acc[r][4 * j + 2] = fmaf(av, wv.z, acc[r][4 * j + 2]);
            acc[r][4 * j + 3] = fmaf(av, wv.w, acc[r][4 * j + 3]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < SKINNY_ROWS / 8; ++r) {
    const int m = m_base + warp + 8 * r;
    if (m >= g.M) continue;
#pragma unroll
    for (int n = 0; n < SKINNY_N; ++n) {
      if (n < g.N) {
        float v = acc[r][n];
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) {
          if (g.bias) v += bf2f(g.bias[n]);
          if (g.act == 1) {
            v = fmaxf(v, 0.f);
            v = v * v;
          }
          if (g.round_c) v = bf2f(f2bf(v));
          g.C[(size_t)m * g.ldc + n] = v;
        }
      }
    }
  }
}

// Few rows (decode steps, lightly loaded experts): one warp per output column streams the weight row with 16-byte
// loads and keeps up to 8 rows of partial sums; experts without rows leave at once, so a mixture of experts reads
// only the chosen experts' weights.  The k order per output is fixed (lane-strided, then a shuffle tree), whatever
// the number of rows.
template <bool VEC>
__global__ void __launch_bounds__(256) gemv_f32_kernel(const GemmF32 g) {
  pdl_wait();
  pdl_trigger();
  const int z = blockIdx.z;
  int row_base = 0, Mz = g.M;
  if (g.grp_off) {
    row_base = g.grp_off[z];
    Mz = g.grp_off[z + 1] - row_base;
  }
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (Mz <= 0 || n >= g.N) return;
  const float* A = g.A + (size_t)z * g.a_batch;
  const bf16* w = g.W + (size_t)z * g.w_batch + (size_t)n * g.ldw;
  float* C = g.C + (size_t)z * g.c_batch;
  for (int m0 = 0; m0 < Mz; m0 += 8) {
    const int mr = min(8, Mz - m0);
    const float* arow[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = m0 + min(i, mr - 1);
      arow[i] = A + (size_t)(g.row_idx ? g.row_idx[row_base + m] : row_base + m) * g.lda;
    }
    float acc[8] = {};
    if (VEC) {
      for (int k = lane * 8; k < g.K; k += 256) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
        const float wf[8] = {lo2f(wv.x), hi2f(wv.x), lo2f(wv.y), hi2f(wv.y), lo2f(wv.z), hi2f(wv.z), lo2f(wv.w), hi2f(wv.w)};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (i < mr) {
            const float4 a0 = *reinterpret_cast<const float4*>(arow[i] + k), a1 = *reinterpret_cast<const float4*>(arow[i] + k + 4);
            float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (g.round_a) av[j] = bf2f(f2bf(av[j]));
              acc[i] = fmaf(av[j], wf[j], acc[i]);
            }
          }
        }
      }
    } else {
      for (int k = lane; k < g.K; k += 32) {
        const float wf = bf2f(w[k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (i < mr) {
            float a = arow[i][k];
            if (g.round_a) a = bf2f(f2bf(a));
            acc[i] = fmaf(a, wf, acc[i]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    if (lane == 0) {
      for (int i = 0; i < mr; ++i) {
        float v = acc[i];
        if (g.bias) v += bf2f(g.bias[(size_t)z * g.bias_batch + n]);
        if (g.act == 1) {
          v = fmaxf(v, 0.f);
          v = v * v;
        }
        if (g.round_c) v = bf2f(f2bf(v));
        C[(size_t)(row_base + m0 + i) * g.ldc + n] = v;
      }
    }
  }
}

// the same for W stored [k, n]: one thread per output column (coalesced over n), k ascending
__global__ void gemv_trans_f32_kernel(const GemmF32 g) {
  pdl_wait();
  pdl_trigger();
  const int z = blockIdx.z, m = blockIdx.y, n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= g.N) return;
  const float* a = g.A + (size_t)z * g.a_batch + (size_t)m * g.lda;
  const bf16* w = g.W + (size_t)z * g.w_batch + n;
  float acc = 0.f;
  for (int k = 0; k < g.K; ++k) {
    float av = a[k];
    if (g.round_a) av = bf2f(f2bf(av));
    acc = fmaf(av, bf2f(w[(size_t)k * g.ldw]), acc);
  }
  if (g.round_c) acc = bf2f(f2bf(acc));
  g.C[(size_t)z * g.c_batch + (size_t)m * g.ldc + n] = acc;
}

__global__ void softcap_kernel(float* z, size_t n, float cap) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

__global__ void cast_f32_bf16_kernel(const float* in, bf16* out, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = f2bf(in[i]);
}

// rows of a strided fp32 matrix -> dense bf16 rows (operand of a tensor-core GEMM); with row_idx a gather
__global__ void rows_f32_to_bf16_kernel(const float* __restrict__ in, int ld_in, const int* __restrict__ row_idx, bf16* __restrict__ out, int cols) {
  pdl_wait();
  pdl_trigger();
  const float* src = in + (size_t)(row_idx ? row_idx[blockIdx.x] : blockIdx.x) * ld_in;
  bf16* dst = out + (size_t)blockIdx.x * cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) dst[i] = f2bf(src[i]);
}

// dense bf16 rows -> rows of a strided fp32 matrix, with the activation of GemmF32::act
__global__ void rows_bf16_to_f32_kernel(const bf16* __restrict__ in, int ld_in, int cols, float* __restrict__ out, int ld_out, int act) {
  pdl_wait();
  pdl_trigger();
  const bf16* src = in + (size_t)blockIdx.x * ld_in;
  float* dst = out + (size_t)blockIdx.x * ld_out;
  if (act == 0 && cols % 8 == 0 && ld_in % 8 == 0 && ld_out % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    for (int i = threadIdx.x * 8; i < cols; i += blockDim.x * 8) {  // 8 elements per 16-byte load
      const uint4 p = *reinterpret_cast<const uint4*>(src + i);
      *reinterpret_cast<float4*>(dst + i) = make_float4(lo2f(p.x), hi2f(p.x), lo2f(p.y), hi2f(p.y));
      *reinterpret_cast<float4*>(dst + i + 4) = make_float4(lo2f(p.z), hi2f(p.z), lo2f(p.w), hi2f(p.w));
    }
    return;
  }
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = bf2f(src[i]);
    if (act == 1) {
      v = fmaxf(v, 0.f);
      v = bf2f(f2bf(v * v));
    }
    dst[i] = v;
  }
}

// one CTA per row: the largest logit, the lowest index among equals.  A thread walks its elements in ascending index (four
// at a time when the row allows 16-byte loads) and keeps the first of equal values; the tree prefers the lower index.
__global__ void __launch_bounds__(1024) argmax_f32_kernel(const float* __restrict__ z, int* __restrict__ out, int vocab) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_wait();
  pdl_trigger();
  const float* row = z + (size_t)blockIdx.x * vocab;
  float v = -INFINITY;
  int idx = 0x7fffffff;
  if (vocab % 4 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
      const float4 x = row4[i];
      if (x.x > v) v = x.x, idx = 4 * i;
      if (x.y > v) v = x.y, idx = 4 * i + 1;
      if (x.z > v) v = x.z, idx = 4 * i + 2;
      if (x.w > v) v = x.w, idx = 4 * i + 3;
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float x = row[i];
      if (x > v) v = x, idx = i;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) v = ov, idx = oi;
  }
  if ((threadIdx.x & 31) == 0) bv[threadIdx.x >> 5] = v, bi[threadIdx.x >> 5] = idx;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    v = threadIdx.x < nw ? bv[threadIdx.x] : -INFINITY;
    idx = threadIdx.x < nw ? bi[threadIdx.x] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) v = ov, idx = oi;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}

}  // namespace

cudaError_t launch_rows_f32_to_bf16(const float* in, int ld_in, const int* row_idx, bf16* out, int cols, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  return launch_k(rows_f32_to_bf16_kernel, dim3(n), dim3(256), 0, st, in, ld_in, row_idx, out, cols);
}

cudaError_t launch_rows_bf16_to_f32(const bf16* in, int cols, float* out, int ld_out, int act, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  return launch_k(rows_bf16_to_f32_kernel, dim3(n), dim3(256), 0, st, in, cols, cols, out, ld_out, act);
}

cudaError_t launch_rows_bf16_to_f32_ld(const bf16* in, int ld_in, int cols, float* out, int ld_out, int n, cudaStream_t st) {
  if (n <= 0 || cols <= 0) return cudaSuccess;
  return launch_k(rows_bf16_to_f32_kernel, dim3(n), dim3(256), 0, st, in, ld_in, cols, out, ld_out, 0);
}

cudaError_t launch_argmax_f32(const float* z, int* out, int n_rows, int vocab, cudaStream_t st) {
  if (n_rows <= 0) return cudaSuccess;
  return launch_k(argmax_f32_kernel, dim3(n_rows), dim3(vocab >= 8192 ? 1024 : 256), 0, st, z, out, vocab);
}

cudaError_t launch_gemm_f32(const GemmF32& g, cudaStream_t st) {
  if (g.M <= 0 || g.N <= 0 || g.batches <= 0) return cudaSuccess;
  // grouped problems (experts) split their rows, so the warp-per-column kernel pays up to far more rows in total
  if (g.M <= (g.grp_off ? 16 * GEMV_MAX_ROWS : GEMV_MAX_ROWS)) {
    if (g.w_trans && !g.grp_off && !g.row_idx && !g.bias && g.act == 0)
      return launch_k(gemv_trans_f32_kernel, dim3((g.N + 127) / 128, g.M, g.batches), dim3(128), 0, st, g);
    if (!g.w_trans) {
      const bool vec = g.K % 8 == 0 && g.ldw % 8 == 0 && g.w_batch % 8 == 0 && g.lda % 4 == 0 && g.a_batch % 4 == 0 &&
                       (reinterpret_cast<uintptr_t>(g.W) & 15) == 0 && (reinterpret_cast<uintptr_t>(g.A) & 15) == 0;
      const dim3 grid((g.N + 7) / 8, 1, g.batches);
      return vec ? launch_k(gemv_f32_kernel<true>, grid, dim3(256), 0, st, g) : launch_k(gemv_f32_kernel<false>, grid, dim3(256), 0, st, g);
    }
  }
  // few columns: the fp32 kernel below, unless the operands are bf16 values anyway (round_a) and the rows are many: then the
  // tensor-core tile kernel is several times faster even with most of its 64 columns idle
  if (g.N <= SKINNY_N && !g.w_trans && !g.grp_off && !g.row_idx && g.batches == 1 && !(g.round_a && g.M >= 256)) {
    const bool wide = g.N > 32;
    const size_t smem = (size_t)((g.N + 3) & ~3) * (wide ? 512 : 1024) * sizeof(float);  // <= 128 KB
    auto* kern = wide ? gemm_skinny_f32_kernel<64, 8, 512> : gemm_skinny_f32_kernel<32, 16, 1024>;
    if (smem > 48 * 1024) {
      cudaError_t r = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
      if (r != cudaSuccess) return r;
    }
    return launch_k(kern, dim3((g.M + (wide ? 8 : 16) - 1) / (wide ? 8 : 16)), dim3(256), smem, st, g);
  }
  dim3 grid((g.N + GT - 1) / GT, (g.M + GT - 1) / GT, g.batches);
  if (g.round_a) return launch_k(gemm_bf16_mma_kernel, grid, dim3(256), 0, st, g);  // bf16 operands: tensor cores
  return launch_k(gemm_f32_kernel, grid, dim3(256), 0, st, g);
}

cudaError_t launch_embed_scale_f32(float* x, const bf16* table, const int* ids, int width, int n, float scale, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  return launch_k(embed_scale_kernel, dim3(n), dim3(256), 0, st, x, table, ids, width, scale);
}

cudaError_t launch_layernorm_f32(const float* y, const bf16* w, float* out, const float* res, const int* gather, int width, int n,
                                 float eps, float mult, cudaStream_t st, const MoeMix& mix) {
  if (n <= 0) return cudaSuccess;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t r = cudaFuncSetAttribute(layernorm_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (r != cudaSuccess) return r;
  }
  return launch_k(layernorm_f32_kernel, dim3(n), dim3(256), smem, st, y, w, out, res, gather, width, eps, mult, mix);
}

cudaError_t launch_softcap_f32(float* z, size_t n, float cap, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  return launch_k(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, z, n, cap);
}

cudaError_t launch_cast_f32_bf16(const float* in, bf16* out, size_t n, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  return launch_k(cast_f32_bf16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, in, out, n);
}

}  // namespace qie
