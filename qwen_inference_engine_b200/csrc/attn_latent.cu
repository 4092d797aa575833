// attn_latent.cu -- latent (low-rank KV) attention over a paged latent cache (nogatar.h).
//
// A cached position holds ONE row shared by all heads: [latent c (rank) | rotated key part (rot)].  With the
// key up-projection folded into the query (qa_h = [W_uk,h^T q_h | rope(q_rot,h)]) a head's score against position
// j is qa_h . row_j, and the head's output is W_uv,h (sum_j p_j c_j): attention runs in the latent space and the
// cache is never expanded to per-head keys and values.  Options: a sliding window, and a per-head softmax sink
// (one extra term exp(sink_h) in the denominator that carries no value).
//
// One CTA per query row: the row's key window is streamed through shared memory in tiles that all heads share;
// scores, the running maximum / sum and the latent accumulator are fp32.  Prompt portions over a bf16 cache run on
// tensor cores, eight query rows per CTA over key blocks staged once (latent_attention_rows_kernel below).  Options of
// the store and the attention: the pairing of the rotated dimensions, a second normed vector per row (a query latent),
// a sigmoid gate per (row, head) on the result.  Keys are always read from the cache (the row's own position was
// stored by launch_latent_store before), so the result does not depend on how a prompt was cut into forwards or on
// the other rows of the launch.
#include <stdlib.h>

#include <algorithm>

#include "launch.h"
#include "nogatar.h"

namespace qie {
namespace {

template <typename T>
__device__ __forceinline__ float ld_elt(const T* p);
template <>
__device__ __forceinline__ float ld_elt<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_elt<bf16>(const bf16* p) { return bf2f(*p); }
template <typename T>
__device__ __forceinline__ void st_elt(T* p, float v);
template <>
__device__ __forceinline__ void st_elt<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_elt<bf16>(bf16* p, float v) { *p = f2bf(v); }

__device__ __forceinline__ float warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// the output gate of (row, head): sigmoid of the gate's pre-activation, 1 without a gate
__device__ __forceinline__ float head_gate(const HeadGate& g, int r, int h) {
  return g.z ? 1.0f / (1.0f + expf(-(g.z[(size_t)r * g.ld + h] + (g.bias ? bf2f(g.bias[h]) : 0.f)))) : 1.0f;
}
__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename T>
__device__ __forceinline__ T* cache_row(const LatentCache& c, const int* block_table, int max_pages, int slot, int pos) {
  const int page = block_table[(size_t)slot * max_pages + pos / c.page_size];
  return reinterpret_cast<T*>(c.pool) + (size_t)page * c.page_elems + c.layer_off + (size_t)(pos % c.page_size) * (c.rank + c.rot);
}

// one CTA per row; 128 threads
template <typename T>
__global__ void latent_store_kernel(const LatentCache c, const float* __restrict__ dkv, int ld, const bf16* __restrict__ w_norm, float eps,
                                    const RopeTable rope, const int* __restrict__ pos, const int* __restrict__ slot,
                                    const int* __restrict__ block_table, int max_pages, const QueryRope qr, const RowNorm qn) {
  __shared__ float red[4];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, p = pos[r];
  const float* src = dkv + (size_t)r * ld;
  T* dst = cache_row<T>(c, block_table, max_pages, slot[r], p);
  float s = 0.f;
  for (int i = threadIdx.x; i < c.rank; i += blockDim.x) s += src[i] * src[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float rinv = 1.0f / sqrtf(tot / (float)c.rank + eps);
  for (int i = threadIdx.x; i < c.rank; i += blockDim.x) st_elt<T>(dst + i, src[i] * rinv * bf2f(w_norm[i]));
  const int half = rope.dims / 2;
  // the two members of rotated pair i: neighbours, or half the rotated dimensions apart
  const int st1 = rope.half_layout ? 1 : 2, off2 = rope.half_layout ? half : 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float cs = rope.cos_t[(size_t)p * half + i], sn = rope.sin_t[(size_t)p * half + i];
    const float u = src[c.rank + st1 * i], v = src[c.rank + st1 * i + off2];
    st_elt<T>(dst + c.rank + st1 * i, u * cs - v * sn);
    st_elt<T>(dst + c.rank + st1 * i + off2, v * cs + u * sn);
  }
  for (int i = rope.dims + threadIdx.x; i < c.rot; i += blockDim.x) st_elt<T>(dst + c.rank + i, src[c.rank + i]);
  // the same rotation on the rotated part of every query head of the row (saves a launch per layer)
  if (qr.src) {
    for (int i = threadIdx.x; i < qr.heads * half; i += blockDim.x) {
      const int h = i / half, j = i % half;
      const float* qs = qr.src + (size_t)r * qr.ld_src + (size_t)h * qr.hs_src;
      float* qd = qr.dst + (size_t)r * qr.ld_dst + (size_t)h * qr.hs_dst;
      const float cs = rope.cos_t[(size_t)p * half + j], sn = rope.sin_t[(size_t)p * half + j];
      const float u = qs[st1 * j], v = qs[st1 * j + off2];
      qd[st1 * j] = u * cs - v * sn;
      qd[st1 * j + off2] = v * cs + u * sn;
    }
    const int rest = c.rot - rope.dims;
    for (int i = threadIdx.x; i < qr.heads * rest; i += blockDim.x) {
      const int h = i / rest, j = rope.dims + i % rest;
      qr.dst[(size_t)r * qr.ld_dst + (size_t)h * qr.hs_dst + j] = qr.src[(size_t)r * qr.ld_src + (size_t)h * qr.hs_src + j];
    }
  }
  // rider: a second vector of the row normed the same way (the query latent of a model whose queries pass a low-rank bottleneck)
  if (qn.src) {
    __syncthreads();  // red is read above
    float t = 0.f;
    const float* ql = qn.src + (size_t)r * qn.ld_src;
    for (int i = threadIdx.x; i < qn.width; i += blockDim.x) t += ql[i] * ql[i];
    t = warp_sum(t);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = t;
    __syncthreads();
    const float qinv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)qn.width + eps);
    for (int i = threadIdx.x; i < qn.width; i += blockDim.x) {
      const float v = ql[i] * qinv * bf2f(qn.w[i]);
      if (qn.dst) qn.dst[(size_t)r * qn.ld_dst + i] = v;
      if (qn.dst_bf) qn.dst_bf[(size_t)r * qn.ld_dst_bf + i] = f2bf(v);
    }
  }
}

// one CTA per row, threads over (head, element)
__global__ void rope_heads_kernel(const float* __restrict__ src, int ld_src, int hs_src, float* __restrict__ dst, int ld_dst, int hs_dst, int heads,
                                  int rot, const RopeTable rope, const int* __restrict__ pos) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, p = pos[r];
  const int half = rope.dims / 2, rest = rot - rope.dims;
  const int st1 = rope.half_layout ? 1 : 2, off2 = rope.half_layout ? half : 1;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const float* s = src + (size_t)r * ld_src + (size_t)h * hs_src;
    float* d = dst + (size_t)r * ld_dst + (size_t)h * hs_dst;
    const float cs = rope.cos_t[(size_t)p * half + j], sn = rope.sin_t[(size_t)p * half + j];
    const float u = s[st1 * j], v = s[st1 * j + off2];
    d[st1 * j] = u * cs - v * sn;
    d[st1 * j + off2] = v * cs + u * sn;
  }
  for (int i = threadIdx.x; i < heads * rest; i += blockDim.x) {
    const int h = i / rest, j = rope.dims + (i - h * rest);
    dst[(size_t)r * ld_dst + (size_t)h * hs_dst + j] = src[(size_t)r * ld_src + (size_t)h * hs_src + j];
  }
}

// Shared memory (floats), HP = heads of this CTA rounded up to 8:
//   q [D][HP] | acc [HP][rank] | tile [TK][D+1] | p [TK][HP] | m [HP] | l [HP] | alpha [HP]
// q and p are stored head-minor so that the score and the value loops read 8 heads with two 16-byte loads per cached
// element: a thread keeps 8 heads' partial sums in registers (scores: one key x 8 heads, values: one latent
// dimension x 8 heads), which makes both loops arithmetic-bound instead of shared-memory-bound.
template <typename T>
__global__ void __launch_bounds__(256) latent_attention_kernel(const LatentCache c, const float* __restrict__ qa, float* __restrict__ out,
                                                                const bf16* __restrict__ sink, float scale, int window, int H_all, int HG, int TK,
                                                                const int* __restrict__ pos, const int* __restrict__ slot,
                                                                const int* __restrict__ block_table, int max_pages, int n_splits,
                                                                float* __restrict__ ws, const HeadGate hg) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  pdl_wait();
  pdl_trigger();
  const int D = c.rank + c.rot, DP = D + 1, R = c.rank;
  const int h0 = blockIdx.y * HG, H = min(HG, H_all - h0);  // this CTA's heads
  const int HP = (HG + 7) & ~7, HC = HP / 8;
  float* s_q = sm;
  float* s_acc = s_q + (size_t)D * HP;
  float* s_p = s_acc + (size_t)HP * R;
  float* s_m = s_p + (size_t)TK * HP;
  float* s_l = s_m + HP;
  float* s_alpha = s_l + HP;
  float* s_tile = s_alpha + HP;
  const int r = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const int p = pos[r], sl = slot[r];
  int j_lo = window > 0 ? max(0, p - window + 1) : 0, j_hi = p;
  const int split = blockIdx.z;
  if (n_splits > 1) {  // this CTA's share of the keys, in whole tiles; the sink goes with split 0
    const int tiles = (p + 1 - j_lo + TK - 1) / TK, per = (tiles + n_splits - 1) / n_splits;
    j_lo += split * per * TK;
    j_hi = min(p, j_lo + per * TK - 1);
  }
  const bool with_sink = sink && split == 0;
  for (int i = tid; i < HP * D; i += nt) {
    const int d = i / HP, h = i % HP;
    s_q[i] = h < H ? qa[((size_t)r * H_all + h0 + h) * D + d] : 0.f;
  }
  for (int i = tid; i < HP * R; i += nt) s_acc[i] = 0.f;
  for (int i = tid; i < TK * HP; i += nt) s_p[i] = 0.f;
  for (int h = tid; h < HP; h += nt) {
    // the sink enters as a key with score sink_h and no value: running maximum sink_h, running sum exp(0) = 1
    s_m[h] = with_sink && h < H ? bf2f(sink[h0 + h]) : -INFINITY;
    s_l[h] = with_sink && h < H ? 1.f : 0.f;
    s_alpha[h] = 0.f;
  }
  __syncthreads();
  for (int j0 = j_lo; j0 <= j_hi; j0 += TK) {
    const int nk = min(TK, j_hi + 1 - j0);
    for (int jj = tid >> 5; jj < nk; jj += nt >> 5) {  // a warp per cached row: one page lookup, coalesced loads
      const T* row = cache_row<T>(c, block_table, max_pages, sl, j0 + jj);
      for (int d = tid & 31; d < D; d += 32) s_tile[jj * DP + d] = ld_elt<T>(row + d);
    }
    __syncthreads();
    for (int i = tid; i < HC * nk; i += nt) {  // scores of one key against 8 heads
      const int hc = i / nk, jj = i % nk;
      const float* k = s_tile + jj * DP;
      const float4* q4 = reinterpret_cast<const float4*>(s_q) + hc * 2;
      float a[8] = {};
      for (int d = 0; d < D; ++d) {
        const float kv = k[d];
        const float4 qa4 = q4[(size_t)d * (HP / 4)], qb4 = q4[(size_t)d * (HP / 4) + 1];
        a[0] = fmaf(kv, qa4.x, a[0]), a[1] = fmaf(kv, qa4.y, a[1]), a[2] = fmaf(kv, qa4.z, a[2]), a[3] = fmaf(kv, qa4.w, a[3]);
        a[4] = fmaf(kv, qb4.x, a[4]), a[5] = fmaf(kv, qb4.y, a[5]), a[6] = fmaf(kv, qb4.z, a[6]), a[7] = fmaf(kv, qb4.w, a[7]);
      }
      float4* dst = reinterpret_cast<float4*>(s_p + (size_t)jj * HP + hc * 8);
      dst[0] = make_float4(a[0] * scale, a[1] * scale, a[2] * scale, a[3] * scale);
      dst[1] = make_float4(a[4] * scale, a[5] * scale, a[6] * scale, a[7] * scale);
    }
    __syncthreads();
    for (int h = tid >> 5; h < HP; h += nt >> 5) {  // one warp per head; heads beyond H keep probability 0
      const int lane = tid & 31;
      if (h >= H) {
        for (int jj = lane; jj < nk; jj += 32) s_p[jj * HP + h] = 0.f;
        continue;
      }
      float mx = -INFINITY;
      for (int jj = lane; jj < nk; jj += 32) mx = fmaxf(mx, s_p[jj * HP + h]);
      mx = warp_max(mx);
      const float m_old = s_m[h], m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int jj = lane; jj < nk; jj += 32) {
        const float e = expf(s_p[jj * HP + h] - m_new);
        s_p[jj * HP + h] = e;
        sum += e;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float a = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        s_alpha[h] = a;
        s_l[h] = s_l[h] * a + sum;
        s_m[h] = m_new;
      }
    }
    __syncthreads();
    for (int i = tid; i < HC * R; i += nt) {  // one latent dimension for 8 heads
      const int hc = i / R, d = i % R;
      float a[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) a[u] = s_acc[(size_t)(hc * 8 + u) * R + d] * s_alpha[hc * 8 + u];
      const float4* p4 = reinterpret_cast<const float4*>(s_p) + hc * 2;
      for (int jj = 0; jj < nk; ++jj) {
        const float cv = s_tile[jj * DP + d];
        const float4 pa = p4[(size_t)jj * (HP / 4)], pb = p4[(size_t)jj * (HP / 4) + 1];
        a[0] = fmaf(pa.x, cv, a[0]), a[1] = fmaf(pa.y, cv, a[1]), a[2] = fmaf(pa.z, cv, a[2]), a[3] = fmaf(pa.w, cv, a[3]);
        a[4] = fmaf(pb.x, cv, a[4]), a[5] = fmaf(pb.y, cv, a[5]), a[6] = fmaf(pb.z, cv, a[6]), a[7] = fmaf(pb.w, cv, a[7]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) s_acc[(size_t)(hc * 8 + u) * R + d] = a[u];
    }
    __syncthreads();
  }
  if (n_splits <= 1) {
    for (int i = tid; i < H * R; i += nt) out[((size_t)r * H_all + h0) * R + i] = s_acc[i] / s_l[i / R] * head_gate(hg, r, h0 + i / R);
    return;
  }
  // partial result of this split: [acc (R) | running maximum | running sum] per (row, head, split)
  for (int i = tid; i < H * R; i += nt) {
    const int h = i / R;
    ws[(((size_t)r * H_all + h0 + h) * n_splits + split) * (R + 2) + i % R] = s_acc[i];
  }
  for (int h = tid; h < H; h += nt) {
    float* w = ws + (((size_t)r * H_all + h0 + h) * n_splits + split) * (R + 2) + R;
    w[0] = s_m[h];
    w[1] = s_l[h];
  }
}

// grid (rows, heads): out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M), splits in ascending order
__global__ void latent_attention_combine_kernel(const float* __restrict__ ws, float* __restrict__ out, int H, int R, int n_splits, const HeadGate hg) {
  pdl_wait();
  pdl_trigger();
  const float* w = ws + ((size_t)blockIdx.x * H + blockIdx.y) * n_splits * (R + 2);
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, w[(size_t)s * (R + 2) + R]);
  float den = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = w[(size_t)s * (R + 2) + R];
    if (ms != -INFINITY) den += w[(size_t)s * (R + 2) + R + 1] * expf(ms - M);
  }
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = w[(size_t)s * (R + 2) + R];
      if (ms != -INFINITY) a = fmaf(w[(size_t)s * (R + 2) + d], expf(ms - M), a);
    }
    out[((size_t)blockIdx.x * H + blockIdx.y) * R + d] = a / den * head_gate(hg, blockIdx.x, blockIdx.y);
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Tensor-core version for bf16 caches and many rows (prompts).  All heads of a row share the cached rows, so the
// HEADS are the M dimension of the MMA: S [16 heads, 64 keys] = Q [16, D] K^T and O [16 heads, rank] += P [16, 64] C,
// mma.sync m16n8k16 with fp32 accumulators.  One CTA per (row, group of <= 16 heads), 8 warps: warp w owns keys
// 8w .. 8w+7 of a tile for the scores and the latent columns 8 (w + 8 i), i < NBW, for the values (accumulators in
// registers across tiles, rescaled like the fp32 kernel).  Softmax state and scores are fp32; the probabilities enter
// the second product as bf16.  Shared memory: q bf16 [16][D+8] | tile bf16 [64][D+8] | scores fp32 [16][65] |
// probabilities bf16 [16][72] | m, l, alpha [16].
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

constexpr int ATK = 64;  // keys per tile

template <int NBW>
__global__ void __launch_bounds__(256) latent_attention_mma_kernel(const LatentCache c, const float* __restrict__ qa, float* __restrict__ out,
                                                                    const bf16* __restrict__ sink, float scale, int window, int H_all,
                                                                    const int* __restrict__ pos, const int* __restrict__ slot,
                                                                    const int* __restrict__ block_table, int max_pages, const HeadGate hg) {
  extern __shared__ uint4 smq[];
  pdl_wait();
  pdl_trigger();
  const int D = c.rank + c.rot, DP = D + 8, R = c.rank, D16 = (D + 15) & ~15;
  const int h0 = blockIdx.y * 16, H = min(16, H_all - h0);
  bf16* s_q = reinterpret_cast<bf16*>(smq);
  bf16* s_tile = s_q + 16 * DP;
  float* s_s = reinterpret_cast<float*>(s_tile + ATK * DP);
  bf16* s_pb = reinterpret_cast<bf16*>(s_s + 16 * 65);
  float* s_m = reinterpret_cast<float*>(s_pb + 16 * 72);
  float* s_l = s_m + 16;
  float* s_alpha = s_l + 16;
  const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int p = pos[r], sl = slot[r];
  const int j_lo = window > 0 ? max(0, p - window + 1) : 0;
  for (int i = tid; i < 16 * DP; i += 256) {
    const int h = i / DP, d = i % DP;
    s_q[i] = f2bf(h < H && d < D ? qa[((size_t)r * H_all + h0 + h) * D + d] : 0.f);
  }
  if (tid < 16) {
    const bool ws = sink && tid < H;
    s_m[tid] = ws ? bf2f(sink[h0 + tid]) : -INFINITY;
    s_l[tid] = ws ? 1.f : 0.f;
    s_alpha[tid] = 0.f;
  }
  float o[NBW][4];
#pragma unroll
  for (int i = 0; i < NBW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int chunks = DP / 8;  // 16-byte pieces of a padded row; the last one is the zero padding
  __syncthreads();
  for (int j0 = j_lo; j0 <= p; j0 += ATK) {
    const int nk = min(ATK, p + 1 - j0);
    for (int jj = warp; jj < ATK; jj += 8) {  // a warp per cached row, 16-byte copies; rows past the window's end are zeros
      uint4* dst = reinterpret_cast<uint4*>(s_tile + jj * DP);
      if (jj < nk) {
        const uint4* row = reinterpret_cast<const uint4*>(cache_row<bf16>(c, block_table, max_pages, sl, j0 + jj));
        for (int ch = lane; ch < chunks; ch += 32) dst[ch] = ch < D / 8 ? row[ch] : make_uint4(0, 0, 0, 0);
      } else {
        for (int ch = lane; ch < chunks; ch += 32) dst[ch] = make_uint4(0, 0, 0, 0);
      }
    }
    __syncthreads();
    {  // scores of keys 8 warp .. 8 warp + 7 against the 16 heads
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
      const bf16* krow = s_tile + (warp * 8 + gq) * DP;
      for (int ks = 0; ks < D16; ks += 16) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(s_q + gq * DP + ks + 2 * tq);
        a[1] = *reinterpret_cast<const uint32_t*>(s_q + (gq + 8) * DP + ks + 2 * tq);
        a[2] = *reinterpret_cast<const uint32_t*>(s_q + gq * DP + ks + 2 * tq + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(s_q + (gq + 8) * DP + ks + 2 * tq + 8);
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks + 2 * tq);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks + 2 * tq + 8);
        mma_16816(sc, a, b0, b1);
      }
      const int col = warp * 8 + 2 * tq;
      s_s[gq * 65 + col] = sc[0] * scale;
      s_s[gq * 65 + col + 1] = sc[1] * scale;
      s_s[(gq + 8) * 65 + col] = sc[2] * scale;
      s_s[(gq + 8) * 65 + col + 1] = sc[3] * scale;
    }
    __syncthreads();
    for (int h = warp; h < 16; h += 8) {  // online softmax, one warp per head
      float mx = -INFINITY;
      for (int jj = lane; jj < nk; jj += 32) mx = fmaxf(mx, s_s[h * 65 + jj]);
      mx = warp_max(mx);
      const float m_old = s_m[h], m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int jj = lane; jj < ATK; jj += 32) {
        const float e = jj < nk && h < H ? expf(s_s[h * 65 + jj] - m_new) : 0.f;
        s_pb[h * 72 + jj] = f2bf(e);
        sum += e;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float a = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        s_alpha[h] = a;
        s_l[h] = s_l[h] * a + sum;
        s_m[h] = m_new;
      }
    }
    __syncthreads();
    {  // O = O * alpha + P C for this warp's latent columns
      const float a_lo = s_alpha[gq], a_hi = s_alpha[gq + 8];
#pragma unroll
      for (int i = 0; i < NBW; ++i) o[i][0] *= a_lo, o[i][1] *= a_lo, o[i][2] *= a_hi, o[i][3] *= a_hi;
#pragma unroll
      for (int kk = 0; kk < ATK; kk += 16) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(s_pb + gq * 72 + kk + 2 * tq);
        a[1] = *reinterpret_cast<const uint32_t*>(s_pb + (gq + 8) * 72 + kk + 2 * tq);
        a[2] = *reinterpret_cast<const uint32_t*>(s_pb + gq * 72 + kk + 2 * tq + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(s_pb + (gq + 8) * 72 + kk + 2 * tq + 8);
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
          const int nb = warp + 8 * i;
          if (nb * 8 < R) {  // warp-uniform
            uint32_t b0, b1;
            ldmatrix_x2_trans(b0, b1, smem_u32(s_tile + (kk + (lane & 15)) * DP + nb * 8));
            mma_16816(o[i], a, b0, b1);
          }
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < NBW; ++i) {
    const int d = (warp + 8 * i) * 8 + 2 * tq;
    if (d < R) {
      if (gq < H) {
        const float inv = head_gate(hg, r, h0 + gq) / s_l[gq];
        float* dst = out + ((size_t)r * H_all + h0 + gq) * R + d;
        dst[0] = o[i][0] * inv, dst[1] = o[i][1] * inv;
      }
      if (gq + 8 < H) {
        const float inv = head_gate(hg, r, h0 + gq + 8) / s_l[gq + 8];
        float* dst = out + ((size_t)r * H_all + h0 + gq + 8) * R + d;
        dst[0] = o[i][2] * inv, dst[1] = o[i][3] * inv;
      }
    }
  }
}

template <int NBW>
cudaError_t launch_attn_mma(const LatentCache& c, const float* qa, float* out, const bf16* sink, float scale, int window, int heads, const int* pos,
                            const int* slot, const int* block_table, int max_pages, int n, cudaStream_t st, const HeadGate& hg) {
  const int DP = c.rank + c.rot + 8;
  const size_t smem = (size_t)(16 + ATK) * DP * sizeof(bf16) + 16 * 65 * sizeof(float) + 16 * 72 * sizeof(bf16) + 48 * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
  if (smem > 48 * 1024) {
    cudaError_t r = cudaFuncSetAttribute(latent_attention_mma_kernel<NBW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (r != cudaSuccess) return r;
  }
  return launch_k(latent_attention_mma_kernel<NBW>, dim3(n, (heads + 15) / 16), dim3(256), smem, st, c, qa, out, sink, scale, window, heads, pos, slot,
                  block_table, max_pages, hg);
}

// ---------------------------------------------------------------------------------------------------------------
// Prompt portions over a bf16 cache, several query rows per CTA.  Consecutive rows of a prompt see almost the same keys,
// so a CTA takes RT = 8 / WPR consecutive rows and stages every block of TK cached rows ONCE for all of them (double
// buffered with cp.async).  A warp owns one query row: its 16 heads are the M dimension, S [16 heads, TK keys] = Q K^T stays
// in registers through mask, online softmax and the re-packing as the A operand of O [16 heads, rank] += P C (the cached
// row's first `rank` columns, read transposed from the same staged block).  A latent too wide for one warp's registers is
// split over WPR warps: each computes the row's scores itself and accumulates its own NBO * 8 columns of O.  Rows of
// another sequence in the same CTA (a batch of short portions) are served in further passes over their own keys.
// Shared memory: Q bf16 [RT][16][DP] | K blocks bf16 [2][TK][DP] | cache row pointers [2][TK]; DP = D padded so that
// rows are an odd number of 16-byte pieces apart (ldmatrix without bank conflicts), the padding zero.
template <int NBO, int TK>
__global__ void __launch_bounds__(256) latent_attention_rows_kernel(const LatentCache c, const float* __restrict__ qa, float* __restrict__ out,
                                                                     const bf16* __restrict__ sink, float scale, int window, int H_all,
                                                                     const int* __restrict__ pos, const int* __restrict__ slot,
                                                                     const int* __restrict__ block_table, int max_pages, int n, int DP, int WPR,
                                                                     const HeadGate hg) {
  extern __shared__ uint4 smq[];
  __shared__ int s_slot[8], s_pos[8], s_done[8], s_pass[3];  // per row of the CTA; the pass: slot, first key, last key
  pdl_wait();
  pdl_trigger();
  const int D = c.rank + c.rot, R = c.rank, D16 = (D + 15) & ~15, RT = 8 / WPR;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int rl = warp / WPR, part = warp % WPR;  // the warp's row of the CTA and its share of the latent's columns
  // late rows first: under a causal mask they see the most keys, and the short early rows fill the SMs that finish first
  const int bx = gridDim.x - 1 - blockIdx.x;
  const int r = bx * RT + rl;
  const bool valid = r < n;
  const int h0 = blockIdx.y * 16, H = min(16, H_all - h0);
  bf16* s_q = reinterpret_cast<bf16*>(smq);
  bf16* s_k = s_q + (size_t)RT * 16 * DP;
  const bf16** krow = reinterpret_cast<const bf16**>(s_k + (size_t)2 * TK * DP);
  for (int i = tid; i < RT * 16 * DP; i += 256) {
    const int rr = i / (16 * DP), h = (i / DP) % 16, d = i % DP, row = bx * RT + rr;
    s_q[i] = f2bf(row < n && h < H && d < D ? qa[((size_t)row * H_all + h0 + h) * D + d] : 0.f);
  }
  for (int i = tid; i < 2 * TK * (DP - D); i += 256) s_k[(size_t)(i / (DP - D)) * DP + D + i % (DP - D)] = f2bf(0.f);  // the padding columns
  if (tid < 8) {
    const int row = bx * RT + tid;
    const bool ok = tid < RT && row < n;
    s_slot[tid] = ok ? slot[row] : -1, s_pos[tid] = ok ? pos[row] : 0, s_done[tid] = ok ? 0 : 1;
  }
  const int p = valid ? pos[r] : 0, sl = valid ? slot[r] : -1;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int chunks = D / 8;
  while (true) {
    __syncthreads();
    if (tid == 0) {  // the next pass: the first unserved row's sequence and the key range of all its rows here
      int ps = -1, j0 = 0, j1 = 0;
      for (int i = 0; i < RT; ++i) {
        if (s_done[i] || (ps >= 0 && s_slot[i] != ps)) continue;
        const int l = window > 0 ? max(0, s_pos[i] - window + 1) : 0;
        if (ps < 0) ps = s_slot[i], j0 = l, j1 = s_pos[i];
        else j0 = min(j0, l), j1 = max(j1, s_pos[i]);
      }
      s_pass[0] = ps, s_pass[1] = j0, s_pass[2] = j1;
    }
    __syncthreads();
    const int ps = s_pass[0], jmin = s_pass[1] / TK * TK, jmax = s_pass[2];
    if (ps < 0) break;
    const bool active = valid && sl == ps && !s_done[rl];
    float o[NBO][4];
#pragma unroll
    for (int i = 0; i < NBO; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    // running maximum and (per thread partial) sum of the warp's head rows gq and gq + 8; the sink enters as a key without a value
    const bool sk0 = sink && gq < H, sk1 = sink && gq + 8 < H;
    float m0 = sk0 ? bf2f(sink[h0 + gq]) : -INFINITY, m1 = sk1 ? bf2f(sink[h0 + gq + 8]) : -INFINITY;
    float l0 = sk0 && tq == 0 ? 1.f : 0.f, l1 = sk1 && tq == 0 ? 1.f : 0.f;
    auto stage = [&](int jb, int buf) {
      if (tid < TK) krow[buf * TK + tid] = jb + tid <= jmax ? cache_row<bf16>(c, block_table, max_pages, ps, jb + tid) : nullptr;
      __syncthreads();
      for (int i = tid; i < TK * chunks; i += 256) {
        const int key = i / chunks, ch = i - key * chunks;
        bf16* dst = s_k + ((size_t)buf * TK + key) * DP + ch * 8;
        const bf16* row = krow[buf * TK + key];
        if (row) cp_async16(smem_u32(dst), row + ch * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
      }
      cp_async_commit();
    };
    int j0 = jmin, buf = 0;
    stage(j0, 0);
    while (true) {
      const int jn = j0 + TK;
      const bool more = jn <= jmax;
      if (more) {
        stage(jn, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (active && j0 <= p && j0 + TK - 1 >= lo) {  // warp-uniform: the block holds keys this row sees
        const bf16* kt = s_k + (size_t)buf * TK * DP;
        const bf16* qt = s_q + (size_t)rl * 16 * DP;
        float s[TK / 8][4];
#pragma unroll
        for (int nb = 0; nb < TK / 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
        for (int ks = 0; ks < D16; ks += 16) {
          uint32_t a[4];
          ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(qt + (size_t)(lane & 15) * DP + ks + (lane >> 4) * 8));
#pragma unroll
          for (int nb = 0; nb < TK / 8; ++nb) {
            uint32_t b0, b1;
            ldmatrix_x2(b0, b1, smem_u32(kt + (size_t)(nb * 8 + (lane & 7)) * DP + ks + ((lane >> 3) & 1) * 8));
            mma_16816(s[nb], a, b0, b1);
          }
        }
        const bool whole = j0 >= lo && j0 + TK - 1 <= p;  // every key of the block is visible: no mask
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < TK / 8; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = j0 + nb * 8 + 2 * tq + (e & 1);
            s[nb][e] = (whole || (j <= p && j >= lo)) ? s[nb][e] * scale : -INFINITY;
            if (e >> 1) mx1 = fmaxf(mx1, s[nb][e]);
            else mx0 = fmaxf(mx0, s[nb][e]);
          }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // the weights become bf16 operands below: the fast exponential's error is far under their rounding
        const float c0 = m0 > -INFINITY ? __expf(m0 - mn0) : 1.f, c1 = m1 > -INFINITY ? __expf(m1 - mn1) : 1.f;
        m0 = mn0, m1 = mn1;
        l0 *= c0, l1 *= c1;
#pragma unroll
        for (int i = 0; i < NBO; ++i) o[i][0] *= c0, o[i][1] *= c0, o[i][2] *= c1, o[i][3] *= c1;
#pragma unroll
        for (int nb = 0; nb < TK / 8; ++nb) {
          s[nb][0] = __expf(s[nb][0] - mn0), s[nb][1] = __expf(s[nb][1] - mn0);  // the block has a visible key, so mn is finite
          s[nb][2] = __expf(s[nb][2] - mn1), s[nb][3] = __expf(s[nb][3] - mn1);
          l0 += s[nb][0] + s[nb][1];
          l1 += s[nb][2] + s[nb][3];
        }
#pragma unroll
        for (int kb = 0; kb < TK / 16; ++kb) {
          uint32_t pa[4];
          pa[0] = pack2(f2bf(s[2 * kb][0]), f2bf(s[2 * kb][1]));
          pa[1] = pack2(f2bf(s[2 * kb][2]), f2bf(s[2 * kb][3]));
          pa[2] = pack2(f2bf(s[2 * kb + 1][0]), f2bf(s[2 * kb + 1][1]));
          pa[3] = pack2(f2bf(s[2 * kb + 1][2]), f2bf(s[2 * kb + 1][3]));
#pragma unroll
          for (int i = 0; i < NBO; ++i) {
            const int nb = part * NBO + i;
            if (nb * 8 < R) {  // warp-uniform
              uint32_t b0, b1;
              ldmatrix_x2_trans(b0, b1, smem_u32(kt + (size_t)(kb * 16 + (lane & 15)) * DP + nb * 8));
              mma_16816(o[i], pa, b0, b1);
            }
          }
        }
      }
      __syncthreads();  // the stage is free for the block after the next
      if (!more) break;
      j0 = jn;
      buf ^= 1;
    }
    if (active) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
      l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
      const float f0 = gq < H ? head_gate(hg, r, h0 + gq) / l0 : 0.f, f1 = gq + 8 < H ? head_gate(hg, r, h0 + gq + 8) / l1 : 0.f;
#pragma unroll
      for (int i = 0; i < NBO; ++i) {
        const int d = (part * NBO + i) * 8 + 2 * tq;
        if (d < R) {
          if (gq < H) {
            float* dst = out + ((size_t)r * H_all + h0 + gq) * R + d;
            dst[0] = o[i][0] * f0, dst[1] = o[i][1] * f0;
          }
          if (gq + 8 < H) {
            float* dst = out + ((size_t)r * H_all + h0 + gq + 8) * R + d;
            dst[0] = o[i][2] * f1, dst[1] = o[i][3] * f1;
          }
        }
      }
    }
    __syncthreads();  // every warp has read s_done of this pass
    if (active && part == 0 && lane == 0) s_done[rl] = 1;
  }
}

// padded row length of the staged blocks: at least 8 more than D (the k-steps of 16 may reach past D), an odd number of 16-byte pieces
inline int rows_kernel_dp(int D) {
  int dp = D + 8;
  if ((dp / 8) % 2 == 0) dp += 8;
  return dp;
}
inline size_t rows_kernel_smem(int D, int RT, int TK) {
  return ((size_t)RT * 16 + 2 * (size_t)TK) * rows_kernel_dp(D) * sizeof(bf16) + (size_t)2 * TK * sizeof(void*);
}

template <int NBO, int TK>
cudaError_t launch_attn_rows(const LatentCache& c, const float* qa, float* out, const bf16* sink, float scale, int window, int heads, const int* pos,
                             const int* slot, const int* block_table, int max_pages, int n, int WPR, cudaStream_t st, const HeadGate& hg) {
  const int D = c.rank + c.rot, RT = 8 / WPR;
  const size_t smem = rows_kernel_smem(D, RT, TK);
  cudaError_t r = cudaFuncSetAttribute(latent_attention_rows_kernel<NBO, TK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (r != cudaSuccess) return r;
  return launch_k(latent_attention_rows_kernel<NBO, TK>, dim3((n + RT - 1) / RT, (heads + 15) / 16), dim3(256), smem, st, c, qa, out, sink, scale, window,
                  heads, pos, slot, block_table, max_pages, n, rows_kernel_dp(D), WPR, hg);
}

size_t attn_smem_floats(int H, int D, int R, int TK) {
  const size_t HP = (size_t)((H + 7) & ~7);
  return HP * D + HP * R + (size_t)TK * (D + 1) + (size_t)TK * HP + 3 * HP;
}

}  // namespace

cudaError_t launch_latent_store(const LatentCache& c, const float* dkv, int ld, const bf16* w_norm, float eps, const RopeTable& rope,
                                const int* pos, const int* slot, const int* block_table, int max_pages, int n, cudaStream_t st,
                                const QueryRope& qr, const RowNorm& qn) {
  if (n <= 0) return cudaSuccess;
  if (c.elt_bytes == 4)
    return launch_k(latent_store_kernel<float>, dim3(n), dim3(128), 0, st, c, dkv, ld, w_norm, eps, rope, pos, slot, block_table, max_pages, qr, qn);
  return launch_k(latent_store_kernel<bf16>, dim3(n), dim3(128), 0, st, c, dkv, ld, w_norm, eps, rope, pos, slot, block_table, max_pages, qr, qn);
}

cudaError_t launch_rope_heads_f32(const float* src, int ld_src, int hs_src, float* dst, int ld_dst, int hs_dst, int heads, int rot,
                                  const RopeTable& rope, const int* pos, int n, cudaStream_t st) {
  if (n <= 0 || heads <= 0) return cudaSuccess;
  return launch_k(rope_heads_kernel, dim3(n), dim3(128), 0, st, src, ld_src, hs_src, dst, ld_dst, hs_dst, heads, rot, rope, pos);
}

cudaError_t launch_latent_attention(const LatentCache& c, const float* qa, float* out, const bf16* sink, float scale, int window, int heads,
                                    const int* pos, const int* slot, const int* block_table, int max_pages, int n, int max_keys, float* ws,
                                    size_t ws_floats, cudaStream_t st, const HeadGate& hg) {
  if (n <= 0) return cudaSuccess;
  const int D = c.rank + c.rot;
  // bf16 cache rows and a prompt's worth of rows: tensor cores (QIE_ATTN_MMA=0 keeps the fp32 kernel)
  static const bool mma_on = [] { const char* v = getenv("QIE_ATTN_MMA"); return !(v && v[0] == '0'); }();
  if (mma_on && c.elt_bytes == 2 && n >= 64 && c.rank % 8 == 0 && c.rot % 8 == 0 && c.rank <= 512 && c.page_elems % 8 == 0 &&
      c.layer_off % 8 == 0 && (reinterpret_cast<uintptr_t>(c.pool) & 15) == 0) {
    // several rows per CTA over shared key blocks (QIE_LATENT_ROWS=0 keeps the one-row kernel for A/B): the fewest warps per
    // row whose accumulators hold the latent (32 blocks of 8 columns each at most) and whose shared memory fits
    static const bool rows_on = [] { const char* v = getenv("QIE_LATENT_ROWS"); return !(v && v[0] == '0'); }();
    if (rows_on) {
      const int nb = (c.rank + 7) / 8;
      for (int tk : {64, 32}) {
        int wpr = 1;
        while (wpr < 8 && (nb > 32 * wpr || rows_kernel_smem(D, 8 / wpr, tk) > 200 * 1024)) wpr *= 2;
        if (nb > 32 * wpr || rows_kernel_smem(D, 8 / wpr, tk) > 200 * 1024 || (tk == 64 && wpr > 2)) continue;
        const int nbo = (nb + wpr - 1) / wpr;
#define ROWS_GO(NBO, TK) launch_attn_rows<NBO, TK>(c, qa, out, sink, scale, window, heads, pos, slot, block_table, max_pages, n, wpr, st, hg)
        if (tk == 64) return nbo <= 4 ? ROWS_GO(4, 64) : nbo <= 8 ? ROWS_GO(8, 64) : nbo <= 16 ? ROWS_GO(16, 64) : ROWS_GO(32, 64);
        return nbo <= 8 ? ROWS_GO(8, 32) : nbo <= 16 ? ROWS_GO(16, 32) : ROWS_GO(32, 32);
#undef ROWS_GO
      }
    }
    cudaError_t r = cudaErrorInvalidConfiguration;
    if (c.rank <= 64) r = launch_attn_mma<1>(c, qa, out, sink, scale, window, heads, pos, slot, block_table, max_pages, n, st, hg);
    else if (c.rank <= 128) r = launch_attn_mma<2>(c, qa, out, sink, scale, window, heads, pos, slot, block_table, max_pages, n, st, hg);
    else if (c.rank <= 256) r = launch_attn_mma<4>(c, qa, out, sink, scale, window, heads, pos, slot, block_table, max_pages, n, st, hg);
    else r = launch_attn_mma<8>(c, qa, out, sink, scale, window, heads, pos, slot, block_table, max_pages, n, st, hg);
    if (r != cudaErrorInvalidConfiguration) return r;  // too large for its shared memory: the fp32 kernel below
  }
  // all heads of a row share the key tiles, so one CTA per row reads them once; with few rows the heads are dealt to
  // more CTAs (each reads the tiles again, from L2) until the GPU has a CTA per SM or so
  int HG = heads;
  while (HG > 8 && (long)n * ((heads + HG - 1) / HG) < 128) HG = (HG + 1) / 2;  // the kernel works on heads in eights
  // many or wide heads: the q / accumulator part of a CTA must leave room for a key tile
  while (HG > 8 && attn_smem_floats(HG, D, c.rank, 8) > 200 * 1024 / sizeof(float)) HG = (HG + 1) / 2;
  int TK = 128;
  if (window > 0)
    while (TK > 8 && TK / 2 >= window) TK /= 2;
  // key tile: as large as fits; with many rows a tile of >= 32 keys that lets two CTAs share an SM is better (the
  // loops wait on shared-memory and cache latency, which more resident warps hide) -- measured 5.1 -> 3.6 ms on the
  // width-1024 comparison model; where the per-CTA q / accumulator part is too large for that, one CTA per SM
  while (TK > 1 && attn_smem_floats(HG, D, c.rank, TK) > 200 * 1024 / sizeof(float)) TK /= 2;
  if (n >= 256) {
    int t2 = TK;
    while (t2 > 32 && attn_smem_floats(HG, D, c.rank, t2) > 110 * 1024 / sizeof(float)) t2 /= 2;
    if (attn_smem_floats(HG, D, c.rank, t2) <= 110 * 1024 / sizeof(float)) TK = t2;
  }
  const size_t smem = attn_smem_floats(HG, D, c.rank, TK) * sizeof(float);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  // few rows and many keys: the key tiles are dealt to several CTAs per (row, head group), then combined
  const int keys = window > 0 ? std::min(window, max_keys) : max_keys;
  const int tiles = (keys + TK - 1) / TK;
  int n_splits = 1;
  if (ws) {
    const long ctas = (long)n * ((heads + HG - 1) / HG);
    while (n_splits < 32 && n_splits < tiles && ctas * n_splits < 256) n_splits *= 2;
    n_splits = std::min(n_splits, tiles);
    if ((size_t)n * heads * n_splits * (c.rank + 2) > ws_floats) n_splits = 1;
  }
  const dim3 grid(n, (heads + HG - 1) / HG, n_splits);
  cudaError_t r;
  if (c.elt_bytes == 4) {
    if (smem > 48 * 1024 && (r = cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess)
      return r;
    r = launch_k(latent_attention_kernel<float>, grid, dim3(256), smem, st, c, qa, out, sink, scale, window, heads, HG, TK, pos, slot, block_table,
                    max_pages, n_splits, ws, hg);
    if (r == cudaSuccess && n_splits > 1) r = launch_k(latent_attention_combine_kernel, dim3(n, heads), dim3(128), 0, st, (const float*)ws, out, heads, c.rank, n_splits, hg);
    return r;
  }
  if (smem > 48 * 1024 && (r = cudaFuncSetAttribute(latent_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess)
    return r;
  r = launch_k(latent_attention_kernel<bf16>, grid, dim3(256), smem, st, c, qa, out, sink, scale, window, heads, HG, TK, pos, slot, block_table,
               max_pages, n_splits, ws, hg);
  if (r == cudaSuccess && n_splits > 1) r = launch_k(latent_attention_combine_kernel, dim3(n, heads), dim3(128), 0, st, (const float*)ws, out, heads, c.rank, n_splits, hg);
  return r;
}

}  // namespace qie
