// attn_gqa.cu -- grouped-query attention over paged key/value rows for the fp32-stream families (fosavik.h): the
// store of new rows (optional per-head unit norm of queries and keys), and an attention whose mask, sink, number of
// score maps and finishing step are arguments: causal or sliding window with kept first tokens, a unit sink in the
// denominator, one or two softmax maps over shared values, and as the last step nothing, a sigmoid gate per head, or
// the differential combination with a unit norm per head.  Softmax and accumulation are fp32; the cache rows are fp32
// or bf16.  Keys are ALWAYS read from the cache (a row's own position is stored first), so a result does not depend
// on how a prompt was cut or what else is in the batch.
#include <stdlib.h>

#include <algorithm>

#include "fosavik.h"
#include "launch.h"

namespace qie {
namespace {

constexpr int ATK = 32;       // keys per tile
constexpr int ATHREADS = 128;
constexpr int AMAXACC = 16;   // accumulators per thread: query vectors x value columns of a CTA <= 2048

__device__ __forceinline__ const char* kv_row_ptr(const KvRowCache& c, const int* block_table, int max_pages, int slot, int pos) {
  const int page = block_table[(size_t)slot * max_pages + pos / c.page_size];
  const size_t off = (size_t)page * c.page_elems + c.layer_off + (size_t)(pos % c.page_size) * (c.kw + c.vw);
  return static_cast<const char*>(c.pool) + off * c.elt_bytes;
}

__device__ __forceinline__ void store_elt(const KvRowCache& c, char* row, int i, float v) {
  if (c.elt_bytes == 4) reinterpret_cast<float*>(row)[i] = v;
  else reinterpret_cast<bf16*>(row)[i] = f2bf(v);
}

// the mixed queries of row r; thread = (head h, kv head c, element e).  smem: q row (bias added) [heads * dim] | talk [heads * heads]
__device__ __forceinline__ void talk_queries_row(const TalkQueries& t, int r, float* smem) {
  const int heads = t.heads, dim = t.dim, hpg = heads / t.kv_heads, kd = t.kv_heads * dim;
  float* qs = smem;
  float* tk = smem + heads * dim;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) qs[i] = t.q[(size_t)r * t.ldq + i] + (t.q_bias ? bf2f(t.q_bias[i]) : 0.f);
  for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) tk[i] = bf2f(t.talk[i]);
  __syncthreads();
  for (int i = threadIdx.x; i < heads * kd; i += blockDim.x) {
    const int h = i / kd, c = (i - h * kd) / dim, e = i - h * kd - c * dim;
    float v = 0.f;
    for (int g = c * hpg; g < (c + 1) * hpg; ++g) v = fmaf(tk[h * heads + g], qs[g * dim + e], v);
    t.qt[(size_t)r * t.ldqt + i] = v;
  }
}

// One group of d consecutive elements, by one warp: unit RMS norm times w (w null: as it is), then the rotation of the
// first rope.dims elements by position p.  get(i) reads element i (bias added), put(i, x) writes it; every element is read
// before the warp's reduction and written after it, by the lane that read it (or its pair), so put may overwrite get's source.
template <typename Get, typename Put>
__device__ __forceinline__ void norm_rope_group(const KvStoreArgs& a, int p, int lane, int d, Get get, const bf16* w, Put put) {
  float rstd = 1.f;
  if (w) {
    float s = 0.f;
    for (int i = lane; i < d; i += 32) s = fmaf(get(i), get(i), s);
    rstd = 1.0f / sqrtf(warp_sum(s) / (float)d + a.eps);
  }
  auto val = [&](int i) { return w ? get(i) * rstd * bf2f(w[i]) : get(i); };
  const int dims = a.rope.dims, half = dims / 2;
  const int st1 = a.rope.half_layout ? 1 : 2, off2 = a.rope.half_layout ? half : 1;
  for (int i = lane; i < half; i += 32) {
    const float cs = a.rope.cos_t[(size_t)p * half + i], sn = a.rope.sin_t[(size_t)p * half + i];
    const float u = val(st1 * i), v = val(st1 * i + off2);
    put(st1 * i, u * cs - v * sn);
    put(st1 * i + off2, v * cs + u * sn);
  }
  for (int i = dims + lane; i < d; i += 32) put(i, val(i));
}

// one CTA per row, one warp per normed group
__global__ void __launch_bounds__(128) kv_store_rows_kernel(const KvStoreArgs a) {
  extern __shared__ float tq_smem[];  // only with the query rider
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  if (a.tq.talk) talk_queries_row(a.tq, r, tq_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (a.c.pool && a.k) {
    char* row = const_cast<char*>(kv_row_ptr(a.c, a.block_table, a.max_pages, a.slot[r], a.pos[r]));
    const float* k = a.k + (size_t)r * a.ldk;
    auto key = [&](int i) { return a.k_bias ? k[i] + bf2f(a.k_bias[i]) : k[i]; };
    if (a.k_norm || a.rope.dims > 0) {
      const int d = a.norm_dim;
      for (int g = warp; g < a.c.kw / d; g += nw) norm_rope_group(a, a.pos[r], lane, d, [&](int i) { return key(g * d + i); }, a.k_norm,
                                                                  [&](int i, float x) { store_elt(a.c, row, g * d + i, x); });
    } else {
      for (int i = threadIdx.x; i < a.c.kw; i += blockDim.x) store_elt(a.c, row, i, key(i));
    }
    const float* v = a.v + (size_t)r * a.ldv;
    const bool blend = a.v_lam && a.v_other;
    const float lam = blend ? bf2f(*a.v_lam) : 0.f;
    for (int i = threadIdx.x; i < a.c.vw; i += blockDim.x) {
      float x = a.v_bias ? v[i] + bf2f(a.v_bias[i]) : v[i];
      if (blend) x = (1.0f - lam) * x + lam * a.v_other[(size_t)r * a.ld_vo + i];
      if (a.v_keep) a.v_keep[(size_t)r * a.ld_vk + i] = x;
      store_elt(a.c, row, a.c.kw + i, x);
    }
  }
  if (a.q && (a.q_norm || a.rope.dims > 0 || a.q_bias)) {
    float* q = a.q + (size_t)r * a.ldq;
    const int d = a.norm_dim;
    for (int h = warp; h < a.q_heads; h += nw)
      norm_rope_group(a, a.pos[r], lane, d, [&](int i) { return a.q_bias ? q[h * d + i] + bf2f(a.q_bias[h * d + i]) : q[h * d + i]; }, a.q_norm,
                      [&](int i, float x) { q[h * d + i] = x; });
  }
}

// CTA (row, kv head x head chunk, key split).  Shared memory: q [QV][dim] (scaled) | K tile [ATK][kd + 1] | V tile
// [ATK][vd] | scores [QV][ATK] | corr [QV] | m [QV] | l [QV], QV = hpc * maps query vectors, kd = maps * dim.
__global__ void __launch_bounds__(ATHREADS) gqa_attention_kernel(const GqaAttnArgs a, int hpc, int chunks, int n_splits) {
  extern __shared__ float sm[];
  __shared__ const char* rowp[ATK];
  __shared__ int dist[ATK];  // pos - j of the tile's keys
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, split = blockIdx.z;
  const int g = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int hpg = a.heads / a.kv_heads;
  const int h0 = g * hpg + chunk * hpc;                 // first head of this CTA
  const int nh = min(hpc, hpg - chunk * hpc);           // heads of this CTA
  const int maps = a.maps, dim = a.dim, vd = a.vdim, kd = maps * dim;
  const int QV = nh * maps;
  float* qs = sm;
  float* Kt = qs + hpc * maps * dim;
  float* Vt = Kt + ATK * (kd + 1);
  float* sc = Vt + ATK * vd;
  float* corr = sc + hpc * maps * ATK;
  float* mrun = corr + hpc * maps;
  float* lrun = mrun + hpc * maps;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = a.pos[r], slot = a.slot[r];
  // visible keys as one virtual range: the kept first tokens below the window, then the window
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int nfirst = a.window > 0 ? min(a.keep_first, lo) : 0;
  const int nkeys = nfirst + (pos - lo + 1);
  int per = (nkeys + n_splits - 1) / n_splits;
  per = (per + ATK - 1) / ATK * ATK;
  const int i0 = split * per, i1 = min(nkeys, i0 + per);
  {
    const float* q = a.q + (size_t)r * a.ldq + (size_t)h0 * kd;
    for (int i = tid; i < QV * dim; i += ATHREADS) qs[i] = q[i] * a.scale;
    for (int i = tid; i < QV; i += ATHREADS) mrun[i] = -INFINITY, lrun[i] = 0.f;
  }
  float acc[AMAXACC];
#pragma unroll
  for (int i = 0; i < AMAXACC; ++i) acc[i] = 0.f;
  const int nacc = QV * vd;
  const size_t koff = a.shared_keys ? 0 : (size_t)g * kd, voff = (size_t)a.c.kw + (size_t)g * vd;
  const bool vec8 = a.c.elt_bytes == 2 && (a.c.page_elems % 8 == 0) && (a.c.layer_off % 8 == 0) && ((a.c.kw + a.c.vw) % 8 == 0) && (kd % 8 == 0) &&
                    (vd % 8 == 0) && (a.c.kw % 8 == 0);
  for (int t0 = i0; t0 < i1; t0 += ATK) {
    const int nk = min(ATK, i1 - t0);
    __syncthreads();  // the previous tile is consumed; q and m/l are written
    if (tid < nk) {
      const int i = t0 + tid;
      const int j = i < nfirst ? i : lo + (i - nfirst);
      rowp[tid] = kv_row_ptr(a.c, a.block_table, a.max_pages, slot, j);
      dist[tid] = pos - j;
    }
    __syncthreads();
    if (a.c.elt_bytes == 4) {
      for (int i = tid; i < nk * kd; i += ATHREADS) {
        const int key = i / kd, c = i - key * kd;
        Kt[key * (kd + 1) + c] = reinterpret_cast<const float*>(rowp[key])[koff + c];
      }
      for (int i = tid; i < nk * vd; i += ATHREADS) {
        const int key = i / vd, c = i - key * vd;
        Vt[key * vd + c] = reinterpret_cast<const float*>(rowp[key])[voff + c];
      }
    } else if (vec8) {  // bf16 rows whose pieces start on 16-byte boundaries: 8 elements per load
      const int kd8 = kd >> 3, vd8 = vd >> 3;
      for (int i = tid; i < nk * kd8; i += ATHREADS) {
        const int key = i / kd8, c = (i - key * kd8) * 8;
        const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(rowp[key]) + koff + c);
        float* d = Kt + key * (kd + 1) + c;
        d[0] = lo2f(v.x), d[1] = hi2f(v.x), d[2] = lo2f(v.y), d[3] = hi2f(v.y), d[4] = lo2f(v.z), d[5] = hi2f(v.z), d[6] = lo2f(v.w), d[7] = hi2f(v.w);
      }
      for (int i = tid; i < nk * vd8; i += ATHREADS) {
        const int key = i / vd8, c = (i - key * vd8) * 8;
        const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(rowp[key]) + voff + c);
        float* d = Vt + key * vd + c;
        d[0] = lo2f(v.x), d[1] = hi2f(v.x), d[2] = lo2f(v.y), d[3] = hi2f(v.y), d[4] = lo2f(v.z), d[5] = hi2f(v.z), d[6] = lo2f(v.w), d[7] = hi2f(v.w);
      }
    } else {
      for (int i = tid; i < nk * kd; i += ATHREADS) {
        const int key = i / kd, c = i - key * kd;
        Kt[key * (kd + 1) + c] = bf2f(reinterpret_cast<const bf16*>(rowp[key])[koff + c]);
      }
      for (int i = tid; i < nk * vd; i += ATHREADS) {
        const int key = i / vd, c = i - key * vd;
        Vt[key * vd + c] = bf2f(reinterpret_cast<const bf16*>(rowp[key])[voff + c]);
      }
    }
    __syncthreads();
    // scores: (query vector, key) pairs, key fastest
    for (int i = tid; i < QV * ATK; i += ATHREADS) {
      const int qv = i / ATK, key = i - qv * ATK;
      float s = -INFINITY;
      if (key < nk) {
        const float* qp = qs + qv * dim;
        const float* kp = Kt + key * (kd + 1) + (qv % maps) * dim;
        s = 0.f;
        for (int c = 0; c < dim; ++c) s = fmaf(qp[c], kp[c], s);
        if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        if (a.slopes) s -= a.slopes[h0 + qv / maps] * (float)dist[key];
      }
      sc[i] = s;
    }
    __syncthreads();
    // online softmax per query vector: a warp per vector, a lane per key
    for (int qv = warp; qv < QV; qv += ATHREADS / 32) {
      const float s = sc[qv * ATK + lane];
      const float mo = mrun[qv];
      const float mn = fmaxf(mo, warp_max(s));
      float p = 0.f, cf = 1.f;
      if (mn > -INFINITY) {
        cf = expf(mo - mn);  // mo = -inf: 0
        p = expf(s - mn);
      }
      const float ps = warp_sum(p);
      sc[qv * ATK + lane] = p;
      if (lane == 0) {
        corr[qv] = cf;
        mrun[qv] = mn;
        lrun[qv] = lrun[qv] * cf + ps;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < AMAXACC; ++i) {
      const int idx = tid + i * ATHREADS;
      if (idx < nacc) {
        const int qv = idx / vd, col = idx - qv * vd;
        float v = acc[i] * corr[qv];
        const float* pp = sc + qv * ATK;
        for (int key = 0; key < nk; ++key) v = fmaf(pp[key], Vt[key * vd + col], v);
        acc[i] = v;
      }
    }
  }
  __syncthreads();
  // partial (m, l, acc) of (row, head, map, split)
#pragma unroll
  for (int i = 0; i < AMAXACC; ++i) {
    const int idx = tid + i * ATHREADS;
    if (idx < nacc) {
      const int qv = idx / vd, col = idx - qv * vd;
      const size_t rec = (((size_t)r * a.heads + h0) * maps + qv) * n_splits + split;
      a.ws[rec * (vd + 2) + 2 + col] = acc[i];
    }
  }
  for (int qv = tid; qv < QV; qv += ATHREADS) {
    const size_t rec = (((size_t)r * a.heads + h0) * maps + qv) * n_splits + split;
    a.ws[rec * (vd + 2)] = mrun[qv];
    a.ws[rec * (vd + 2) + 1] = lrun[qv];
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Prompt portions over a bf16 cache on tensor cores (mma.sync m16n8k16, fp32 accumulation): a CTA takes 64 consecutive
// rows of one segment and one query head; each of its 4 warps owns 16 rows and walks the key blocks of 64 keys that the
// CTA stages in shared memory once for all rows (the windows of neighbouring rows overlap almost completely).  Scores,
// the online softmax and the accumulators stay in registers (the score accumulators are re-packed as the A operand of
// the P V product); softmax, sink, gate and the differential finish are fp32.  Head sizes are padded with zeros to
// DP / VP.  Two score maps run one after the other; the first map's result waits in the output rows.
constexpr int PT_ROWS = 64, PT_KEYS = 64;

__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

template <int DP, int VP>
__global__ void __launch_bounds__(128) gqa_prefill_mma_kernel(const GqaAttnArgs a, const int* __restrict__ seg_start,
                                                              const int* __restrict__ seg_slot, int n_seg) {
  extern __shared__ __align__(16) unsigned char pt_smem[];  // two stages of a key block: K [2][64][DP + 8], V [2][64][VP + 8]
  typedef bf16 KTile[PT_KEYS][DP + 8];
  typedef bf16 VTile[PT_KEYS][VP + 8];
  KTile* Ks = reinterpret_cast<KTile*>(pt_smem);
  VTile* Vs = reinterpret_cast<VTile*>(pt_smem + 2 * sizeof(KTile));
  __shared__ int tile_info[5];  // segment's first row, its length, slot, the CTA's two tiles (-1: none)
  __shared__ const bf16* krow[2][PT_KEYS];  // cache rows of the keys of a stage (null: beyond the tile's last position)
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    // a CTA takes tile p and tile nt-1-p of a segment: under a causal mask the late tiles see many key blocks and the early
    // ones few, so every CTA gets about the same number
    // (under a sliding window every tile sees about the same number: one tile per CTA, twice the CTAs)
    const bool pair = a.window <= 0;
    int left = blockIdx.x, found = 0;
    for (int s = 0; s < n_seg && !found; ++s) {
      const int r0 = seg_start[s], len = seg_start[s + 1] - r0, nt = (len + PT_ROWS - 1) / PT_ROWS, np = pair ? (nt + 1) / 2 : nt;
      if (left < np) {
        tile_info[0] = r0, tile_info[1] = len, tile_info[2] = seg_slot[s];
        tile_info[3] = pair ? nt - 1 - left : left;
        tile_info[4] = pair && left != nt - 1 - left ? left : -1;
        found = 1;
      }
      left -= np;
    }
    if (!found) tile_info[3] = tile_info[4] = -1;
  }
  __syncthreads();
  const int slot = tile_info[2];
  const int h = blockIdx.y, g = h / (a.heads / a.kv_heads);
  const int dim = a.dim, vd = a.vdim, maps = a.maps, kd = maps * dim;
  for (int which = 0; which < 2; ++which) {
  const int tile = tile_info[3 + which];
  if (tile < 0) break;
  const int row0 = tile_info[0] + tile * PT_ROWS, nrows = min(PT_ROWS, tile_info[1] - tile * PT_ROWS);
  const int pos0 = a.pos[row0];                       // rows of a segment are consecutive positions
  const int pmax = pos0 + nrows - 1;
  const int lo_min = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const float slope = a.slopes ? a.slopes[h] : 0.f;
  // soft cap of a scaled score: cap * tanh(s / cap) as cap * (1 - 2 / (exp(2 s / cap) + 1)); the weights become bf16 operands
  // below, far coarser than the fast exponential
  const float cap = a.softcap, cap2 = cap > 0.f ? 2.0f / cap : 0.f;
  auto capped = [&](float v) { return cap > 0.f ? cap - 2.0f * cap / (__expf(fminf(v * cap2, 80.f)) + 1.0f) : v; };
  const int qr = lane >> 2, qc = (lane & 3) * 2;      // this thread's rows qr, qr + 8 and column pair of every 8-block
  const int wrow = warp * 16;
  const bool rv0 = wrow + qr < nrows, rv1 = wrow + qr + 8 < nrows;
  const int i0 = pos0 + wrow + qr, i1 = i0 + 8;       // positions of the thread's two rows
  // 16-byte staging when every cache row piece starts on a 16-byte boundary
  const bool vec = (a.c.page_elems % 8 == 0) && (a.c.layer_off % 8 == 0) && ((a.c.kw + a.c.vw) % 8 == 0) && (dim % 8 == 0) && (vd % 8 == 0) &&
                   (a.c.kw % 8 == 0);
  for (int mp = 0; mp < maps; ++mp) {
    uint32_t qf[DP / 16][4];
    {
      const float* q0 = a.q + (size_t)(row0 + wrow + qr) * a.ldq + (size_t)h * kd + mp * dim;
      const float* q1 = q0 + (size_t)8 * a.ldq;
#pragma unroll
      for (int kk = 0; kk < DP / 16; ++kk) {
        const int c = kk * 16 + qc;
        float v[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {  // columns c, c+1, c+8, c+9
          const int cc = c + (e >> 1) * 8 + (e & 1);
          v[e] = (rv0 && cc < dim) ? q0[cc] : 0.f;
          v[4 + e] = (rv1 && cc < dim) ? q1[cc] : 0.f;
        }
        qf[kk][0] = pack2(f2bf(v[0]), f2bf(v[1]));
        qf[kk][1] = pack2(f2bf(v[4]), f2bf(v[5]));
        qf[kk][2] = pack2(f2bf(v[2]), f2bf(v[3]));
        qf[kk][3] = pack2(f2bf(v[6]), f2bf(v[7]));
      }
    }
    float o[VP / 8][4];
#pragma unroll
    for (int i = 0; i < VP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    // key blocks that some row of the tile sees: the blocks of the kept first tokens, then from the window's lower edge on
    auto skipped = [&](int j) { return a.window > 0 && j + PT_KEYS - 1 < lo_min && j >= a.keep_first; };
    auto next_block = [&](int j) {
      j += PT_KEYS;
      return skipped(j) ? lo_min / PT_KEYS * PT_KEYS : j;
    };
    // a key block -> stage `buf` (cp.async when every piece of a cache row starts on a 16-byte boundary); one commit group
    auto stage = [&](int jb, int buf) {
      if (tid < PT_KEYS)  // one page lookup per key, not per 16-byte piece
        krow[buf][tid] = jb + tid <= pmax ? reinterpret_cast<const bf16*>(kv_row_ptr(a.c, a.block_table, a.max_pages, slot, jb + tid)) : nullptr;
      __syncthreads();
      for (int i = tid; i < PT_KEYS * (DP / 8); i += 128) {
        const int key = i / (DP / 8), c = (i % (DP / 8)) * 8;
        bf16* dst = &Ks[buf][key][c];
        const bf16* row = krow[buf][key];
        if (row && c < dim) {
          const bf16* src = row + (a.shared_keys ? 0 : (size_t)g * kd) + mp * dim + c;
          if (vec) cp_async16(smem_u32(dst), src);
          else
            for (int e = 0; e < 8; ++e) dst[e] = c + e < dim ? src[e] : f2bf(0.f);
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      for (int i = tid; i < PT_KEYS * (VP / 8); i += 128) {
        const int key = i / (VP / 8), c = (i % (VP / 8)) * 8;
        bf16* dst = &Vs[buf][key][c];
        const bf16* row = krow[buf][key];
        if (row && c < vd) {
          const bf16* src = row + a.c.kw + (size_t)g * vd + c;
          if (vec) cp_async16(smem_u32(dst), src);
          else
            for (int e = 0; e < 8; ++e) dst[e] = c + e < vd ? src[e] : f2bf(0.f);
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      cp_async_commit();
    };
    int j0 = skipped(0) ? lo_min / PT_KEYS * PT_KEYS : 0, buf = 0;
    stage(j0, 0);
    while (true) {
      const int jn = next_block(j0);
      const bool more = jn <= pmax;
      if (more) {  // the next block streams in while this one is multiplied
        stage(jn, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      // scores of the warp's 16 rows against the 64 keys
      float s[PT_KEYS / 8][4];
#pragma unroll
      for (int nb = 0; nb < PT_KEYS / 8; ++nb) {
        s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
          uint32_t b0, b1;
          ldmatrix_x2(b0, b1, smem_u32(&Ks[buf][nb * 8 + (lane & 7)][kk * 16 + ((lane >> 3) & 1) * 8]));
          mma_bf16_16816(s[nb], qf[kk], b0, b1);
        }
      }
      // mask, running maximum
      float mx0 = -INFINITY, mx1 = -INFINITY;
      // a block that every row of the warp sees whole (below the diagonal, inside the window) needs no mask
      const bool whole = j0 + PT_KEYS - 1 <= pos0 + wrow && (a.window <= 0 || pos0 + wrow + 15 - j0 < a.window);
      if (whole) {
        const float d0 = -slope * (float)(i0 - j0 - qc), d1 = -slope * (float)(i1 - j0 - qc);  // minus slope times the distance to the thread's first column
#pragma unroll
        for (int nb = 0; nb < PT_KEYS / 8; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[nb][e] = capped(s[nb][e] * a.scale) + fmaf(slope, (float)(nb * 8 + (e & 1)), (e >> 1) ? d1 : d0);
            if (e >> 1) mx1 = fmaxf(mx1, s[nb][e]);
            else mx0 = fmaxf(mx0, s[nb][e]);
          }
      } else {
#pragma unroll
        for (int nb = 0; nb < PT_KEYS / 8; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = j0 + nb * 8 + qc + (e & 1);
            const int i = (e >> 1) ? i1 : i0;
            const bool ok = j <= i && (a.window <= 0 || i - j < a.window || j < a.keep_first);
            s[nb][e] = ok ? capped(s[nb][e] * a.scale) - slope * (float)(i - j) : -INFINITY;  // the scale meets the fp32 score, not the bf16 operand
            if (e >> 1) mx1 = fmaxf(mx1, s[nb][e]);
            else mx0 = fmaxf(mx0, s[nb][e]);
          }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // the weights become bf16 operands below: the fast exponential's error is far under their rounding
      const float c0 = mn0 > -INFINITY ? __expf(m0 - mn0) : 1.f, c1 = mn1 > -INFINITY ? __expf(m1 - mn1) : 1.f;
      m0 = mn0, m1 = mn1;
      l0 *= c0, l1 *= c1;
#pragma unroll
      for (int i = 0; i < VP / 8; ++i) o[i][0] *= c0, o[i][1] *= c0, o[i][2] *= c1, o[i][3] *= c1;
#pragma unroll
      for (int nb = 0; nb < PT_KEYS / 8; ++nb) {
        s[nb][0] = mn0 > -INFINITY ? __expf(s[nb][0] - mn0) : 0.f;
        s[nb][1] = mn0 > -INFINITY ? __expf(s[nb][1] - mn0) : 0.f;
        s[nb][2] = mn1 > -INFINITY ? __expf(s[nb][2] - mn1) : 0.f;
        s[nb][3] = mn1 > -INFINITY ? __expf(s[nb][3] - mn1) : 0.f;
        l0 += s[nb][0] + s[nb][1];
        l1 += s[nb][2] + s[nb][3];
      }
      // O += P V, 16 keys per step; the softmax weights go in as bf16 hi + lo pairs (two MMAs), so they keep ~16 bits
#pragma unroll
      for (int kb = 0; kb < PT_KEYS / 16; ++kb) {
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          const float x0 = s[2 * kb + (f >> 1)][(f & 1) * 2], x1 = s[2 * kb + (f >> 1)][(f & 1) * 2 + 1];
          const bf16 h0 = f2bf(x0), h1 = f2bf(x1);
          ph[f] = pack2(h0, h1);
          pl[f] = pack2(f2bf(x0 - bf2f(h0)), f2bf(x1 - bf2f(h1)));
        }
#pragma unroll
        for (int vb = 0; vb < VP / 8; ++vb) {
          uint32_t b0, b1;
          ldmatrix_x2_trans(b0, b1, smem_u32(&Vs[buf][kb * 16 + (lane & 15)][vb * 8]));
          mma_bf16_16816(o[vb], ph, b0, b1);
          mma_bf16_16816(o[vb], pl, b0, b1);
        }
      }
      __syncthreads();  // the stage is free for the block after the next
      if (!more) break;
      j0 = jn;
      buf ^= 1;
    }
    // the rows' sums over the quad, the sink, the normalisation
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float f0, f1;
    if (a.unit_sink) {
      const float M0 = fmaxf(m0, 0.f), M1 = fmaxf(m1, 0.f);
      const float e0 = m0 > -INFINITY ? expf(m0 - M0) : 0.f, e1 = m1 > -INFINITY ? expf(m1 - M1) : 0.f;
      f0 = e0 / (l0 * e0 + expf(-M0));
      f1 = e1 / (l1 * e1 + expf(-M1));
    } else {
      f0 = l0 > 0.f ? 1.0f / l0 : 0.f;
      f1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    }
    float* out0 = a.out + (size_t)(row0 + wrow + qr) * a.ldo + (size_t)h * vd;
    float* out1 = out0 + (size_t)8 * a.ldo;
    const bool last = mp == maps - 1;
    float g0 = 1.f, g1 = 1.f;
    if (a.finish == 1) {
      if (rv0) g0 = 1.0f / (1.0f + expf(-a.gate[(size_t)(row0 + wrow + qr) * a.ldg + h]));
      if (rv1) g1 = 1.0f / (1.0f + expf(-a.gate[(size_t)(row0 + wrow + qr + 8) * a.ldg + h]));
    }
    float sq0 = 0.f, sq1 = 0.f;
#pragma unroll
    for (int vb = 0; vb < VP / 8; ++vb) {
      const int c = vb * 8 + qc;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (c + e >= vd) continue;
        float v0 = o[vb][e] * f0, v1 = o[vb][2 + e] * f1;
        if (last && a.finish == 1) v0 *= g0, v1 *= g1;
        if (last && a.finish == 3) {
          if (rv0) v0 *= 1.0f / (1.0f + expf(-a.gate[(size_t)(row0 + wrow + qr) * a.ldg + (size_t)h * vd + c + e]));
          if (rv1) v1 *= 1.0f / (1.0f + expf(-a.gate[(size_t)(row0 + wrow + qr + 8) * a.ldg + (size_t)h * vd + c + e]));
        }
        if (last && a.finish == 2) {  // the first map's result was parked in the output rows by this thread
          v0 = (rv0 ? out0[c + e] : 0.f) - a.lam * v0;
          v1 = (rv1 ? out1[c + e] : 0.f) - a.lam * v1;
          sq0 = fmaf(v0, v0, sq0), sq1 = fmaf(v1, v1, sq1);
          o[vb][e] = v0, o[vb][2 + e] = v1;
        } else if (a.out_bf && last) {  // (the first of two maps waits in the fp32 rows)
          if (rv0) a.out_bf[(size_t)(row0 + wrow + qr) * a.ldo_bf + (size_t)h * vd + c + e] = f2bf(v0);
          if (rv1) a.out_bf[(size_t)(row0 + wrow + qr + 8) * a.ldo_bf + (size_t)h * vd + c + e] = f2bf(v1);
        } else {
          if (rv0) out0[c + e] = v0;
          if (rv1) out1[c + e] = v1;
        }
      }
    }
    if (last && a.finish == 2) {
      sq0 += __shfl_xor_sync(0xffffffffu, sq0, 1);
      sq0 += __shfl_xor_sync(0xffffffffu, sq0, 2);
      sq1 += __shfl_xor_sync(0xffffffffu, sq1, 1);
      sq1 += __shfl_xor_sync(0xffffffffu, sq1, 2);
      const float r0 = a.post / sqrtf(sq0 / (float)vd + a.eps), r1 = a.post / sqrtf(sq1 / (float)vd + a.eps);
#pragma unroll
      for (int vb = 0; vb < VP / 8; ++vb) {
        const int c = vb * 8 + qc;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          if (c + e >= vd) continue;
          if (a.out_bf) {
            if (rv0) a.out_bf[(size_t)(row0 + wrow + qr) * a.ldo_bf + (size_t)h * vd + c + e] = f2bf(o[vb][e] * r0);
            if (rv1) a.out_bf[(size_t)(row0 + wrow + qr + 8) * a.ldo_bf + (size_t)h * vd + c + e] = f2bf(o[vb][2 + e] * r1);
            continue;
          }
          if (rv0) out0[c + e] = o[vb][e] * r0;
          if (rv1) out1[c + e] = o[vb][2 + e] * r1;
        }
      }
    }
  }
  }
}

template <int DP, int VP>
cudaError_t launch_prefill_mma_dv(const GqaAttnArgs& a, const int* seg_start, const int* seg_slot, int n_seg, cudaStream_t st) {
  const int per_cta = a.window <= 0 ? 2 * PT_ROWS : PT_ROWS;
  const dim3 grid((a.n + per_cta - 1) / per_cta + n_seg, a.heads), block(128);  // upper bound of the tiles / tile pairs
  const size_t smem = (size_t)2 * PT_KEYS * ((DP + 8) + (VP + 8)) * sizeof(bf16);
  if (smem > 48 * 1024) {
    cudaError_t r = cudaFuncSetAttribute(gqa_prefill_mma_kernel<DP, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (r != cudaSuccess) return r;
  }
  return launch_k(gqa_prefill_mma_kernel<DP, VP>, grid, block, smem, st, a, seg_start, seg_slot, n_seg);
}

template <int DP>
cudaError_t launch_prefill_mma_v(const GqaAttnArgs& a, const int* seg_start, const int* seg_slot, int n_seg, cudaStream_t st) {
  if (a.vdim <= 32) return launch_prefill_mma_dv<DP, 32>(a, seg_start, seg_slot, n_seg, st);
  if (a.vdim <= 64) return launch_prefill_mma_dv<DP, 64>(a, seg_start, seg_slot, n_seg, st);
  return launch_prefill_mma_dv<DP, 128>(a, seg_start, seg_slot, n_seg, st);
}

// CTA (row, head): merges the key splits of each map, adds the sink, applies the finishing step
__global__ void __launch_bounds__(128) gqa_finish_kernel(const GqaAttnArgs a, int n_splits) {
  extern __shared__ float o[];  // [vd]
  __shared__ float red[4];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, vd = a.vdim, maps = a.maps;
  float wsp[2][16];  // per map and split: weight of the split's accumulator (n_splits <= 16)
  float inv_l[2];
  for (int m = 0; m < maps; ++m) {
    const float* rec = a.ws + ((((size_t)r * a.heads + h) * maps + m) * n_splits) * (vd + 2);
    float M = a.unit_sink ? 0.f : -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, rec[(size_t)s * (vd + 2)]);
    float L = a.unit_sink ? expf(-M) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = rec[(size_t)s * (vd + 2)];
      const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
      wsp[m][s] = w;
      L = fmaf(rec[(size_t)s * (vd + 2) + 1], w, L);
    }
    inv_l[m] = 1.0f / L;
  }
  float gate = 1.f;
  if (a.finish == 1) gate = 1.0f / (1.0f + expf(-a.gate[(size_t)r * a.ldg + h]));
  float sq = 0.f;
  for (int c = threadIdx.x; c < vd; c += blockDim.x) {
    float am[2] = {0.f, 0.f};
    for (int m = 0; m < maps; ++m) {
      const float* rec = a.ws + ((((size_t)r * a.heads + h) * maps + m) * n_splits) * (vd + 2);
      float v = 0.f;
      for (int s = 0; s < n_splits; ++s) v = fmaf(rec[(size_t)s * (vd + 2) + 2 + c], wsp[m][s], v);
      am[m] = v * inv_l[m];
    }
    float v = am[0];
    if (a.finish == 1) v *= gate;
    else if (a.finish == 2) v = am[0] - a.lam * am[1];
    else if (a.finish == 3) v *= 1.0f / (1.0f + expf(-a.gate[(size_t)r * a.ldg + (size_t)h * vd + c]));
    o[c] = v;
    sq = fmaf(v, v, sq);
  }
  float rstd = 1.f;
  if (a.finish == 2) {
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    rstd = a.post / sqrtf(t / (float)vd + a.eps);
  }
  if (a.out_bf) {
    bf16* ob = a.out_bf + (size_t)r * a.ldo_bf + (size_t)h * vd;
    for (int c = threadIdx.x; c < vd; c += blockDim.x) ob[c] = f2bf(o[c] * rstd);
    return;
  }
  float* out = a.out + (size_t)r * a.ldo + (size_t)h * vd;
  for (int c = threadIdx.x; c < vd; c += blockDim.x) out[c] = o[c] * rstd;
}

}  // namespace

static size_t talk_smem(const TalkQueries& t) { return ((size_t)t.heads * t.dim + (size_t)t.heads * t.heads) * sizeof(float); }

cudaError_t launch_kv_store_rows(const KvStoreArgs& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  if ((a.k_norm || a.rope.dims > 0) && (a.norm_dim <= 0 || a.c.kw % a.norm_dim || a.rope.dims > a.norm_dim || a.rope.dims % 2)) return cudaErrorInvalidValue;
  size_t smem = 0;
  if (a.tq.talk) {
    if (a.tq.heads <= 0 || a.tq.kv_heads <= 0 || a.tq.heads % a.tq.kv_heads) return cudaErrorInvalidValue;
    smem = talk_smem(a.tq);
    if (smem > 48 * 1024) {
      if (smem > 200 * 1024) return cudaErrorInvalidValue;
      cudaError_t r = cudaFuncSetAttribute(kv_store_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (r != cudaSuccess) return r;
    }
  }
  return launch_k(kv_store_rows_kernel, dim3(a.n), dim3(128), smem, st, a);
}

cudaError_t launch_gqa_attention(const GqaAttnArgs& a, cudaStream_t st, int* n_launches) {
  if (n_launches) *n_launches = 0;
  if (a.n <= 0) return cudaSuccess;
  if (a.shared_keys && (a.maps != 1 || a.dim != a.c.kw)) return cudaErrorInvalidValue;
  if (a.finish == 3 && !a.gate) return cudaErrorInvalidValue;
  if (a.out_bf && a.maps != 1 && !a.out) return cudaErrorInvalidValue;  // two maps: the first one's result waits in the fp32 rows
  // prompt portions over a bf16 cache: the tensor-core kernel (one launch, no workspace); QIE_ATTN_MMA=0 keeps the per-row kernel (A/B)
  static const bool mma_on = [] { const char* v = getenv("QIE_ATTN_MMA"); return !(v && v[0] == '0'); }();
  if (mma_on && a.seg_start && a.c.elt_bytes == 2 && a.n >= 64 && a.dim <= 128 && a.vdim <= 128 && a.maps <= 2 && a.heads % a.kv_heads == 0 &&
      (a.finish != 2 || a.maps == 2)) {
    if (n_launches) *n_launches = 1;
    if (a.dim <= 32) return launch_prefill_mma_v<32>(a, a.seg_start, a.seg_slot, a.n_seg, st);
    if (a.dim <= 64) return launch_prefill_mma_v<64>(a, a.seg_start, a.seg_slot, a.n_seg, st);
    return launch_prefill_mma_v<128>(a, a.seg_start, a.seg_slot, a.n_seg, st);
  }
  if (a.maps < 1 || a.maps > 2 || a.heads % a.kv_heads || (a.finish == 2 && a.maps != 2) || a.maps * a.vdim > ATHREADS * AMAXACC)
    return cudaErrorInvalidValue;
  const int hpg = a.heads / a.kv_heads;
  const int hpc = std::max(1, std::min(hpg, ATHREADS * AMAXACC / (a.maps * a.vdim)));
  const int chunks = (hpg + hpc - 1) / hpc;
  // key splits: fill the machine when there are few rows, within the workspace
  int splits = 1;
  const long ctas = (long)a.n * a.kv_heads * chunks;
  if (ctas < 2L * a.num_sms && a.max_keys > 2 * ATK) {
    splits = (int)std::min<long>((2L * a.num_sms + ctas - 1) / ctas, (a.max_keys + 2 * ATK - 1) / (2 * ATK));
    splits = std::max(1, std::min(splits, 16));
  }
  const size_t one = gqa_ws_floats(a.n, a.heads, a.maps, a.vdim);
  if (one > a.ws_floats) return cudaErrorInvalidValue;
  splits = (int)std::min<size_t>(splits, a.ws_floats / one);
  const int kd = a.maps * a.dim, qvm = hpc * a.maps;
  const size_t smem = ((size_t)qvm * a.dim + (size_t)ATK * (kd + 1) + (size_t)ATK * a.vdim + (size_t)qvm * ATK + 3 * (size_t)qvm) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t r = cudaFuncSetAttribute(gqa_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (r != cudaSuccess) return r;
  }
  cudaError_t r = launch_k(gqa_attention_kernel, dim3(a.n, a.kv_heads * chunks, splits), dim3(ATHREADS), smem, st, a, hpc, chunks, splits);
  if (r != cudaSuccess) return r;
  if (n_launches) *n_launches = 2;
  return launch_k(gqa_finish_kernel, dim3(a.n, a.heads), dim3(128), (size_t)a.vdim * sizeof(float), st, a, splits);
}

}  // namespace qie
