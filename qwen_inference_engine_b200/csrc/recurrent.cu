// recurrent.cu -- the short causal convolution and the two linear recurrences of the fp32-stream families
// (fosavik.h): the real-gated linear recurrent unit of Griffin (one state per channel) and the state-space recurrence
// of Mamba-2 (a state matrix per head), with the gated group norm behind it and the clamped gated activation of the
// feed-forward; and the minGRU recurrence (dedunex.h: one state per channel, gates that read only the current token).  A launch walks SEGMENTS: runs of consecutive rows of one sequence, whose state lives in the
// sequence's slot and is carried from call to call.  Everything that enters a recurrence is fp32.
#include <algorithm>

#include "dedunex.h"
#include "fosavik.h"
#include "launch.h"

namespace qie {
namespace {

constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_ROWS = 64;  // rows of a segment per CTA
constexpr int LRU_PF = 16;     // rows whose loads a scan thread keeps in flight

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanhf_(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// grid (segments, channel blocks, row chunks): a thread owns a channel and walks CONV_ROWS rows of the segment with
// the last taps-1 inputs in registers; inputs before the segment come from the slot's tail
__global__ void __launch_bounds__(128) causal_conv_kernel(const ConvArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  const int t0 = r0 + blockIdx.z * CONV_ROWS, t1 = min(r1, t0 + CONV_ROWS);
  if (t0 >= r1 || c >= a.channels) return;
  const int taps = a.taps;
  const float* tail = a.tail + (size_t)a.seg_slot[seg] * a.slot_stride;
  const float ib = a.in_bias ? bf2f(a.in_bias[c]) : 0.f;
  float w[CONV_MAX_TAPS], win[CONV_MAX_TAPS];  // win[i]: input at t - (taps-1-i)
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) win[i] = 0.f;
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    w[i] = i < taps ? bf2f(a.w[(size_t)c * taps + i]) : 0.f;
    if (i < taps - 1) {  // input at row t0 - (taps-1-i)
      const int t = t0 - (taps - 1 - i);
      win[i + 1] = t >= r0 ? a.x[(size_t)t * a.ldx + c] + ib : tail[(size_t)(taps - 1 - (r0 - t)) * a.channels + c];
    }
  }
  const float bias = bf2f(a.b[c]);
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) win[i] = win[i + 1];
    // after the shift win[taps-1] must hold the current input: the window is kept right-aligned at index taps-1
    const float cur = a.x[(size_t)t * a.ldx + c] + ib;
    float acc = bias;
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i) {
      if (i == taps - 1) win[i] = cur;
      if (i < taps) acc = fmaf(w[i], win[i], acc);
    }
    a.out[(size_t)t * a.ldo + c] = a.act == 1 ? siluf_(acc) : acc;
  }
}

// thread (segment, channel): the new tail = the last taps-1 inputs (rows of the segment, older ones from the old tail)
__global__ void conv_tail_kernel(const ConvArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1], taps = a.taps;
  float* tail = a.tail + (size_t)a.seg_slot[seg] * a.slot_stride;
  const float ib = a.in_bias ? bf2f(a.in_bias[c]) : 0.f;
  float nv[CONV_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    nv[i] = 0.f;
    if (i < taps - 1) {  // new tail[i] = input at row r1 - (taps-1) + i
      const int t = r1 - (taps - 1) + i;
      nv[i] = t >= r0 ? a.x[(size_t)t * a.ldx + c] + ib : tail[(size_t)(taps - 1 - (r0 - t)) * a.channels + c];
    }
  }
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i)
    if (i < taps - 1) tail[(size_t)i * a.channels + c] = nv[i];
}

// thread (segment, channel) walks the segment's rows
__global__ void __launch_bounds__(64) lru_scan_kernel(const LruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  float* sp = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + c;
  float S = *sp;
  const float k_ = -a.decay_c * softplusf_(bf2f(a.lam[c]));
  const float yb = a.y_bias ? bf2f(a.y_bias[c]) : 0.f;
  for (int t0 = r0; t0 < r1; t0 += LRU_PF) {  // the loads of LRU_PF rows are in flight together; the recurrence itself is one FMA per row
    float zr[LRU_PF], zi[LRU_PF], uv[LRU_PF], yv[LRU_PF];
#pragma unroll
    for (int k = 0; k < LRU_PF; ++k) {
      const int t = min(t0 + k, r1 - 1);
      zr[k] = a.zr[(size_t)t * a.ldz + c];
      zi[k] = a.zi[(size_t)t * a.ldz + c];
      uv[k] = a.u[(size_t)t * a.ldu + c];
      yv[k] = a.yb[(size_t)t * a.ldy + c];
    }
#pragma unroll
    for (int k = 0; k < LRU_PF; ++k) {
      if (t0 + k < r1) {
        const float la = k_ * sigmoidf_(zr[k]);
        const float av = expf(la);
        const float mult = sqrtf(fmaxf(-expm1f(2.0f * la), 0.f));  // sqrt(1 - a^2) without cancellation near a = 1
        S = fmaf(av, S, mult * (sigmoidf_(zi[k]) * uv[k]));
        a.out[(size_t)(t0 + k) * a.ldo + c] = S * gelu_tanhf_(yv[k] + yb);
      }
    }
  }
  *sp = S;
}

// The same recurrence for long segments in three parallel steps over chunks of LRU_CHUNK rows (a chunk starts at a
// multiple of LRU_CHUNK rows from its segment's start).  (1) every chunk runs from a zero state: the local states go to
// `out`, the running product of the decays replaces zr, the chunk's total decay P and end state Q go to the workspace;
// (2) one thread per channel carries the true state over the chunks (S_in of every chunk, the slot's final state);
// (3) S_t = local_t + decay_t * S_in, times the gelu branch.  Only the rounding differs from the row-by-row kernel.
constexpr int LRU_CHUNK = 64;
__device__ __forceinline__ int lru_chunk_id(int r0, int seg, int k) { return r0 / LRU_CHUNK + seg + k; }  // unique over the batch

__global__ void __launch_bounds__(64) lru_chunk_local_kernel(const LruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x, k = blockIdx.z;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  const int t0 = r0 + k * LRU_CHUNK, t1 = min(r1, t0 + LRU_CHUNK);
  if (t0 >= r1 || c >= a.channels) return;
  const float k_ = -a.decay_c * softplusf_(bf2f(a.lam[c]));
  float* cum_out = const_cast<float*>(a.zr);
  float S = 0.f, cum = 1.f;
  for (int tb = t0; tb < t1; tb += LRU_PF) {
    float zr[LRU_PF], zi[LRU_PF], uv[LRU_PF];
#pragma unroll
    for (int j = 0; j < LRU_PF; ++j) {
      const int t = min(tb + j, t1 - 1);
      zr[j] = a.zr[(size_t)t * a.ldz + c];
      zi[j] = a.zi[(size_t)t * a.ldz + c];
      uv[j] = a.u[(size_t)t * a.ldu + c];
    }
#pragma unroll
    for (int j = 0; j < LRU_PF; ++j) {
      if (tb + j < t1) {
        const float la = k_ * sigmoidf_(zr[j]);
        const float av = expf(la);
        const float mult = sqrtf(fmaxf(-expm1f(2.0f * la), 0.f));
        S = fmaf(av, S, mult * (sigmoidf_(zi[j]) * uv[j]));
        cum *= av;
        a.out[(size_t)(tb + j) * a.ldo + c] = S;
        cum_out[(size_t)(tb + j) * a.ldz + c] = cum;
      }
    }
  }
  float* w = a.ws + (size_t)lru_chunk_id(r0, seg, k) * 2 * a.channels;
  w[c] = cum;
  w[a.channels + c] = S;
}

__global__ void __launch_bounds__(64) lru_chunk_carry_kernel(const LruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  float* sp = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + c;
  float S = *sp;
  for (int k = 0; r0 + k * LRU_CHUNK < r1; ++k) {
    float* w = a.ws + (size_t)lru_chunk_id(r0, seg, k) * 2 * a.channels;
    const float P = w[c], Q = w[a.channels + c];
    w[c] = S;  // the chunk's incoming state
    S = fmaf(P, S, Q);
  }
  *sp = S;
}

__global__ void __launch_bounds__(128) lru_chunk_apply_kernel(const LruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x, k = blockIdx.z;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  const int t0 = r0 + k * LRU_CHUNK, t1 = min(r1, t0 + LRU_CHUNK);
  if (t0 >= r1 || c >= a.channels) return;
  const float Sin = a.ws[(size_t)lru_chunk_id(r0, seg, k) * 2 * a.channels + c];
  const float yb = a.y_bias ? bf2f(a.y_bias[c]) : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float S = fmaf(a.zr[(size_t)t * a.ldz + c], Sin, a.out[(size_t)t * a.ldo + c]);
    a.out[(size_t)t * a.ldo + c] = S * gelu_tanhf_(a.yb[(size_t)t * a.ldy + c] + yb);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// minGRU: S = (1 - z) S + z cand, one state per channel.  The gate z = sigmoid(zp), so the decay 1 - z is sigmoid(-zp)
// (exact where z is close to 1); the candidate is u + 1/2 for u >= 0 and sigmoid(u) below (continuous at 0).
__device__ __forceinline__ float mg_ld(const float* f, const bf16* b, size_t i) { return f ? f[i] : bf2f(b[i]); }
__device__ __forceinline__ void mg_gates(float zp, float u, float* decay, float* in) {
  const float z = sigmoidf_(zp);
  *decay = sigmoidf_(-zp);
  *in = z * (u >= 0.f ? u + 0.5f : sigmoidf_(u));
}
__device__ __forceinline__ void mg_store(const MinGruArgs& a, size_t t, int c, float S, float gp) {
  const float v = S * siluf_(gp);
  if (a.out) a.out[t * a.ldo + c] = v;
  if (a.out_bf) a.out_bf[t * a.ldo_bf + c] = f2bf(v);
}
constexpr int MG_PF = 16;  // rows whose loads a scan thread keeps in flight

// thread (segment, channel) walks the segment's rows
__global__ void __launch_bounds__(64) mingru_scan_kernel(const MinGruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  const size_t ld = a.zp ? a.ld : a.ld_bf;
  float* sp = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + c;
  float S = *sp;
  const float zb = a.z_bias ? bf2f(a.z_bias[c]) : 0.f, ub = a.u_bias ? bf2f(a.u_bias[c]) : 0.f;
  for (int t0 = r0; t0 < r1; t0 += MG_PF) {
    float zv[MG_PF], uv[MG_PF], gv[MG_PF];
#pragma unroll
    for (int k = 0; k < MG_PF; ++k) {
      const size_t t = min(t0 + k, r1 - 1);
      zv[k] = mg_ld(a.zp, a.zp_bf, t * ld + c);
      uv[k] = mg_ld(a.up, a.up_bf, t * ld + c);
      gv[k] = mg_ld(a.gp, a.gp_bf, t * ld + c);
    }
#pragma unroll
    for (int k = 0; k < MG_PF; ++k) {
      if (t0 + k < r1) {
        float d, in;
        mg_gates(zv[k] + zb, uv[k] + ub, &d, &in);
        S = fmaf(d, S, in);
        mg_store(a, (size_t)(t0 + k), c, S, gv[k]);
      }
    }
  }
  *sp = S;
}

// The same recurrence for long portions in three parallel steps over chunks of MG_CHUNK rows (a chunk starts a multiple
// of MG_CHUNK rows from its segment's start).  (1) every chunk runs from a zero state: the local states and the running
// product of the decays go to the workspace, the chunk's total decay P and end state Q to its summary; (2) one thread per
// channel carries the true state over the chunks; (3) S_t = local_t + decay_t * S_in, times the output gate.
// Workspace: local [n_rows, channels] | cum [n_rows, channels] | summaries [ids, 2, channels].
constexpr int MG_CHUNK = 64;
__device__ __forceinline__ int mg_chunk_id(int r0, int seg, int k) { return r0 / MG_CHUNK + seg + k; }  // unique over the batch

__global__ void __launch_bounds__(64) mingru_chunk_local_kernel(const MinGruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x, k = blockIdx.z;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  const int t0 = r0 + k * MG_CHUNK, t1 = min(r1, t0 + MG_CHUNK);
  if (t0 >= r1 || c >= a.channels) return;
  const size_t ld = a.zp ? a.ld : a.ld_bf, C = a.channels;
  float* local = a.ws;
  float* cumw = a.ws + (size_t)a.n_rows * C;
  float* sums = cumw + (size_t)a.n_rows * C;
  const float zb = a.z_bias ? bf2f(a.z_bias[c]) : 0.f, ub = a.u_bias ? bf2f(a.u_bias[c]) : 0.f;
  float S = 0.f, cum = 1.f;
  for (int tb = t0; tb < t1; tb += MG_PF) {
    float zv[MG_PF], uv[MG_PF];
#pragma unroll
    for (int j = 0; j < MG_PF; ++j) {
      const size_t t = min(tb + j, t1 - 1);
      zv[j] = mg_ld(a.zp, a.zp_bf, t * ld + c);
      uv[j] = mg_ld(a.up, a.up_bf, t * ld + c);
    }
#pragma unroll
    for (int j = 0; j < MG_PF; ++j) {
      if (tb + j < t1) {
        float d, in;
        mg_gates(zv[j] + zb, uv[j] + ub, &d, &in);
        S = fmaf(d, S, in);
        cum *= d;
        local[(size_t)(tb + j) * C + c] = S;
        cumw[(size_t)(tb + j) * C + c] = cum;
      }
    }
  }
  float* w = sums + (size_t)mg_chunk_id(r0, seg, k) * 2 * C;
  w[c] = cum;
  w[C + c] = S;
}

__global__ void __launch_bounds__(64) mingru_chunk_carry_kernel(const MinGruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  const size_t C = a.channels;
  float* sums = a.ws + 2 * (size_t)a.n_rows * C;
  float* sp = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + c;
  float S = *sp;
  const int nk = (r1 - r0 + MG_CHUNK - 1) / MG_CHUNK;
  for (int k0 = 0; k0 < nk; k0 += 8) {  // the summaries of eight chunks are loaded together; the chain itself is one FMA per chunk
    float P[8], Q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float* w = sums + (size_t)mg_chunk_id(r0, seg, min(k0 + j, nk - 1)) * 2 * C;
      P[j] = w[c], Q[j] = w[C + c];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (k0 + j < nk) {
        sums[(size_t)mg_chunk_id(r0, seg, k0 + j) * 2 * C + c] = S;  // the chunk's incoming state
        S = fmaf(P[j], S, Q[j]);
      }
  }
  *sp = S;
}

// block (128 channels, 4 row lanes): the apply pass is elementwise over a chunk's rows
__global__ void __launch_bounds__(512) mingru_chunk_apply_kernel(const MinGruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x, k = blockIdx.z;
  const int r0 = a.seg_start[seg], r1 = a.seg_start[seg + 1];
  const int t0 = r0 + k * MG_CHUNK, t1 = min(r1, t0 + MG_CHUNK);
  if (t0 >= r1 || c >= a.channels) return;
  const size_t ld = a.zp ? a.ld : a.ld_bf, C = a.channels;
  const float* local = a.ws;
  const float* cumw = a.ws + (size_t)a.n_rows * C;
  const float Sin = cumw[(size_t)a.n_rows * C + (size_t)mg_chunk_id(r0, seg, k) * 2 * C + c];
  for (int t = t0 + threadIdx.y; t < t1; t += blockDim.y) {
    const float S = fmaf(cumw[(size_t)t * C + c], Sin, local[(size_t)t * C + c]);
    mg_store(a, (size_t)t, c, S, mg_ld(a.gp, a.gp_bf, (size_t)t * ld + c));
  }
}

// CTA (segment, head, column block): thread (ns, p) keeps rows ns, ns + NS, ... of column p of the head's state in
// registers; the inputs of SSD_TOK tokens are staged in shared memory, the partial outputs of the NS row slices are
// summed in a fixed order.
constexpr int SSD_TOK = 8, SSD_NR = 32;

// NR state rows per thread; EXACT: N == NR * NS, so no row needs a bound check (the loop bodies stay branch-free).
// MODE 0 walks a whole segment from the slot's state.  Long portions run in three parallel steps over chunks of SSD_CH
// tokens (a chunk starts a multiple of SSD_CH rows from its segment's start), as the decay is one number per head and token:
// MODE 1 runs every chunk from a zero state (local outputs to y, the running product of the decays to ws_cum, the chunk's
// total decay and end state to ws_p / ws_state), ssd_carry_kernel carries the true state over the chunks (leaving every
// chunk's incoming state in ws_state), MODE 2 adds C_t^T (cum_t * S_in) to y.  Only the rounding differs from MODE 0.
constexpr int SSD_CH = 64;
__device__ __forceinline__ int ssd_chunk_id(int r0, int seg, int k) { return r0 / SSD_CH + seg + k; }  // unique over the batch

template <int NR, bool EXACT, int MODE>
__global__ void __launch_bounds__(512) ssd_scan_kernel(const SsdArgs a, int PB, int NS, int chunks) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x / chunks, ck = blockIdx.x % chunks, hd = blockIdx.y, p0 = blockIdx.z * PB;
  const int N = a.N, P = a.P;
  const int p = threadIdx.x % PB, ns = threadIdx.x / PB;
  const int grp = hd / (a.heads / a.groups);
  float* Bs = sm;                       // [SSD_TOK][N]
  float* Cs = Bs + SSD_TOK * N;         // [SSD_TOK][N]
  float* xs = Cs + SSD_TOK * N;         // [SSD_TOK][PB]
  float* dts = xs + SSD_TOK * PB;       // [SSD_TOK] dt (MODE 2: cum), then [SSD_TOK] decay
  float* yp = dts + 2 * SSD_TOK;        // [SSD_TOK][NS][PB]
  const int s0 = a.seg_start[seg], s1 = a.seg_start[seg + 1];
  const int r0 = MODE == 0 ? s0 : s0 + ck * SSD_CH, r1 = MODE == 0 ? s1 : min(s1, r0 + SSD_CH);
  if (r0 >= s1) return;
  const bool colok = p0 + p < P;
  float* sp = MODE == 0 ? a.state + (size_t)a.seg_slot[seg] * a.slot_stride + (size_t)hd * N * P
                        : a.ws_state + ((size_t)ssd_chunk_id(s0, seg, ck) * a.heads + hd) * N * P;
  float S[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int n = ns + i * NS;
    S[i] = (MODE != 1 && (EXACT || n < N) && colok) ? sp[(size_t)n * P + p0 + p] : 0.f;
  }
  const float Dh = bf2f(a.D[hd]), Aneg = -expf(bf2f(a.A_log[hd])), dtb = bf2f(a.dt_bias[hd]);
  const int nthr = blockDim.x;
  const bool scribe = threadIdx.x == 0 && blockIdx.z == 0;  // writes what is one number per (token, head)
  float cum = 1.f;
  for (int t0 = r0; t0 < r1; t0 += SSD_TOK) {
    const int nt = min(SSD_TOK, r1 - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * N; i += nthr) {
      const int t = i / N, n = i - t * N;
      if (MODE != 2) Bs[t * N + n] = a.B[(size_t)(t0 + t) * a.ld + grp * N + n];
      Cs[t * N + n] = a.C[(size_t)(t0 + t) * a.ld + grp * N + n];
    }
    if (MODE != 2) {
      for (int i = threadIdx.x; i < nt * PB; i += nthr) {
        const int t = i / PB, pp = i - t * PB;
        xs[t * PB + pp] = p0 + pp < P ? a.x[(size_t)(t0 + t) * a.ld + (size_t)hd * P + p0 + pp] : 0.f;
      }
      for (int i = threadIdx.x; i < nt; i += nthr) {
        const float dt = softplusf_(a.dt_raw[(size_t)(t0 + i) * a.ld_dt + hd] + dtb);
        dts[i] = dt;
        dts[SSD_TOK + i] = expf(Aneg * dt);
      }
    } else {
      for (int i = threadIdx.x; i < nt; i += nthr) dts[i] = a.ws_cum[(size_t)(t0 + i) * a.heads + hd];
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      float y = 0.f;
      if (MODE != 2) {
        const float dt = dts[t], dec = dts[SSD_TOK + t];
        const float dx = dt * xs[t * PB + p];
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int n = ns + i * NS;
          if (EXACT || n < N) {
            S[i] = fmaf(dec, S[i], Bs[t * N + n] * dx);
            y = fmaf(S[i], Cs[t * N + n], y);
          }
        }
        if (MODE == 1) {
          cum *= dec;
          if (scribe) a.ws_cum[(size_t)(t0 + t) * a.heads + hd] = cum;
        }
      } else {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int n = ns + i * NS;
          if (EXACT || n < N) y = fmaf(S[i], Cs[t * N + n], y);
        }
      }
      yp[(t * NS + ns) * PB + p] = y;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * PB; i += nthr) {
      const int t = i / PB, pp = i - t * PB;
      if (p0 + pp >= P) continue;
      float y = 0.f;
      for (int s = 0; s < NS; ++s) y += yp[(t * NS + s) * PB + pp];
      float* dst = a.y + (size_t)(t0 + t) * a.ldy + (size_t)hd * P + p0 + pp;
      if (MODE != 2) *dst = fmaf(Dh, xs[t * PB + pp], y);
      else *dst = fmaf(dts[t], y, *dst);
    }
  }
  if (MODE == 2) return;
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int n = ns + i * NS;
    if ((EXACT || n < N) && colok) sp[(size_t)n * P + p0 + p] = S[i];
  }
  if (MODE == 1 && scribe) a.ws_p[(size_t)ssd_chunk_id(s0, seg, ck) * a.heads + hd] = cum;
}

// thread (segment, head, state element): S_in of every chunk replaces its local end state; the slot gets the final state
__global__ void __launch_bounds__(256) ssd_carry_kernel(const SsdArgs a) {
  pdl_wait();
  pdl_trigger();
  const int seg = blockIdx.x, hd = blockIdx.y;
  const size_t e = (size_t)blockIdx.z * blockDim.x + threadIdx.x, NP = (size_t)a.N * a.P;
  if (e >= NP) return;
  const int s0 = a.seg_start[seg], s1 = a.seg_start[seg + 1];
  float* sp = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + (size_t)hd * NP + e;
  float S = *sp;
  for (int k = 0; s0 + k * SSD_CH < s1; ++k) {
    const size_t id = (size_t)ssd_chunk_id(s0, seg, k);
    float* q = a.ws_state + (id * a.heads + hd) * NP + e;
    const float Q = *q, Pk = a.ws_p[id * a.heads + hd];
    *q = S;
    S = fmaf(Pk, S, Q);
  }
  *sp = S;
}

// CTA (row, group)
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ z, int ldz,
                                                               const bf16* __restrict__ w, float* __restrict__ out, int ldo, int gw, float eps) {
  __shared__ float red[8];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, c0 = blockIdx.y * gw;
  float sq = 0.f;
  for (int i = threadIdx.x; i < gw; i += blockDim.x) {
    const float v = y[(size_t)r * ldy + c0 + i] * siluf_(z[(size_t)r * ldz + c0 + i]);
    sq = fmaf(v, v, sq);
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
  const float rstd = 1.0f / sqrtf(t / (float)gw + eps);
  for (int i = threadIdx.x; i < gw; i += blockDim.x) {
    const float v = y[(size_t)r * ldy + c0 + i] * siluf_(z[(size_t)r * ldz + c0 + i]);
    out[(size_t)r * ldo + c0 + i] = v * rstd * bf2f(w[c0 + i]);
  }
}

__global__ void clamped_glu_kernel(const float* __restrict__ gu, int ld, float* __restrict__ out, int ff, float limit, float alpha, size_t total) {
  pdl_wait();
  pdl_trigger();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / ff;
    const int c = (int)(i - r * ff);
    const float g = fminf(gu[r * ld + c], limit);
    const float u = fminf(fmaxf(gu[r * ld + ff + c], -limit), limit);
    out[i] = g * sigmoidf_(alpha * g) * (u + 1.0f);
  }
}

}  // namespace

cudaError_t launch_causal_conv(const ConvArgs& a, cudaStream_t st) {
  if (a.n_seg <= 0 || a.n_rows <= 0) return cudaSuccess;
  if (a.taps < 1 || a.taps > CONV_MAX_TAPS) return cudaErrorInvalidValue;
  const int cb = (a.channels + 127) / 128;
  // the longest segment bounds the row chunks (n_rows rows at most)
  cudaError_t r = launch_k(causal_conv_kernel, dim3(a.n_seg, cb, (a.n_rows + CONV_ROWS - 1) / CONV_ROWS), dim3(128), 0, st, a);
  if (r != cudaSuccess || a.taps == 1) return r;
  return launch_k(conv_tail_kernel, dim3(a.n_seg, cb), dim3(128), 0, st, a);
}

cudaError_t launch_lru_scan(const LruArgs& a, cudaStream_t st) {
  if (a.n_seg <= 0 || a.n_rows <= 0) return cudaSuccess;
  const size_t ws_need = ((size_t)a.n_rows / LRU_CHUNK + a.n_seg + 2) * 2 * a.channels;
  if (a.ws && a.n_rows >= 4 * LRU_CHUNK && a.n_seg <= 64 && ws_need <= a.ws_floats) {  // long portions: chunks in parallel
    const int chunks = (a.n_rows + LRU_CHUNK - 1) / LRU_CHUNK;
    cudaError_t r = launch_k(lru_chunk_local_kernel, dim3(a.n_seg, (a.channels + 63) / 64, chunks), dim3(64), 0, st, a);
    if (r != cudaSuccess) return r;
    if ((r = launch_k(lru_chunk_carry_kernel, dim3(a.n_seg, (a.channels + 63) / 64), dim3(64), 0, st, a)) != cudaSuccess) return r;
    return launch_k(lru_chunk_apply_kernel, dim3(a.n_seg, (a.channels + 127) / 128, chunks), dim3(128), 0, st, a);
  }
  return launch_k(lru_scan_kernel, dim3(a.n_seg, (a.channels + 63) / 64), dim3(64), 0, st, a);
}

cudaError_t launch_mingru_scan(const MinGruArgs& a, cudaStream_t st) {
  if (a.n_seg <= 0 || a.n_rows <= 0) return cudaSuccess;
  if (!(a.zp && a.up && a.gp) && !(a.zp_bf && a.up_bf && a.gp_bf)) return cudaErrorInvalidValue;
  if ((!a.out && !a.out_bf) || !a.state || a.channels <= 0) return cudaErrorInvalidValue;
  if (a.ws && a.n_rows >= 4 * MG_CHUNK && a.n_seg <= 64 && mingru_ws_floats(a.n_rows, a.n_seg, a.channels) <= a.ws_floats) {
    const int chunks = (a.n_rows + MG_CHUNK - 1) / MG_CHUNK;
    cudaError_t r = launch_k(mingru_chunk_local_kernel, dim3(a.n_seg, (a.channels + 63) / 64, chunks), dim3(64), 0, st, a);
    if (r != cudaSuccess) return r;
    if ((r = launch_k(mingru_chunk_carry_kernel, dim3(a.n_seg, (a.channels + 63) / 64), dim3(64), 0, st, a)) != cudaSuccess) return r;
    return launch_k(mingru_chunk_apply_kernel, dim3(a.n_seg, (a.channels + 127) / 128, chunks), dim3(128, 4), 0, st, a);
  }
  return launch_k(mingru_scan_kernel, dim3(a.n_seg, (a.channels + 63) / 64), dim3(64), 0, st, a);
}

cudaError_t launch_ssd_scan(const SsdArgs& a, cudaStream_t st) {
  if (a.n_seg <= 0 || a.n_rows <= 0) return cudaSuccess;
  if (a.heads % a.groups) return cudaErrorInvalidValue;
  // long portions run chunk-parallel.  Workspace: cum [n_rows, heads] | chunk decays [ids, heads] | chunk states [ids, heads, N, P]
  const size_t ids = (size_t)a.n_rows / SSD_CH + a.n_seg + 2, NP = (size_t)a.N * a.P;
  const size_t need = (size_t)a.n_rows * a.heads + ids * a.heads + ids * a.heads * NP;
  const bool chunked = a.ws && a.n_rows >= 4 * SSD_CH && a.n_seg <= 16 && need <= a.ws_floats;
  // state rows per thread, a divisor of N out of 4 / 8 / 16 / 32 (branch-free loops), else 32 with bound checks: the smallest
  // when a segment is walked token by token (many threads per column hide the serial chain), the largest when the chunks
  // supply the parallelism (fewer partial sums to combine per token); the CTA's ~256 threads are NS row slices x PB columns
  int NR = 0;
  for (int c : {4, 8, 16, 32})
    if ((!NR || chunked) && a.N % c == 0 && a.N / c <= 64) NR = c;
  const bool exact = NR != 0;
  if (!exact) NR = SSD_NR;
  const int NS = (a.N + NR - 1) / NR;
  if (NS > 64) return cudaErrorInvalidValue;  // more than 32 x 64 state rows per column
  int PB = std::max(1, std::min(a.P, std::max(4, 256 / NS)));
  const size_t smem = ((size_t)2 * SSD_TOK * a.N + (size_t)SSD_TOK * PB + 2 * SSD_TOK + (size_t)SSD_TOK * NS * PB) * sizeof(float);
  if (smem > 160 * 1024) return cudaErrorInvalidValue;
  const dim3 block(PB * NS);
  const int colblocks = (a.P + PB - 1) / PB;
  auto go = [&](auto kern, const SsdArgs& args, int chunks) {
    if (smem > 48 * 1024) {
      cudaError_t r = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (r != cudaSuccess) return r;
    }
    return launch_k(kern, dim3(args.n_seg * chunks, args.heads, colblocks), block, smem, st, args, PB, NS, chunks);
  };
#define SSD_GO(MODE, args, chunks)                                                      \
  (!exact ? go(ssd_scan_kernel<SSD_NR, false, MODE>, args, chunks)                      \
          : NR == 4 ? go(ssd_scan_kernel<4, true, MODE>, args, chunks)                  \
          : NR == 8 ? go(ssd_scan_kernel<8, true, MODE>, args, chunks)                  \
          : NR == 16 ? go(ssd_scan_kernel<16, true, MODE>, args, chunks) : go(ssd_scan_kernel<32, true, MODE>, args, chunks))
  if (chunked) {
    SsdArgs c = a;
    c.ws_cum = a.ws;
    c.ws_p = c.ws_cum + (size_t)a.n_rows * a.heads;
    c.ws_state = c.ws_p + ids * a.heads;
    const int chunks = (a.n_rows + SSD_CH - 1) / SSD_CH;
    cudaError_t r = SSD_GO(1, c, chunks);
    if (r != cudaSuccess) return r;
    if ((r = launch_k(ssd_carry_kernel, dim3(a.n_seg, a.heads, (unsigned)((NP + 255) / 256)), dim3(256), 0, st, c)) != cudaSuccess) return r;
    return SSD_GO(2, c, chunks);
  }
  return SSD_GO(0, a, 1);
#undef SSD_GO
}

cudaError_t launch_gated_group_norm(const float* y, int ldy, const float* z, int ldz, const bf16* w, float* out, int ldo, int width, int groups,
                                    float eps, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  if (groups < 1 || width % groups) return cudaErrorInvalidValue;
  return launch_k(gated_group_norm_kernel, dim3(n, groups), dim3(256), 0, st, y, ldy, z, ldz, w, out, ldo, width / groups, eps);
}

cudaError_t launch_clamped_glu(const float* gu, int ld, float* out, int ff, float limit, float alpha, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const size_t total = (size_t)n * ff;
  const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 8);
  return launch_k(clamped_glu_kernel, dim3(blocks), dim3(256), 0, st, gu, ld, out, ff, limit, alpha, total);
}

}  // namespace qie
