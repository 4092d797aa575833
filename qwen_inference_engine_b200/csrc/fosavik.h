// fosavik.h -- the Fosavik model family: a decoder that carries several copies of the residual stream
// (hyper-connections: every sublayer reads a learned combination of the streams and writes back through a learned
// mixing matrix), whose layers mix by differential attention (two softmax maps over shared values, optionally over
// another layer's keys and values), by a gated window attention beside a gated linear recurrence (RG-LRU), or by
// the state-space recurrence of Mamba-2, followed by a clamped gated feed-forward.  The stream, norms, softmax and
// recurrent state are fp32.  The mechanisms are separate launchers with their constants as arguments (hyper.cu,
// attn_gqa.cu, recurrent.cu) so that another design can use them; fosavik_model.cu holds the configuration
// reader, the weight loader and the launch order.  The family shares the engine's sequences, page allocator, block
// tables, row metadata, sampler, scheduler and C ABI with the other families (engine.h, family.h).
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "common.cuh"
#include "family.h"

struct qie_engine;

namespace qie {

// ---------------------------------------------------------------- hyper-connections (hyper.cu)
// The streams of row r are X[r, s, :] (s < streams), fp32.
// X[r, s, :] = embed[ids[r], :] + pos_table[pos[r], :] for every s (pos_table may be null)
cudaError_t launch_embed_streams(float* X, const bf16* embed, const bf16* pos_table, const int* ids, const int* pos, int width, int streams,
                                 int n, cudaStream_t st);
// One step over the streams of every row, both halves optional:
//   write (y1 != null):  X'[t] = sum_s mix[s, t] X[s] + out[t] * (s1 * y1 + s2 * y2)      (all t at once from the old X)
//   read  (h != null):   u = sum_s in[s] X'[s]  (in == null: plain sum);  h = u / sqrt(mean(u^2) + eps) * w
//                        rows: src(r) = gather ? gather[r] : r;  sum_out (optional) receives u itself
// A sublayer's write and the next sublayer's read are one launch.
struct HyperStep {
  float* X = nullptr;
  int width = 0, streams = 0, n = 0;
  // write half
  const bf16* mix = nullptr;  // [streams, streams], indexed [from, to]
  const bf16* out = nullptr;  // [streams]
  const float* y1 = nullptr;
  const float* y2 = nullptr;
  float s1 = 1.f, s2 = 0.f;
  // read half
  const bf16* in = nullptr;  // [streams]
  const bf16* w = nullptr;   // [width] norm weight (null: no norm, h = u)
  float eps = 0.f;
  float* h = nullptr;
  float* sum_out = nullptr;
  const int* gather = nullptr;
};
cudaError_t launch_hyper_step(const HyperStep& a, cudaStream_t st);

// ---------------------------------------------------------------- grouped-query attention over paged rows (attn_gqa.cu)
// A page holds page_size positions of every caching layer; a layer's rows are [keys of all kv heads | values of all
// kv heads] = kw + vw elements, starting layer_off elements into the page.
struct KvRowCache {
  void* pool = nullptr;
  int elt_bytes = 4;  // 4: fp32 rows, 2: bf16 rows
  int page_size = 0;
  size_t page_elems = 0;  // elements per page over all layers
  size_t layer_off = 0;
  int kw = 0, vw = 0;
};
// per row: keys k[r, 0:kw] (optionally unit-RMS normed per `norm_dim` consecutive elements, times k_norm) and values
// v[r, 0:vw] -> cache row (slot, pos).  Rider: the row's queries q[r, 0:q_heads*norm_dim] normed in place with q_norm.
// Optional: biases added to keys and values first; values blended with another layer's values of the same rows,
// v = (1 - lam) v + lam v_other (lam one bf16 number on the device); the stored values also kept as fp32 rows (v_keep);
// the head-mixed queries of the row (TalkQueries below) written in the same launch.
// Rotary positions (rope.dims > 0): after the norm, the first rope.dims elements of every `norm_dim` consecutive elements
// of the keys and of the queries are rotated by the row's position (with two score maps every map of every head is such a
// group); q_bias is added to the queries before their norm.
// Mixing the heads' scores before the softmax, score'_h = sum_g talk[h, g] score_g, is linear in the queries: with
// qt[r, h, c * dim + e] = sum over the heads g of kv head c of talk[h, g] * (q[r, g, e] + q_bias[g * dim + e])
// head h's mixed score against key j is qt[r, h, :] . [keys of all kv heads of j] (GqaAttnArgs::shared_keys), and distance
// slopes mix the same way (slopes'_h = sum_g talk[h, g] slopes_g, a constant of the layer).  q_bias may be null.
struct TalkQueries {
  const float* q = nullptr;
  int ldq = 0;
  const bf16* q_bias = nullptr;
  const bf16* talk = nullptr;  // [heads, heads]; null: no rider
  float* qt = nullptr;
  int ldqt = 0, heads = 0, kv_heads = 0, dim = 0;
};
struct KvStoreArgs {
  KvRowCache c;
  const float* k = nullptr;
  int ldk = 0;
  const float* v = nullptr;
  int ldv = 0;
  const bf16* k_norm = nullptr;  // [norm_dim] or null
  int norm_dim = 0;
  float eps = 0.f;
  float* q = nullptr;
  int ldq = 0, q_heads = 0;
  const bf16* q_norm = nullptr;
  const bf16* k_bias = nullptr;  // [kw]
  const bf16* v_bias = nullptr;  // [vw]
  const bf16* q_bias = nullptr;  // [q_heads * norm_dim]
  RopeTable rope;
  const bf16* v_lam = nullptr;
  const float* v_other = nullptr;
  int ld_vo = 0;
  float* v_keep = nullptr;
  int ld_vk = 0;
  TalkQueries tq;
  const int *pos = nullptr, *slot = nullptr, *block_table = nullptr;
  int max_pages = 0, n = 0;
};
cudaError_t launch_kv_store_rows(const KvStoreArgs& a, cudaStream_t st);
// out[r, h, :] over the keys j of row r's sequence with j <= pos and (window <= 0 or pos - j < window or j < keep_first).
// `maps` score maps per head (queries [h][map][dim], keys [g][map][dim]) share the values [g][vdim]; head h reads kv
// head h / (heads / kv_heads).  unit_sink adds 1 to every softmax denominator (as if one more key with a zero score and nothing to contribute took part).
// finish 0: out = a_1;  1: out = a_1 * sigmoid(gate[r, h]);  2 (maps == 2): o = a_1 - lam * a_2, out = o / sqrt(mean(o^2) + eps) * post;
// 3: out[r, h, c] = a_1[c] * sigmoid(gate[r, h * vdim + c]) (a gate per element).
// softcap > 0: the scaled score s becomes softcap * tanh(s / softcap) before the mask, the slopes and the softmax.
// slopes (optional, [heads] fp32): slopes[h] * (pos - j) is taken off the scaled score of key j (a linear distance penalty).
// shared_keys: every head scores against the WHOLE key part of the cached row (dim = kw / maps elements: the keys of all
// kv heads side by side) while its values stay those of kv head h / (heads / kv_heads); the queries are then
// [h][map][kw / maps] (TalkQueries builds them).
// The keys of a row may be split over CTAs; partial (max, sum, acc) go through ws and a second kernel finishes.
struct GqaAttnArgs {
  KvRowCache c;
  const float* q = nullptr;
  int ldq = 0;
  float* out = nullptr;
  int ldo = 0;
  bf16* out_bf = nullptr;  // the result goes here as bf16 rows (row stride ldo_bf) instead of `out` (two maps: `out` is still needed as scratch)
  int ldo_bf = 0;
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, maps = 1;
  float scale = 1.f, softcap = 0.f;
  int window = 0, keep_first = 0, unit_sink = 0;
  int finish = 0;
  const float* gate = nullptr;
  int ldg = 0;
  const float* slopes = nullptr;
  int shared_keys = 0;
  float lam = 0.f, post = 1.f, eps = 0.f;
  const int *pos = nullptr, *slot = nullptr, *block_table = nullptr;
  int max_pages = 0, n = 0, max_keys = 0;
  float* ws = nullptr;
  size_t ws_floats = 0;
  int num_sms = 148;
  // segments of the batch (runs of consecutive rows of one sequence, [n_seg + 1] row bounds and [n_seg] slots): with
  // them, 64 rows or more and a bf16 cache the rows run 64 at a time on tensor cores
  const int* seg_start = nullptr;
  const int* seg_slot = nullptr;
  int n_seg = 0;
};
// floats of workspace that n rows need with one split
inline size_t gqa_ws_floats(int n, int heads, int maps, int vdim) { return (size_t)n * heads * maps * (vdim + 2); }
cudaError_t launch_gqa_attention(const GqaAttnArgs& a, cudaStream_t st, int* n_launches = nullptr);

// ---------------------------------------------------------------- short convolution and recurrences (recurrent.cu)
// Causal per-channel convolution over the rows of each segment: out[t, c] = act(b[c] + sum_i w[c, i] * in(t - (taps-1-i), c)),
// in(t, c) = x[t, c] + in_bias[c] for rows of the segment, the carried tail for the taps-1 positions before it (zeros
// before the start of the sequence).  tail of slot s: [taps-1, channels] fp32 at tail + s * slot_stride, oldest first;
// it is updated to the segment's last inputs by a second kernel.
struct ConvArgs {
  const float* x = nullptr;
  int ldx = 0;
  const bf16* in_bias = nullptr;  // [channels] or null
  const bf16* w = nullptr;        // [channels, taps]
  const bf16* b = nullptr;        // [channels]
  int channels = 0, taps = 0;
  int act = 0;  // 0 none, 1 silu
  float* out = nullptr;
  int ldo = 0;
  float* tail = nullptr;
  size_t slot_stride = 0;
  const int* seg_start = nullptr;
  const int* seg_slot = nullptr;
  int n_seg = 0, n_rows = 0;
};
cudaError_t launch_causal_conv(const ConvArgs& a, cudaStream_t st);
// Real-gated linear recurrence per channel c over the rows of each segment:
//   r = sigmoid(zr), i = sigmoid(zi), a = exp(-decay_c * r * softplus(lam[c])), S = a S + sqrt(1 - a^2) * i * u,
//   out = S * gelu_tanh(yb[t, c] + y_bias[c]).   state of slot s: [channels] fp32 at state + s * slot_stride.
struct LruArgs {
  const float* zr = nullptr;  // [n, channels] gate pre-activations (bias added); overwritten when the chunked form runs
  const float* zi = nullptr;
  int ldz = 0;
  const float* u = nullptr;
  int ldu = 0;
  const float* yb = nullptr;
  int ldy = 0;
  const bf16* y_bias = nullptr;
  const bf16* lam = nullptr;
  float decay_c = 8.f;
  int channels = 0;
  float* out = nullptr;
  int ldo = 0;
  float* state = nullptr;
  size_t slot_stride = 0;
  const int* seg_start = nullptr;
  const int* seg_slot = nullptr;
  int n_seg = 0, n_rows = 0;
  // optional workspace of (n_rows / 64 + n_seg + 2) * 2 * channels floats: with it, portions of 256 rows and more in at
  // most 64 segments run chunk-parallel (local scans, a carry pass, an apply pass)
  float* ws = nullptr;
  size_t ws_floats = 0;
};
cudaError_t launch_lru_scan(const LruArgs& a, cudaStream_t st);
// State-space recurrence per head (state S [N, P] fp32 per head and slot):
//   dt = softplus(dt_raw[t, h] + dt_bias[h]);  S = exp(-exp(A_log[h]) dt) S + dt * B_t x_t^T;  y_t = S^T C_t + D[h] x_t
// x [n, heads*P], B and C [n, groups*N] (head h reads group h / (heads / groups)).
struct SsdArgs {
  const float* x = nullptr;
  const float* B = nullptr;
  const float* C = nullptr;
  int ld = 0;  // row stride of x, B, C (they are parts of one buffer)
  const float* dt_raw = nullptr;
  int ld_dt = 0;
  const bf16 *dt_bias = nullptr, *A_log = nullptr, *D = nullptr;
  int heads = 0, P = 0, N = 0, groups = 1;
  float* y = nullptr;
  int ldy = 0;
  float* state = nullptr;  // slot s: [heads, N, P] at state + s * slot_stride
  size_t slot_stride = 0;
  const int* seg_start = nullptr;
  const int* seg_slot = nullptr;
  int n_seg = 0, n_rows = 0;
  // optional workspace (ssd_ws_floats): with it, portions of 256 rows and more in at most 16 segments run chunk-parallel
  float* ws = nullptr;
  size_t ws_floats = 0;
  float *ws_cum = nullptr, *ws_p = nullptr, *ws_state = nullptr;  // set by the launcher: parts of ws
};
inline size_t ssd_ws_floats(size_t rows, int heads, int N, int P) {
  const size_t ids = rows / 64 + 16 + 2;
  return rows * heads + ids * heads + ids * heads * (size_t)N * P;
}
cudaError_t launch_ssd_scan(const SsdArgs& a, cudaStream_t st);
// out[r, c] = v / sqrt(mean_group(v^2) + eps) * w[c] with v = y[r, c] * silu(z[r, c]); `groups` equal parts of `width`
cudaError_t launch_gated_group_norm(const float* y, int ldy, const float* z, int ldz, const bf16* w, float* out, int ldo, int width, int groups,
                                    float eps, int n, cudaStream_t st);
// out[r, c] = g * sigmoid(alpha * g) * (u + 1), g = min(gu[r, c], limit), u = clamp(gu[r, ff + c], -limit, limit)
cudaError_t launch_clamped_glu(const float* gu, int ld, float* out, int ff, float limit, float alpha, int n, cudaStream_t st);

// ---------------------------------------------------------------- the model (fosavik_model.cu)
struct FvAttn {  // one attention: the differential mixer, or the left half of the parallel mixer
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, maps = 1;
  float scale = 1.f;
  int window = 0, keep_first = 0;
  int cache_id = -1;  // index into FvModel::kv_off (the layer's own rows, or those of the layer it reads)
  bool own_kv = true;
};
struct FvLayer {
  int type = 0;  // 0 attention (differential), 1 parallel (window attention + linear recurrence), 2 mamba2
  FvAttn at;
  float diff = 0.f, lam = 0.f;  // differential attention: lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, worked out at load time
  int kv_from = -1;
  // parallel: right half
  float left_scale = 1.f, right_scale = 1.f;
  int lru_width = 0, lru_blocks = 1, lru_taps = 0;
  // mamba2
  int m_heads = 0, m_P = 0, m_N = 0, m_groups = 1, m_norm_groups = 1, m_taps = 0;
  size_t state_off = 0;  // floats into a slot's state: [recurrent state | convolution tail]
  // feed-forward (ff 0 = none)
  int ff = 0;
  float limit = 0.f;
  // weights (device)
  const bf16 *norm1 = nullptr, *norm2 = nullptr;
  const bf16 *hc1_in = nullptr, *hc1_out = nullptr, *hc1_mix = nullptr, *hc2_in = nullptr, *hc2_out = nullptr, *hc2_mix = nullptr;
  const bf16 *w_in = nullptr;  // the mixer's input projections, one matrix
  const bf16 *q_norm = nullptr, *k_norm = nullptr, *wo = nullptr;
  const bf16 *y_b = nullptr, *x_b = nullptr, *conv_w = nullptr, *conv_b = nullptr, *ra = nullptr, *ra_b = nullptr, *ri = nullptr, *ri_b = nullptr,
             *lam_w = nullptr, *wo2 = nullptr;
  const bf16 *dt_bias = nullptr, *A_log = nullptr, *Dw = nullptr, *gn_w = nullptr;
  const bf16 *w_gu = nullptr, *w_down = nullptr;
};
struct FvModel : RowFamily {
  const char* family_name() const override { return "fosavik"; }
  cudaError_t forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) override;
  void reset_slot(qie_engine* e, int seq) override;
  void release() override;
  size_t layer_runs() const override { return layers.size(); }

  int streams = 1, max_positions = 0;
  float eps = 1e-6f;
  std::vector<FvLayer> layers;
  const bf16 *embed = nullptr, *pos_table = nullptr, *final_norm = nullptr, *head = nullptr;
  bf16* blob = nullptr;
  size_t blob_bytes = 0;
  // paged key/value rows
  void* kv_pool = nullptr;
  size_t page_elems = 0;
  std::vector<size_t> kv_off;  // per caching layer
  // recurrent state: slot s at state + s * slot_floats
  float* state = nullptr;
  size_t slot_floats = 0;
  // activations (fp32), sized by max_batch_tokens: X streams, hn normed sublayer input, y / y2 sublayer outputs,
  // p0..p3 projections and intermediates, xo normed output rows
  float *X = nullptr, *hn = nullptr, *y = nullptr, *y2 = nullptr, *p0 = nullptr, *p1 = nullptr, *p2 = nullptr, *p3 = nullptr, *xo = nullptr;
  TcProjector tc;
  float* attn_ws = nullptr;
  size_t attn_ws_floats = 0;
  float* scan_ws = nullptr;  // chunk summaries of the chunk-parallel linear recurrence
  size_t scan_ws_floats = 0;
};

std::string fosavik_create(qie_engine* e, const std::string& dir, int* code);
std::string fosavik_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code);

}  // namespace qie
