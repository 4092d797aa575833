// dedunex.h -- the Dedunex model family: a decoder with one fp32 residual stream whose layers are PARALLEL blocks:
// one grouped RMS norm feeds both the mixer and the gated feed-forward, and both outputs are added to the stream,
// x += mixer(h) + ff(h) with h = norm(x).  A run of consecutive layers may be repeated (a loop: the same weights, a
// cache / state of its own per pass, a learned vector added to the stream before each pass).  A layer's mixer is one of
//  * differential attention with grouped-query heads over a sliding window: two softmax maps per head over the same
//    values, queries and keys with biases, a per-head RMS norm with a shared weight, partial rotary positions in the
//    "rotate half" pairing with optionally YaRN-blended frequencies, and tanh soft-capped scores;
//  * latent attention: queries through a normed low-rank bottleneck, one cached row [normed latent | rotated shared key]
//    per position for all heads, causal, a sigmoid output gate per head;
//  * minGRU: S_t = (1 - z_t) S_(t-1) + z_t c_t per channel with gates that read only the current token, an fp32 state per
//    sequence, and a SiLU output gate.
// The feed-forward is W_down (gelu_tanh(W_gate h) * (W_up h)).  Residual, norms, scores, softmax, rotary angles, the
// recurrence and its gates are fp32.
//
// New mechanisms are launchers with their constants as arguments, beside the ones they resemble: the grouped norm step
// (rmsnorm_f32.cu), the gated activation (activations.cu), the minGRU scan (recurrent.cu); rotary positions and query
// biases of the key/value store and the score soft cap (attn_gqa.cu), the pairing of rotated dimensions, the query-latent
// norm and the head gate of the latent attention (attn_latent.cu) are options of the existing launchers.
// dedunex_model.cu holds the configuration reader, the weight loader and the launch order.  The family shares the
// engine's sequences, page allocator, block tables, row metadata, sampler, scheduler and C ABI with the other families.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "common.cuh"
#include "family.h"
#include "fosavik.h"
#include "nogatar.h"

struct qie_engine;

namespace qie {

// ---------------------------------------------------------------- grouped RMS norm around a parallel block (rmsnorm_f32.cu)
// gnorm(v) w: v is split into `groups` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps), the
// whole multiplied by w.  One CTA per row r, src(r) = gather ? gather[r] : r, in this order (every part optional):
//   source  x[src] as it is, or (ids != null) gnorm(embed[ids[r]]) w_pre : the first norm of a model that norms its embedding
//   add     x[src] += y1[src] + y2[src]       the two sublayer outputs of the block before (fp32 or dense bf16 rows)
//   dump    dump[r] = x[src]                  the stream after a layer, for the parity hook
//   step    x[src] += step                    a vector of the model (before a pass of a loop)
//   read    h[r] = gnorm(x[src]) w_in         fp32 rows and / or dense bf16 rows
// x[src] is written back when it changed.
struct GroupNormStep {
  float* x = nullptr;
  int width = 0, groups = 1, n = 0;
  float eps = 0.f;
  const int* ids = nullptr;
  const bf16* embed = nullptr;
  const bf16* w_pre = nullptr;
  const float* y1 = nullptr;
  const float* y2 = nullptr;
  const bf16* y1_bf = nullptr;
  const bf16* y2_bf = nullptr;
  float* dump = nullptr;
  const bf16* step = nullptr;
  const bf16* w_in = nullptr;
  float* h = nullptr;
  bf16* h_bf = nullptr;
  const int* gather = nullptr;
};
cudaError_t launch_group_norm_step(const GroupNormStep& a, cudaStream_t st);

// ---------------------------------------------------------------- gated activation (activations.cu)
// out[r, c] = act(g[r, c]) * u[r, c], c < ff; act 0: silu, 1: gelu in its tanh form.  g and u are columns of fp32 rows
// (row stride ld) or of bf16 rows (g_bf / u_bf, row stride ld_bf); the result goes to fp32 rows and / or bf16 rows.
struct GatedAct {
  const float* g = nullptr;
  const float* u = nullptr;
  int ld = 0;
  const bf16* g_bf = nullptr;
  const bf16* u_bf = nullptr;
  int ld_bf = 0;
  float* out = nullptr;
  int ldo = 0;
  bf16* out_bf = nullptr;
  int ldo_bf = 0;
  int ff = 0, act = 0, n = 0;
};
cudaError_t launch_gated_act(const GatedAct& a, cudaStream_t st);

// ---------------------------------------------------------------- minGRU (recurrent.cu)
// Per channel c over the rows of each segment, state S of slot s at state[s * slot_stride + c] (fp32, carried):
//   z = sigmoid(zp[t, c] + z_bias[c]);  u = up[t, c] + u_bias[c];  cand = u >= 0 ? u + 1/2 : sigmoid(u)
//   S = (1 - z) S + z cand;   out[t, c] = S * silu(gp[t, c])
// zp, up, gp are columns of fp32 rows (row stride ld) or of bf16 rows (*_bf, ld_bf).  With a workspace of
// mingru_ws_floats() long portions run chunk-parallel (local scans from a zero state, a carry pass, an apply pass).
struct MinGruArgs {
  const float *zp = nullptr, *up = nullptr, *gp = nullptr;
  int ld = 0;
  const bf16 *zp_bf = nullptr, *up_bf = nullptr, *gp_bf = nullptr;
  int ld_bf = 0;
  const bf16* z_bias = nullptr;
  const bf16* u_bias = nullptr;
  int channels = 0;
  float* out = nullptr;
  int ldo = 0;
  bf16* out_bf = nullptr;
  int ldo_bf = 0;
  float* state = nullptr;
  size_t slot_stride = 0;
  const int* seg_start = nullptr;
  const int* seg_slot = nullptr;
  int n_seg = 0, n_rows = 0;
  float* ws = nullptr;
  size_t ws_floats = 0;
};
inline size_t mingru_ws_floats(size_t rows, size_t segs, int channels) { return (2 * rows + (rows / 64 + segs + 2) * 2) * (size_t)channels; }
cudaError_t launch_mingru_scan(const MinGruArgs& a, cudaStream_t st);

// dense bf16 rows with a row stride -> fp32 rows (ops_f32.cu)
cudaError_t launch_rows_bf16_to_f32_ld(const bf16* in, int ld_in, int cols, float* out, int ld_out, int n, cudaStream_t st);

// ---------------------------------------------------------------- the model (dedunex_model.cu)
struct DdLayer {
  int type = 0;  // 0 attention (differential), 1 latent_attention, 2 mingru
  // attention / latent attention
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, window = 0;
  float scale = 1.f, softcap = 0.f, diff = 0.f, lam = 0.f;
  int rot_dim = 0, kv_rank = 0, q_rank = 0;
  RotaryCfg rot;
  int rope_id = -1;
  // mingru
  int gru_width = 0;
  // feed-forward (ff 0 = none)
  int ff = 0;
  // the input projection [mixer parts | gate | up] as one matrix: column offsets of its parts and its width (parts start
  // at multiples of 8 columns; the columns between them are zero rows of the matrix)
  int o_a = 0, o_b = 0, o_c = 0, o_gate = 0, o_up = 0, n_in = 0;
  // weights (device)
  const bf16 *norm1 = nullptr, *w_in = nullptr, *wo = nullptr, *w_down = nullptr;
  const bf16 *q_b = nullptr, *k_b = nullptr, *v_b = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  const bf16 *dq_norm = nullptr, *dkv_norm = nullptr, *wuq = nullptr, *wuk = nullptr, *wuv = nullptr;
  const bf16 *z_b = nullptr, *x_b = nullptr;
};
// one execution of a layer: a layer inside the loop runs `times` times, each with its own cache rows / state
struct DdRun {
  int layer = 0;
  int pass = -1;        // >= 0: the first layer of this pass of the loop (the pass vector is added in front of it)
  size_t kv_off = 0;    // elements into a page (attention, latent attention)
  size_t state_off = 0; // floats into a slot's state (mingru)
};
struct DdModel : RowFamily {
  const char* family_name() const override { return "dedunex"; }
  cudaError_t forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) override;
  void reset_slot(qie_engine* e, int seq) override;
  void release() override;
  size_t layer_runs() const override { return runs.size(); }

  float eps = 1e-6f;
  int groups = 1;
  int loop_start = 0, loop_stop = 0, loop_times = 1;
  std::vector<DdLayer> layers;
  std::vector<DdRun> runs;
  const bf16 *embed = nullptr, *embed_norm = nullptr, *loop_step = nullptr, *final_norm = nullptr, *head = nullptr;
  bf16* blob = nullptr;
  size_t blob_bytes = 0;
  std::vector<RotaryCfg> rope_cfg;
  std::vector<float*> rope_cos, rope_sin;
  // one page pool for the key/value rows and the latent rows of every caching run
  void* kv_pool = nullptr;
  size_t page_elems = 0;
  // recurrent state: slot s at state + s * slot_floats
  float* state = nullptr;
  size_t slot_floats = 0;
  // activations (fp32), sized by max_batch_tokens: x residual stream, hn normed input, p0 input projection, p1 / p2 / p3
  // mixer intermediates, y1 / y2 the two sublayer outputs, xo normed output rows
  float *x = nullptr, *hn = nullptr, *p0 = nullptr, *p1 = nullptr, *p2 = nullptr, *p3 = nullptr, *y1 = nullptr, *y2 = nullptr, *xo = nullptr;
  TcProjector tc;
  // bf16 rows between the producers and consumers of tensor-core GEMMs: hb normed input, mb mixer output, fb feed-forward
  // hidden rows, qb normed query latent, y1b / y2b sublayer outputs
  bf16 *hb = nullptr, *mb = nullptr, *fb = nullptr, *qb = nullptr, *y1b = nullptr, *y2b = nullptr;
  float* attn_ws = nullptr;
  size_t attn_ws_floats = 0;
  float* scan_ws = nullptr;
  size_t scan_ws_floats = 0;
};

std::string dedunex_create(qie_engine* e, const std::string& dir, int* code);
std::string dedunex_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code);

}  // namespace qie
