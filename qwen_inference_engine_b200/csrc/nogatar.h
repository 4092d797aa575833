// nogatar.h -- the Nogatar model family: a decoder whose layers mix by latent (low-rank KV) attention with a
// sliding window and a softmax sink, or by the matrix-memory recurrence of xLSTM (mLSTM), followed by a
// mixture-of-experts feed-forward; the norm sits on each sublayer's OUTPUT and the residual stream is fp32.
// The mechanisms are separate launchers with their constants as arguments (ops_f32.cu, attn_latent.cu, mlstm.cu,
// moe.cu) so that another design can use them; nogatar_model.cu holds the configuration reader, the weight
// loader and the launch order.  The family shares the engine's sequences, page allocator, block tables, row
// metadata, sampler, scheduler and C ABI with the Qwen family (engine.h).
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "common.cuh"
#include "family.h"

struct qie_engine;

namespace qie {

// ---------------------------------------------------------------- generic fp32-stream operators (ops_f32.cu)
// C[m, n] = act(sum_k A[m, k] * W[n, k]); fp32 accumulation in ascending k, so a row's result does not depend
// on which other rows share the launch.  blockIdx.z walks `batches` problems whose operands are `*_batch`
// elements apart (per-head projections, experts).  With grp_off the rows of problem z are
// grp_off[z] .. grp_off[z+1]-1 of A / C (M is then the upper bound used for the grid) and row_idx, if given,
// names the source row of A for each of them (token gather of a mixture of experts).
struct GemmF32 {
  const float* A = nullptr;
  int lda = 0;
  long a_batch = 0;
  const bf16* W = nullptr;
  int ldw = 0;
  long w_batch = 0;
  int w_trans = 0;  // 1: W is stored [k, n] (row k, column n) instead of [n, k]
  float* C = nullptr;
  int ldc = 0;
  long c_batch = 0;
  int M = 0, N = 0, K = 0, batches = 1;
  const int* grp_off = nullptr;
  const int* row_idx = nullptr;
  const bf16* bias = nullptr;  // [N] added before the activation
  long bias_batch = 0;         // elements between the bias vectors of consecutive problems
  int act = 0;                 // 0 none, 1 relu(z)^2
  int round_a = 0;             // 1: A is rounded to bf16 before the product (bf16 serving precision)
  int round_c = 0;             // 1: the result is rounded to bf16 (still stored as fp32)
};
cudaError_t launch_gemm_f32(const GemmF32& g, cudaStream_t st);
// x[r, :] = table[ids[r], :] * scale
cudaError_t launch_embed_scale_f32(float* x, const bf16* table, const int* ids, int width, int n, float scale, cudaStream_t st);
// out[r, :] = (res ? res[r, :] : 0) + mult * LN(y[src(r), :]) * w, LN = (y - mean) / sqrt(mean((y - mean)^2) + eps);
// src(r) = gather ? gather[r] : r.  out may alias res.
// With `mix` (y == nullptr) the normed vector is the mixture-of-experts combine of row r, computed on the fly:
// sum_k top_w[r,k] * ye[slot_of[r,k]] (+ sigmoid(z[r, gate_col]) * ys[r]).
struct MoeMix {
  const float* ye = nullptr;
  const int* slot_of = nullptr;
  const float* top_w = nullptr;
  int top = 0;
  const float* ys = nullptr;
  const float* z = nullptr;
  int ldz = 0, gate_col = 0;
};
cudaError_t launch_layernorm_f32(const float* y, const bf16* w, float* out, const float* res, const int* gather, int width, int n,
                                 float eps, float mult, cudaStream_t st, const MoeMix& mix = MoeMix());
// z = cap * tanh(z / cap) in place
cudaError_t launch_softcap_f32(float* z, size_t n, float cap, cudaStream_t st);
cudaError_t launch_cast_f32_bf16(const float* in, bf16* out, size_t n, cudaStream_t st);
// operand / result conversion around a bf16 tensor-core GEMM: strided fp32 rows (optionally gathered) <-> dense bf16 rows
cudaError_t launch_rows_f32_to_bf16(const float* in, int ld_in, const int* row_idx, bf16* out, int cols, int n, cudaStream_t st);
cudaError_t launch_rows_bf16_to_f32(const bf16* in, int cols, float* out, int ld_out, int act, int n, cudaStream_t st);
// greedy choice over fp32 rows: out[r] = index of the largest value, the lowest index among equals
cudaError_t launch_argmax_f32(const float* z, int* out, int n_rows, int vocab, cudaStream_t st);

// ---------------------------------------------------------------- latent attention (attn_latent.cu)
// Paged latent cache: a page holds page_size positions of every attention layer; layer l's rows are `width`
// = kv_rank + rot_dim elements ([normed latent | rotated shared key]) starting `layer_off` elements into the page.
struct LatentCache {
  void* pool = nullptr;
  int elt_bytes = 4;  // 4: fp32 rows, 2: bf16 rows
  int page_size = 0;
  size_t page_elems = 0;  // elements per page over all layers
  size_t layer_off = 0;
  int rank = 0, rot = 0;  // width = rank + rot
};
// optional rider of launch_latent_store: rotary positions on src[r, h, 0:rot] -> dst[r, h, 0:rot] of the row's query heads
struct QueryRope {
  const float* src = nullptr;
  int ld_src = 0, hs_src = 0;
  float* dst = nullptr;
  int ld_dst = 0, hs_dst = 0, heads = 0;
};
// optional rider of launch_latent_store: dst[r, 0:width] = src[r, 0:width] / sqrt(mean(src^2) + eps) * w (fp32 rows and / or
// dense bf16 rows), the norm of a low-rank query latent that sits in the same projection output as the key/value latent
struct RowNorm {
  const float* src = nullptr;
  int ld_src = 0, width = 0;
  const bf16* w = nullptr;
  float* dst = nullptr;
  int ld_dst = 0;
  bf16* dst_bf = nullptr;
  int ld_dst_bf = 0;
};
// per row: latent = rms_unit(dkv[:rank]) * w_norm, key = rope(dkv[rank:], pos) -> cache row (slot, pos)
cudaError_t launch_latent_store(const LatentCache& c, const float* dkv, int ld, const bf16* w_norm, float eps, const RopeTable& rope,
                                const int* pos, const int* slot, const int* block_table, int max_pages, int n, cudaStream_t st,
                                const QueryRope& qr = QueryRope(), const RowNorm& qn = RowNorm());
// rotary positions on src[r, h, 0:rot] -> dst[r, h, 0:rot] (row strides ld_*, head strides hs_*)
cudaError_t launch_rope_heads_f32(const float* src, int ld_src, int hs_src, float* dst, int ld_dst, int hs_dst, int heads, int rot,
                                  const RopeTable& rope, const int* pos, int n, cudaStream_t st);
// out[r, h, 0:rank] = sum_j p_j * latent_j with p = softmax over the keys j of row r's sequence that satisfy
// max(0, pos - window + 1) <= j <= pos (window <= 0: all j <= pos) of (qa[r, h, :] . [latent_j | key_j]) * scale;
// with `sink` the denominator also holds exp(sink[h]).  qa rows are heads * (rank + rot), out rows heads * rank.
// max_keys bounds pos + 1 over the rows; with a workspace (ws, ws_floats) and few rows the keys of a row are split
// over several CTAs and combined (needs rows * heads * splits * (rank + 2) floats).
// With a head gate the result of (row, head) is multiplied by sigmoid(z[r, h] + bias[h]) (one number per head commutes with
// the value up-projection that follows, so it is applied to the attended latent).
struct HeadGate {
  const float* z = nullptr;  // [n, ld] pre-activations, head h at column h; null: no gate
  int ld = 0;
  const bf16* bias = nullptr;
};
cudaError_t launch_latent_attention(const LatentCache& c, const float* qa, float* out, const bf16* sink, float scale, int window, int heads,
                                    const int* pos, const int* slot, const int* block_table, int max_pages, int n, int max_keys, float* ws,
                                    size_t ws_floats, cudaStream_t st, const HeadGate& hg = HeadGate());

// ---------------------------------------------------------------- mLSTM (mlstm.cu)
// Recurrent state of one (sequence slot, layer), fp32: S [heads][dim][vdim], then n [heads][blocks][dim] and
// m [heads][blocks] with blocks = ceil(vdim / 32) (every 32-column block of S keeps its own copy of n and m).
struct MlstmArgs {
  const float* qkvg = nullptr;  // [n, 2*heads*dim + 2*heads*vdim]: q | k | v | output gate, head by head
  int ld = 0;
  float* gates = nullptr;  // [n, 2*heads]: input-gate and forget-gate pre-activations (bias added); overwritten by the log gates
  float* state = nullptr;        // slot s at state + s * slot_stride
  size_t slot_stride = 0;
  float* out = nullptr;  // [n, heads*vdim]
  const bf16* w_norm = nullptr;  // [heads*vdim]
  int heads = 0, dim = 0, vdim = 0;
  float gate_cap = 0.f, eps = 0.f;
  const int* seg_start = nullptr;  // [n_seg + 1] row ranges; rows of a segment are consecutive positions of one sequence
  const int* seg_slot = nullptr;   // [n_seg]
  int n_seg = 0;
  int n_rows = 0;  // rows of all segments
};
inline size_t mlstm_state_floats(int heads, int dim, int vdim) {
  return (size_t)heads * ((size_t)dim * vdim + (size_t)((vdim + 31) / 32) * (dim + 1));
}
cudaError_t launch_mlstm_scan(const MlstmArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- mixture of experts (moe.cu)
// route: scores = softmax(z[r, 0:experts]); the `top` largest (lowest index first among equals) with weights
// score / (sum of the chosen + 1e-20).  group: rows sorted by expert: grp_off[experts + 1], perm_row[n*top] (source
// row of each slot), slot_of[n*top] (slot of assignment (r, k)).  combine: y[r] = sum_k w[r,k] * ye[slot_of[r,k]]
// (+ sigmoid(z[r, gate_col]) * ys[r] with a shared expert).
cudaError_t launch_moe_route(const float* z, int ldz, int experts, int top, int* top_idx, float* top_w, int n, cudaStream_t st);
cudaError_t launch_moe_group(const int* top_idx, int n_assign, int top, int experts, int* grp_off, int* perm_row, int* slot_of, cudaStream_t st);
cudaError_t launch_moe_combine(const float* ye, const int* slot_of, const float* top_w, int top, const float* ys, const float* z, int ldz,
                               int gate_col, float* y, int width, int n, cudaStream_t st);

// Expert GEMMs on tensor cores over bf16 rows (gemm_grouped.cu): C[row, :] = A[src(row), :] W_z^T for the rows
// grp_off[z] .. grp_off[z + 1] - 1 of expert z, src(row) = row_idx ? row_idx[row] : row; W_z = W + z * w_batch, [N, K] row-major.
// gated: W_z = [gate rows | up rows] (N = 2 ff) and out_bf[row, c] = bf16(silu(gate_c) * up_c), c < ff; else out[row, n] fp32.
struct GroupedGemmBf16 {
  const bf16* A = nullptr;
  int lda = 0;
  const int* row_idx = nullptr;
  const int* grp_off = nullptr;
  const bf16* W = nullptr;
  long w_batch = 0;
  int N = 0, K = 0, groups = 0;
  int rows = 0;  // rows over all groups (bounds the grid)
  int gated = 0;
  float* out = nullptr;
  bf16* out_bf = nullptr;
  int ldo = 0;
};
bool grouped_gemm_bf16_fits(const GroupedGemmBf16& g);  // K a multiple of 32, 16-byte aligned rows
cudaError_t launch_grouped_gemm_bf16(const GroupedGemmBf16& g, cudaStream_t st);

// ---------------------------------------------------------------- the model (nogatar_model.cu)
typedef RotaryCfg NgRot;
struct NgLayer {
  int type = 0;  // 0 latent_attention, 1 mlstm
  // mixers
  int heads = 0, dim = 0, vdim = 0;
  int rot_dim = 0, kv_rank = 0, window = 0;  // latent attention (window 0 = none)
  float scale = 1.f;
  NgRot rot;
  int rope_id = -1;
  float gate_cap = 0.f;  // mlstm
  int state_id = -1, attn_id = -1;
  // feed-forward (experts 0 = none)
  int experts = 0, top = 0, ff = 0, shared_ff = 0;
  // weights (device)
  const bf16 *norm1 = nullptr, *norm2 = nullptr;
  const bf16 *wq = nullptr, *wdkv = nullptr, *dkv_norm = nullptr, *wuk = nullptr, *wuv = nullptr, *sink = nullptr, *wo = nullptr;
  const bf16 *wqkvg = nullptr, *wif = nullptr, *bif = nullptr, *out_norm = nullptr;
  const bf16 *w_up = nullptr, *w_down = nullptr, *w_router = nullptr, *w_sup = nullptr, *w_sdown = nullptr;
};
struct NgModel : RowFamily {
  const char* family_name() const override { return "nogatar"; }
  cudaError_t forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) override;
  void reset_slot(qie_engine* e, int seq) override;
  void release() override;
  size_t layer_runs() const override { return layers.size(); }

  float embed_scale = 1.f, eps = 1e-6f, res_mult = 1.f, softcap = 0.f;
  std::vector<NgLayer> layers;
  const bf16 *embed = nullptr, *final_norm = nullptr, *head = nullptr;
  bf16* blob = nullptr;
  size_t blob_bytes = 0;
  // rotary tables, one per distinct configuration
  std::vector<NgRot> rope_cfg;
  std::vector<float*> rope_cos, rope_sin;
  // latent cache
  void* lat_pool = nullptr;
  size_t page_elems = 0;
  std::vector<size_t> lat_off;  // per attention layer
  // recurrent state: slot s, mlstm layer j at state + s * slot_floats + state_off[j]
  float* state = nullptr;
  size_t slot_floats = 0;
  std::vector<size_t> state_off;
  // activations (fp32), sized by max_batch_tokens
  // x: residual stream, y: sublayer output, p0..p3: projections of the mixers, zr/top_*: router, he/ye: expert
  // hidden and output rows grouped by expert, hs/ys: shared expert, xo: normed output rows
  float *x = nullptr, *y = nullptr, *p0 = nullptr, *p1 = nullptr, *p2 = nullptr, *p3 = nullptr, *zr = nullptr, *top_w = nullptr;
  float *he = nullptr, *ye = nullptr, *hs = nullptr, *ys = nullptr, *xo = nullptr;
  int *top_idx = nullptr, *grp_off = nullptr, *perm_row = nullptr, *slot_of = nullptr;
  // bf16 serving precision, more than 16 rows: projections run on the tcgen05 GEMM between two conversion kernels
  TcProjector tc;
  float* attn_ws = nullptr;  // partial results of the key-split attention of small batches
  size_t attn_ws_floats = 0;
  int max_experts = 0;
};

// reads <dir>/config.json and <dir>/model.safetensors; fills e->ng and the engine's shared parts (page pool
// bookkeeping, block tables, row metadata).  Returns "" or the error text; *code receives the QIE_E* class.
std::string nogatar_create(qie_engine* e, const std::string& dir, int* code);
// same model over generated weights (bench / tests): cfg_json is the text of a config.json
std::string nogatar_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code);

}  // namespace qie
