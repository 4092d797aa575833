// ditenex.h -- the Ditenex model family: a decoder with learned position vectors whose sublayers sit between two RMS
// norms (x += m * norm_out(f(norm_in(x)))).  Every layer mixes by a grouped-query window attention whose scores carry a
// linear distance penalty per head and are mixed over the heads BEFORE the softmax ("talking heads"), whose values may
// be blended with the values of the first such layer, and whose output passes an elementwise sigmoid gate; the
// mixer reads a blend of its normed input with the previous token's (token shift, one carried row per layer and
// sequence).  The feed-forward is dense (xIELU activation), a mixture of experts (sigmoid router with a choice
// correction, group-limited top-k, unnormalised weights, always-on shared expert) or absent.  The logits reuse the
// embedding table.  Residual stream, norms, softmax, router and the carried rows are fp32.
//
// The mechanisms are launchers with their constants as arguments so that another design can use them: the norms and
// the token shift (rmsnorm_f32.cu), the activations (activations.cu), the router (moe_route.cuh), the query mixing, distance
// slopes, shared keys and elementwise gate of the paged attention (attn_gqa.cu, fosavik.h).  ditenex_model.cu holds the
// configuration reader, the weight loader and the launch order.  The family shares the engine's sequences, page
// allocator, block tables, row metadata, sampler, scheduler and C ABI with the other families (engine.h, family.h).
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

// ---------------------------------------------------------------- RMS norms around a sublayer, token shift (rmsnorm_f32.cu)
// rms(v) w = v / sqrt(mean(v^2) + eps) * w, fp32.  One CTA per row, both halves optional:
//   add  (y != null or mix.ye != null):  x[r] += mult * rms(y[r]) w_out      (y may be the mixture-of-experts combine
//                                        of the row, computed on the fly from `mix`; mix.z == null: shared expert ungated)
//   read (h != null):                    h[r] = rms(x[src(r)]) w_in,  src(r) = gather ? gather[r] : r
// Rider of the read half in front of a mixture of experts: the row's router logits z_e = w_router[e, :] . h (fp32, from the
// normed row while it is in shared memory) and the choice (moe_route.cuh), by the same CTA:
// s = sigmoid(z); choice score c = s + correction.  The experts form `groups` equal runs of neighbours; a group's score is
// the sum of its two largest c; only experts of the `keep` best groups can be chosen; the `top` largest c among them
// (lowest index first among equals) are chosen with weights s * scale (not renormalised).
struct RouteRider {
  const bf16* w_router = nullptr;  // [experts, width]; null: no rider
  const bf16* correction = nullptr;
  int experts = 0, top = 0, groups = 1, keep = 1;
  float scale = 1.f;
  int* top_idx = nullptr;  // [n, top]
  float* top_w = nullptr;
};
struct RmsStep {
  float* x = nullptr;
  int width = 0, n = 0;
  float eps = 0.f;
  const float* y = nullptr;
  MoeMix mix;
  const bf16* w_out = nullptr;
  float mult = 1.f;
  const bf16* w_in = nullptr;
  float* h = nullptr;
  const int* gather = nullptr;
  // bf16 rows around tensor-core GEMMs: y / the shared expert's output given as dense bf16 rows [n, width] (instead of y / mix.ys),
  // the normed row also (or only) written as dense bf16
  const bf16* y_bf = nullptr;
  const bf16* ys_bf = nullptr;
  bf16* h_bf = nullptr;
  RouteRider route;
};
cudaError_t launch_rms_step(const RmsStep& a, cudaStream_t st);
// Norm + token shift over the rows of each segment: h_t = rms(x_t) w;  out_t = h_t + (h_{t-1} - h_t) * mu, where the row
// before a segment's first is the carried row of its sequence slot (zeros for a new sequence); the carried row becomes
// the segment's last h.  carry of slot s: [width] fp32 at carry + s * slot_stride.
struct RmsShiftArgs {
  const float* x = nullptr;
  int width = 0, n = 0;
  float eps = 0.f;
  const bf16* w = nullptr;
  const bf16* mu = nullptr;  // [width]
  float* out = nullptr;
  bf16* out_bf = nullptr;  // optional dense bf16 copy [n, width] (the operand of a tensor-core GEMM)
  float* carry = nullptr;
  size_t slot_stride = 0;
  const int* seg_start = nullptr;
  const int* seg_slot = nullptr;
  int n_seg = 0;
};
cudaError_t launch_rms_shift(const RmsShiftArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- activations (activations.cu)
// in place over z[r, 0:cols]: xIELU with the two raw parameters pq[0], pq[1]:
//   z > 0: softplus(pq[0]) z^2 + z / 2;   z <= 0: (1/2 + softplus(pq[1])) (exp(z) - 1 - z) + z / 2
cudaError_t launch_xielu(float* z, int ld, int cols, const bf16* pq, int n, cudaStream_t st);
cudaError_t launch_xielu_bf16(bf16* z, int ld, int cols, const bf16* pq, int n, cudaStream_t st);  // bf16 rows, fp32 arithmetic
// out[r, c] = silu(gu[r, c]) * gu[r, ff + c]
cudaError_t launch_silu_glu(const float* gu, int ld, float* out, int ldo, int ff, int n, cudaStream_t st);
cudaError_t launch_silu_glu_bf16(const bf16* gu, int ld, bf16* out, int ldo, int ff, int n, cudaStream_t st);

// ---------------------------------------------------------------- the model (ditenex_model.cu)
struct DxLayer {
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0, window = 0;
  float scale = 1.f;
  bool v_mix = false;
  bool v_first = false;  // the first layer with v_mix: its values are kept for the later ones
  size_t kv_off = 0;     // elements into a page
  // feed-forward: kind 0 none, 1 dense, 2 mixture of experts
  int kind = 0, ff = 0;
  int experts = 0, top = 0, groups = 1, keep = 1, shared_ff = 0;
  float route_scale = 1.f;
  // weights (device)
  const bf16 *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr, *shift = nullptr;
  const bf16 *w_in = nullptr;  // q | k | v | g rows of one matrix
  const bf16 *q_b = nullptr, *k_b = nullptr, *v_b = nullptr, *vmix = nullptr, *talk = nullptr, *wo = nullptr;
  float* slopes = nullptr;  // [heads] fp32: the distance slopes after the head mixing
  const bf16 *w_up = nullptr, *w_down = nullptr, *act = nullptr;
  const bf16 *w_router = nullptr, *correction = nullptr, *w_egu = nullptr, *w_edown = nullptr, *w_sgu = nullptr, *w_sdown = nullptr;
};
struct DxModel : RowFamily {
  const char* family_name() const override { return "ditenex"; }
  cudaError_t forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) override;
  void reset_slot(qie_engine* e, int seq) override;
  void release() override;
  size_t layer_runs() const override { return layers.size(); }

  int max_positions = 0;
  float eps = 1e-6f, res_mult = 1.f;
  std::vector<DxLayer> layers;
  const bf16 *embed = nullptr, *pos_table = nullptr, *final_norm = nullptr;
  bf16* blob = nullptr;
  size_t blob_bytes = 0;
  float* slopes_all = nullptr;
  // paged key/value rows
  void* kv_pool = nullptr;
  size_t page_elems = 0;
  // carried rows of the token shift: slot s, layer l at carry + s * slot_floats + l * width
  float* carry = nullptr;
  size_t slot_floats = 0;
  // activations (fp32), sized by max_batch_tokens: x residual stream, hn normed sublayer input, y sublayer output,
  // p0 projections / hidden rows, p1 attention output, p2 mixed queries, vf first-layer values, top_w / top_idx router choice,
  // he / hg / ye expert rows grouped by expert, hs / ys shared expert, xo normed output rows
  float *x = nullptr, *hn = nullptr, *y = nullptr, *p0 = nullptr, *p1 = nullptr, *p2 = nullptr, *vf = nullptr, *top_w = nullptr;
  float *he = nullptr, *hg = nullptr, *ye = nullptr, *hs = nullptr, *ys = nullptr, *xo = nullptr;
  int *top_idx = nullptr, *grp_off = nullptr, *perm_row = nullptr, *slot_of = nullptr;
  int vf_width = 0;
  TcProjector tc;
  // bf16 rows between the producers and consumers of tensor-core GEMMs (bf16 precision): hb normed input, ub / ub2 hidden rows,
  // yb sublayer output, ysb shared expert output
  bf16 *hb = nullptr, *ub = nullptr, *ub2 = nullptr, *yb = nullptr, *ysb = nullptr;
  bf16* hgb = nullptr;  // gated hidden rows of the experts, grouped by expert
  float* attn_ws = nullptr;
  size_t attn_ws_floats = 0;
};

std::string ditenex_create(qie_engine* e, const std::string& dir, int* code);
std::string ditenex_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code);

}  // namespace qie
