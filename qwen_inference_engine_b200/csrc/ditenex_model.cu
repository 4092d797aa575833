// ditenex_model.cu -- the Ditenex family on the engine: configuration reader (config.json), weight loader
// (model.safetensors -> one device blob), the paged key/value rows and the carried rows of the token shift, and the
// launch order of one forward over a batch of rows.  A row is (sequence slot, position) exactly as in the other
// families; rows of one sequence are consecutive and in position order, rows of different sequences may be portions of
// prompts next to single decoded tokens.  Every size and constant comes from the configuration.
#include "ditenex.h"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>

#include "engine.h"
#include "json_min.h"
#include "launch.h"

namespace qie {
namespace {

#define NEED(cond, msg)      \
  do {                       \
    if (!(cond)) return msg; \
  } while (0)

int as_int(const JsonValue* v, int dflt) { return v && v->is_number() ? (int)llround(v->num) : dflt; }
float as_float(const JsonValue* v, float dflt) { return v && v->is_number() ? (float)v->num : dflt; }
bool present(const JsonValue* v) { return v && v->kind != JsonValue::Null; }
bool as_bool(const JsonValue* v) { return v && ((v->kind == JsonValue::Bool && v->b) || (v->is_number() && v->num != 0.0)); }

std::string parse_config(const JsonValue& root, DxModel* m) {
  NEED(root.kind == JsonValue::Object, "config.json: not an object");
  m->vocab = as_int(root.have("vocab"), 0);
  m->width = as_int(root.have("width"), 0);
  m->max_positions = as_int(root.have("max_positions"), 0);
  NEED(m->vocab > 0 && m->width > 0, "config.json: vocab / width missing");
  NEED(m->max_positions > 0, "config.json: max_positions missing");
  if (const JsonValue* nm = root.have("norm")) m->eps = as_float(nm->have("eps"), 1e-6f);
  m->res_mult = as_float(root.have("residual_mult"), 1.0f);
  const JsonValue* layers = root.have("layers");
  NEED(layers && layers->kind == JsonValue::Array && !layers->arr.empty(), "config.json: layers missing");
  bool seen_vmix = false;
  int vw_first = 0;
  for (const JsonValue& jl : layers->arr) {
    DxLayer L;
    const JsonValue* type = jl.have("type");
    const JsonValue* mx = jl.have("mixer");
    NEED(type && type->kind == JsonValue::String && mx && mx->kind == JsonValue::Object, "config.json: layer without type / mixer");
    NEED(type->str == "attention", "config.json: unknown layer type '" + type->str + "'");
    L.heads = as_int(mx->have("heads"), 0);
    L.kv_heads = as_int(mx->have("kv_heads"), L.heads);
    L.dim = as_int(mx->have("dim"), 0);
    L.vdim = as_int(mx->have("vdim"), L.dim);
    NEED(L.heads > 0 && L.kv_heads > 0 && L.dim > 0 && L.vdim > 0, "config.json: attention heads / kv_heads / dim / vdim missing");
    NEED(L.heads % L.kv_heads == 0, "config.json: heads must be a multiple of kv_heads");
    NEED(mx->have("scale") && mx->have("scale")->is_number(), "config.json: attention without scale");
    L.scale = (float)mx->have("scale")->num;
    if (const JsonValue* mk = mx->have("mask"))
      if (present(mk)) L.window = as_int(mk->have("size"), 0);
    L.v_mix = as_bool(mx->have("v_mix"));
    if (L.v_mix) {
      if (!seen_vmix) L.v_first = true, seen_vmix = true, vw_first = L.kv_heads * L.vdim;
      else NEED(L.kv_heads * L.vdim == vw_first, "config.json: layers that blend values must have equal value widths");
    }
    if (const JsonValue* mlp = jl.have("mlp"))
      if (present(mlp)) {
        const JsonValue* kind = mlp->have("kind");
        NEED(kind && kind->kind == JsonValue::String, "config.json: mlp without kind");
        if (kind->str == "dense") {
          L.kind = 1;
          L.ff = as_int(mlp->have("ff"), 0);
          NEED(L.ff > 0, "config.json: dense mlp without ff");
        } else if (kind->str == "moe") {
          L.kind = 2;
          const JsonValue* ex = mlp->have("expert");
          const JsonValue* rt = mlp->have("router");
          NEED(ex && rt, "config.json: moe mlp without expert / router");
          L.ff = as_int(ex->have("ff"), 0);
          L.experts = as_int(rt->have("experts"), 0);
          L.top = as_int(rt->have("top"), 0);
          L.route_scale = as_float(rt->have("scale"), 1.0f);
          if (const JsonValue* g = rt->have("groups"))
            if (present(g)) {
              L.groups = as_int(g->have("count"), 1);
              L.keep = as_int(g->have("keep"), L.groups);
            }
          NEED(L.ff > 0 && L.experts > 0 && L.top > 0 && L.top <= L.experts, "config.json: moe ff / experts / top");
          NEED(L.groups > 0 && L.experts % L.groups == 0 && L.keep > 0 && L.keep <= L.groups, "config.json: expert groups must divide the experts");
          NEED((long)L.keep * (L.experts / L.groups) >= L.top, "config.json: the kept groups hold fewer experts than are chosen");
          if (const JsonValue* sh = mlp->have("shared"))
            if (present(sh)) L.shared_ff = as_int(sh->have("ff"), 0);
        } else {
          return "config.json: unknown mlp kind '" + kind->str + "'";
        }
      }
    m->layers.push_back(L);
  }
  return "";
}

// tensors in blob order; tensors that one GEMM reads as a single matrix are adjacent (no padding between them)
std::vector<TensorSpec> build_layout(const DxModel& m) {
  BlobLayout bl;
  auto pad = [&]() { bl.pad(); };
  auto add = [&](const std::string& name, size_t rows, size_t cols, int kind) { bl.add(name, rows, cols, kind); };
  const size_t W = m.width;
  pad(), add("embed", m.vocab, W, 0);
  pad(), add("pos", m.max_positions, W, 2);
  for (size_t i = 0; i < m.layers.size(); ++i) {
    const DxLayer& L = m.layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const size_t H = L.heads, G = L.kv_heads, d = L.dim, vd = L.vdim;
    pad(), add(p + "norm1", W, 0, 1);
    pad(), add(p + "norm1b", W, 0, 1);
    pad(), add(p + "shift", W, 0, 2);
    pad(), add(p + "mix.q", H * d, W, 0), add(p + "mix.k", G * d, W, 0), add(p + "mix.v", G * vd, W, 0), add(p + "mix.g", H * vd, W, 0);
    pad(), add(p + "mix.q.b", H * d, 0, 2);
    pad(), add(p + "mix.k.b", G * d, 0, 2);
    pad(), add(p + "mix.v.b", G * vd, 0, 2);
    pad(), add(p + "mix.vmix", 1, 0, 2);
    pad(), add(p + "mix.talk", H, H, 0);
    pad(), add(p + "mix.o", W, H * vd, 0);
    if (L.kind == 0) continue;
    pad(), add(p + "norm2", W, 0, 1);
    pad(), add(p + "norm2b", W, 0, 1);
    if (L.kind == 1) {
      pad(), add(p + "mlp.up", L.ff, W, 0);
      pad(), add(p + "mlp.down", W, L.ff, 0);
      pad(), add(p + "mlp.act", 2, 0, 2);
    } else {
      pad(), add(p + "mlp.router", L.experts, W, 0);
      pad(), add(p + "mlp.correction", L.experts, 0, 2);
      pad();
      for (int e = 0; e < L.experts; ++e) {
        const std::string q = p + "mlp.e" + std::to_string(e) + ".";
        add(q + "gate", L.ff, W, 0), add(q + "up", L.ff, W, 0);
      }
      pad();
      for (int e = 0; e < L.experts; ++e) add(p + "mlp.e" + std::to_string(e) + ".down", W, L.ff, 0);
      if (L.shared_ff > 0) {
        pad(), add(p + "mlp.shared.gate", L.shared_ff, W, 0), add(p + "mlp.shared.up", L.shared_ff, W, 0);
        pad(), add(p + "mlp.shared.down", W, L.shared_ff, 0);
      }
    }
  }
  pad(), add("final.norm", W, 0, 1);
  return bl.t;
}

float bits_to_float(uint16_t b) {
  const uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

#define CUS(expr)                                                      \
  do {                                                                 \
    cudaError_t _e = (expr);                                           \
    if (_e != cudaSuccess) {                                           \
      *code = QIE_ECUDA;                                               \
      return std::string(#expr) + ": " + cudaGetErrorString(_e);       \
    }                                                                  \
  } while (0)

std::string finish_setup(qie_engine* e, const std::vector<TensorSpec>& t, const std::vector<uint16_t>& blob, int* code) {
  DxModel* m = e->dx;
  const qie_engine_opts& o = e->opts;
  // a sequence cannot grow beyond the learned position vectors, whatever the pool holds
  const int context = std::min(o.context, m->max_positions);
  m->f32 = o.compute_dtype == QIE_DTYPE_F32;
  m->blob_bytes = blob.size() * 2;
  CUS(cudaMalloc(&m->blob, m->blob_bytes));
  CUS(cudaMemcpy(m->blob, blob.data(), m->blob_bytes, cudaMemcpyHostToDevice));
  std::map<std::string, const TensorSpec*> at;
  for (const TensorSpec& s : t) at[s.name] = &s;
  auto P = [&](const std::string& n) -> const bf16* {
    auto it = at.find(n);
    return it == at.end() ? nullptr : m->blob + it->second->off;
  };
  m->embed = P("embed");
  m->pos_table = P("pos");
  m->final_norm = P("final.norm");
  e->cfg = qie_config{m->width, 0, (int)m->layers.size(), 0, 0, 0, m->vocab, context};
  size_t page_elems = 0, total_heads = 0;
  size_t w0 = 1, w1 = 1, w2 = 1, hmv = 1, maxk = m->width, maxn = m->width;
  size_t w_top = 1, w_he = 1, w_hs = 1, w_ff = 1;
  int max_experts = 0;
  for (const DxLayer& L : m->layers) total_heads += L.heads;
  std::vector<float> slopes(total_heads);
  size_t slope_at = 0;
  CUS(cudaMalloc(&m->slopes_all, std::max<size_t>(total_heads, 1) * sizeof(float)));
  for (size_t i = 0; i < m->layers.size(); ++i) {
    DxLayer& L = m->layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const size_t H = L.heads, G = L.kv_heads, d = L.dim, vd = L.vdim;
    L.norm1 = P(p + "norm1"), L.norm1b = P(p + "norm1b"), L.shift = P(p + "shift");
    L.w_in = P(p + "mix.q");
    L.q_b = P(p + "mix.q.b"), L.k_b = P(p + "mix.k.b"), L.v_b = P(p + "mix.v.b");
    L.vmix = P(p + "mix.vmix"), L.talk = P(p + "mix.talk"), L.wo = P(p + "mix.o");
    {  // the distance penalty of head g is 2^(-8 (g + 1) / H) per position; mixing the heads' scores mixes the slopes alike
      const TensorSpec* tk = at[p + "mix.talk"];
      for (size_t h = 0; h < H; ++h) {
        double s = 0.0;
        for (size_t g = 0; g < H; ++g) s += (double)bits_to_float(blob[tk->off + h * H + g]) * exp2(-8.0 * (double)(g + 1) / (double)H);
        slopes[slope_at + h] = (float)s;
      }
      L.slopes = m->slopes_all + slope_at;
      slope_at += H;
    }
    L.kv_off = page_elems;
    page_elems += (size_t)o.page_size * (G * d + G * vd);
    if (L.v_first) m->vf_width = (int)(G * vd);
    w0 = std::max(w0, H * d + G * d + G * vd + H * vd);
    w1 = std::max(w1, H * vd);
    w2 = std::max(w2, H * G * d);
    hmv = std::max(hmv, H * (vd + 2));
    maxk = std::max(maxk, H * vd);
    maxn = std::max(maxn, H * d + G * d + G * vd + H * vd);
    if (L.kind == 0) continue;
    L.norm2 = P(p + "norm2"), L.norm2b = P(p + "norm2b");
    if (L.kind == 1) {
      L.w_up = P(p + "mlp.up"), L.w_down = P(p + "mlp.down"), L.act = P(p + "mlp.act");
      w0 = std::max(w0, (size_t)L.ff);
      w_ff = std::max(w_ff, (size_t)L.ff);
      maxk = std::max(maxk, (size_t)L.ff);
      maxn = std::max(maxn, (size_t)L.ff);
    } else {
      L.w_router = P(p + "mlp.router"), L.correction = P(p + "mlp.correction");
      L.w_egu = P(p + "mlp.e0.gate"), L.w_edown = P(p + "mlp.e0.down");
      w_top = std::max(w_top, (size_t)L.top);
      w_he = std::max(w_he, (size_t)L.top * 2 * L.ff);
      max_experts = std::max(max_experts, L.experts);
      if (L.shared_ff > 0) {
        L.w_sgu = P(p + "mlp.shared.gate"), L.w_sdown = P(p + "mlp.shared.down");
        w_hs = std::max(w_hs, (size_t)2 * L.shared_ff);
        maxk = std::max(maxk, (size_t)L.shared_ff);
        maxn = std::max(maxn, (size_t)2 * L.shared_ff);
      }
    }
  }
  CUS(cudaMemcpy(m->slopes_all, slopes.data(), total_heads * sizeof(float), cudaMemcpyHostToDevice));
  // key/value pages
  m->page_elems = page_elems;
  const size_t elt = m->f32 ? 4 : 2;
  const size_t page_bytes = std::max<size_t>(page_elems * elt, 16);
  int n_pages = o.max_pages;
  if (n_pages <= 0) n_pages = (int)std::max<size_t>(1, (o.kv_bytes ? o.kv_bytes : ((size_t)1 << 30)) / page_bytes);
  CUS(cudaMalloc(&m->kv_pool, (size_t)n_pages * page_bytes));
  CUS(cudaMemsetAsync(m->kv_pool, 0, (size_t)n_pages * page_bytes, e->stream));
  e->kv = KvGeom{nullptr, n_pages, o.page_size, (int)m->layers.size(), 1, 0};
  CUS(engine_alloc_shared(e, n_pages, context));
  // carried rows of the token shift
  m->slot_floats = m->layers.size() * (size_t)m->width;
  CUS(cudaMalloc(&m->carry, (size_t)o.max_seqs * m->slot_floats * sizeof(float)));
  CUS(cudaMemsetAsync(m->carry, 0, (size_t)o.max_seqs * m->slot_floats * sizeof(float), e->stream));
  // activations
  const size_t R = o.max_batch_tokens, W = m->width;
  auto fbuf = [&](float** p, size_t n) { return cudaMalloc(p, std::max<size_t>(n, 1) * sizeof(float)); };
  CUS(fbuf(&m->x, R * W));
  CUS(fbuf(&m->hn, R * W));
  CUS(fbuf(&m->y, R * W));
  CUS(fbuf(&m->p0, R * w0));
  CUS(fbuf(&m->p1, R * w1));
  CUS(fbuf(&m->p2, R * w2));
  CUS(fbuf(&m->vf, R * std::max(m->vf_width, 1)));
  CUS(fbuf(&m->top_w, R * w_top));
  CUS(fbuf(&m->he, R * w_he));
  CUS(fbuf(&m->hg, R * w_he / 2 + 1));
  CUS(fbuf(&m->ye, max_experts ? R * w_top * W : 1));
  CUS(fbuf(&m->hs, R * w_hs));
  CUS(fbuf(&m->ys, R * W));
  CUS(fbuf(&m->xo, R * W));
  CUS(cudaMalloc(&m->top_idx, R * w_top * sizeof(int)));
  CUS(cudaMalloc(&m->perm_row, R * w_top * sizeof(int)));
  CUS(cudaMalloc(&m->slot_of, R * w_top * sizeof(int)));
  CUS(cudaMalloc(&m->grp_off, ((size_t)max_experts + 2) * sizeof(int)));
  m->attn_ws_floats = (R + 2048) * hmv;  // room for key splits when a step has few rows
  CUS(fbuf(&m->attn_ws, m->attn_ws_floats));
  if (!m->f32) {
    CUS(m->tc.alloc(R, maxk, std::max(maxn, (size_t)m->vocab), e->stream));
    auto bbuf = [&](bf16** p, size_t n) { return cudaMalloc(p, std::max<size_t>(n, 8) * sizeof(bf16)); };
    CUS(bbuf(&m->hb, R * W));
    CUS(bbuf(&m->ub, R * std::max(w_ff, w_hs)));
    CUS(bbuf(&m->ub2, R * std::max(w1, w_hs / 2 + 1)));
    CUS(bbuf(&m->yb, R * W));
    CUS(bbuf(&m->ysb, R * W));
    CUS(bbuf(&m->hgb, R * w_he / 2 + 8));
  }
  CUS(m->alloc_row_buffers(R));
  e->logits_rows = (int)R;
  CUS(cudaStreamSynchronize(e->stream));
  return "";
}

std::string create_common(qie_engine* e, const std::string& cfg_text, const std::string* st_path, uint64_t seed, int* code) {
  *code = QIE_EIO;
  JsonValue root;
  std::string err;
  if (!JsonReader::parse(cfg_text.data(), cfg_text.data() + cfg_text.size(), &root, &err)) return "config.json: " + err;
  e->dx = new DxModel();
  e->fam = e->dx;
  err = parse_config(root, e->dx);
  if (!err.empty()) return err;
  const std::vector<TensorSpec> t = build_layout(*e->dx);
  std::vector<uint16_t> blob(t.empty() ? 0 : t.back().off + t.back().elems(), 0);
  if (st_path) {
    err = load_safetensors_blob(*st_path, t, &blob);
    if (!err.empty()) return err;
  } else {
    fill_synthetic_blob(t, seed, &blob);
  }
  return finish_setup(e, t, blob, code);
}

}  // namespace

std::string ditenex_create(qie_engine* e, const std::string& dir, int* code) {
  std::string cfg;
  *code = QIE_EIO;
  if (!read_text_file(dir + "/config.json", &cfg)) return "cannot read " + dir + "/config.json";
  const std::string st = dir + "/model.safetensors";
  return create_common(e, cfg, &st, 0, code);
}

std::string ditenex_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code) {
  return create_common(e, cfg_json, nullptr, seed, code);
}

void DxModel::release() {
  void* dev[] = {blob, slopes_all, kv_pool, carry, x, hn, y, p0, p1, p2, vf, top_w, he, hg, ye, hs, ys, xo, top_idx, perm_row, slot_of, grp_off, attn_ws,
                 hb, ub, ub2, yb, ysb, hgb};
  tc.release();
  release_row_buffers();
  for (void* p : dev)
    if (p) cudaFree(p);
}

void DxModel::reset_slot(qie_engine* e, int seq) {
  if (carry) cudaMemsetAsync(carry + (size_t)seq * slot_floats, 0, slot_floats * sizeof(float), e->stream);
}

cudaError_t DxModel::forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) {
  DxModel* m = this;
  cudaStream_t st = e->stream;
  const int W = m->width;
  const int rnd = m->f32 ? 0 : 1;  // bf16 serving precision: the operands of the projections are bf16 values
  const int* segs = advance ? m->iota : m->seg_start;
  const int* seg_sl = advance ? e->slot_d : m->seg_slot;
  const int* outs = advance ? m->iota : m->out_rows;
  // plain projection C[rows, N] = A[rows, K] Wt[N, K]^T: the tcgen05 GEMM when the shape and the precision allow, else the
  // fp32-accumulate kernels (tensor cores on bf16 operands, plain fp32 in 32-bit mode)
  auto proj = [&](const float* A, int lda, const bf16* Wt, int K, int N, float* C, int ldc, int rows) {
    if (!m->f32 && m->tc.fits(rows, K, N, Wt)) return m->tc.gemm(e, A, lda, Wt, K, N, C, ldc, 0, rows);
    GemmF32 g;
    g.A = A, g.lda = lda, g.W = Wt, g.ldw = K, g.C = C, g.ldc = ldc, g.M = rows, g.N = N, g.K = K, g.round_a = rnd;
    return launch_gemm_f32(g, st);
  };
  if (m->dump_layers && !m->layer_dump)
    if (cudaMalloc(&m->layer_dump, m->layers.size() * (size_t)e->opts.max_batch_tokens * W * sizeof(float)) != cudaSuccess) return cudaErrorMemoryAllocation;
  FAM_TRY(KK_EMBED, launch_embed_streams(m->x, m->embed, m->pos_table, e->ids_d, e->pos_d, W, 1, n, st));
  // bf16 precision and a GEMM the tcgen05 kernel takes: its producer writes bf16 rows and its consumer reads them, with
  // no conversion kernels in between (the same bf16 values as on the fp32-row path: operands and results are rounded once)
  auto tcfit = [&](int K, int N, const bf16* Wt) { return !m->f32 && m->tc.fits(n, K, N, Wt); };
  for (size_t li = 0; li < m->layers.size(); ++li) {
    const DxLayer& L = m->layers[li];
    const int H = L.heads, G = L.kv_heads, d = L.dim, vd = L.vdim;
    const int Nq = H * d, Nk = G * d, Nv = G * vd, Ng = H * vd, Nin = Nq + Nk + Nv + Ng;
    const bool tc_in = tcfit(W, Nin, L.w_in), tc_o = tcfit(Ng, W, L.wo);
    {  // input norm + token shift
      RmsShiftArgs s;
      s.x = m->x, s.width = W, s.n = n, s.eps = m->eps, s.w = L.norm1, s.mu = L.shift;
      if (tc_in) s.out_bf = m->hb;
      else s.out = m->hn;
      s.carry = m->carry + li * (size_t)W, s.slot_stride = m->slot_floats;
      s.seg_start = segs, s.seg_slot = seg_sl, s.n_seg = n_seg;
      FAM_TRY(KK_F32_NORM, launch_rms_shift(s, st));
    }
    if (tc_in) {
      FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, m->hb, L.w_in, W, Nin, m->tc.cb, n));
      FAM_TRY(KK_F32_PROJ, launch_rows_bf16_to_f32(m->tc.cb, Nin, m->p0, Nin, 0, n, st));
    } else {
      FAM_TRY(KK_F32_PROJ, proj(m->hn, W, L.w_in, W, Nin, m->p0, Nin, n));
    }
    KvRowCache c;
    c.pool = m->kv_pool, c.elt_bytes = m->f32 ? 4 : 2, c.page_size = e->kv.page_size, c.page_elems = m->page_elems;
    c.layer_off = L.kv_off, c.kw = Nk, c.vw = Nv;
    {  // keys and values (+ biases, values blended with the first blending layer's) -> cache rows; head-mixed queries
      KvStoreArgs ks;
      ks.c = c, ks.k = m->p0 + Nq, ks.ldk = Nin, ks.v = m->p0 + Nq + Nk, ks.ldv = Nin;
      ks.k_bias = L.k_b, ks.v_bias = L.v_b;
      if (L.v_first) ks.v_keep = m->vf, ks.ld_vk = Nv;
      else if (L.v_mix) ks.v_lam = L.vmix, ks.v_other = m->vf, ks.ld_vo = Nv;
      // rider: the queries (+ bias) mixed over the heads, one vector per head against the whole key row
      ks.tq.q = m->p0, ks.tq.ldq = Nin, ks.tq.q_bias = L.q_b, ks.tq.talk = L.talk, ks.tq.qt = m->p2, ks.tq.ldqt = H * Nk;
      ks.tq.heads = H, ks.tq.kv_heads = G, ks.tq.dim = d;
      ks.pos = e->pos_d, ks.slot = e->slot_d, ks.block_table = e->block_table_d, ks.max_pages = e->max_pages_per_seq, ks.n = n;
      FAM_TRY(KK_KV_STORE, launch_kv_store_rows(ks, st));
    }
    {
      GqaAttnArgs g;
      g.c = c, g.q = m->p2, g.ldq = H * Nk, g.out = m->p1, g.ldo = Ng;
      if (tc_o) g.out_bf = m->ub2, g.ldo_bf = Ng;
      g.heads = H, g.kv_heads = G, g.dim = Nk, g.vdim = vd, g.maps = 1, g.scale = L.scale, g.shared_keys = 1, g.slopes = L.slopes;
      g.window = L.window, g.finish = 3, g.gate = m->p0 + Nq + Nk + Nv, g.ldg = Nin, g.eps = m->eps;
      g.pos = e->pos_d, g.slot = e->slot_d, g.block_table = e->block_table_d, g.max_pages = e->max_pages_per_seq, g.n = n, g.max_keys = max_kv_len;
      g.ws = m->attn_ws, g.ws_floats = m->attn_ws_floats, g.num_sms = e->num_sms;
      g.seg_start = segs, g.seg_slot = seg_sl, g.n_seg = n_seg;
      int nl = 0;
      FAM_TRY(KK_GQA_ATTN, launch_gqa_attention(g, st, &nl));
      e->launches += nl > 0 ? nl - 1 : 0;
    }
    if (tc_o) FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, m->ub2, L.wo, Ng, W, m->yb, n));
    else FAM_TRY(KK_F32_PROJ, proj(m->p1, Ng, L.wo, Ng, W, m->y, W, n));
    // which rows the feed-forward's GEMMs want
    const bool tc_up = L.kind == 1 && tcfit(W, L.ff, L.w_up), tc_down = tc_up && tcfit(L.ff, W, L.w_down);
    const bool tc_sh = L.kind == 2 && L.shared_ff > 0 && tcfit(W, 2 * L.shared_ff, L.w_sgu) && tcfit(L.shared_ff, W, L.w_sdown);
    // the experts' GEMMs over bf16 rows on the tensor-core tile kernel (more rows than the GEMV serves)
    GroupedGemmBf16 eg, ed;
    bool tc_ex = false;
    if (L.kind == 2 && !m->f32 && n * L.top > 16 * 16) {
      eg.A = m->hb, eg.lda = W, eg.row_idx = m->perm_row, eg.grp_off = m->grp_off, eg.W = L.w_egu, eg.w_batch = (long)2 * L.ff * W;
      eg.N = 2 * L.ff, eg.K = W, eg.groups = L.experts, eg.rows = n * L.top, eg.gated = 1, eg.out_bf = m->hgb, eg.ldo = L.ff;
      ed.A = m->hgb, ed.lda = L.ff, ed.grp_off = m->grp_off, ed.W = L.w_edown, ed.w_batch = (long)W * L.ff;
      ed.N = W, ed.K = L.ff, ed.groups = L.experts, ed.rows = n * L.top, ed.out = m->ye, ed.ldo = W;
      tc_ex = grouped_gemm_bf16_fits(eg) && grouped_gemm_bf16_fits(ed);
    }
    {  // x += m * rms(y) norm1b; the same launch norms for the feed-forward
      RmsStep s;
      s.x = m->x, s.width = W, s.n = n, s.eps = m->eps, s.w_out = L.norm1b, s.mult = m->res_mult;
      if (tc_o) s.y_bf = m->yb;
      else s.y = m->y;
      if (L.kind) {
        s.w_in = L.norm2;
        if (tc_up || tc_sh || tc_ex) s.h_bf = m->hb;
        if (!tc_up) s.h = m->hn;  // the experts' GEMV reads fp32 rows
        if (L.kind == 2) {  // the router's logits and choice ride this launch
          s.route.w_router = L.w_router, s.route.correction = L.correction, s.route.experts = L.experts, s.route.top = L.top;
          s.route.groups = L.groups, s.route.keep = L.keep, s.route.scale = L.route_scale, s.route.top_idx = m->top_idx, s.route.top_w = m->top_w;
        }
      }
      FAM_TRY(KK_F32_NORM, launch_rms_step(s, st));
    }
    if (L.kind == 1) {
      RmsStep s;
      s.x = m->x, s.width = W, s.n = n, s.eps = m->eps, s.w_out = L.norm2b, s.mult = m->res_mult;
      if (tc_up) {
        FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, m->hb, L.w_up, W, L.ff, m->ub, n));
        FAM_TRY(KK_GLU, launch_xielu_bf16(m->ub, L.ff, L.ff, L.act, n, st));
        if (tc_down) {
          FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, m->ub, L.w_down, L.ff, W, m->yb, n));
          s.y_bf = m->yb;
        } else {
          FAM_TRY(KK_F32_PROJ, launch_rows_bf16_to_f32(m->ub, L.ff, m->p0, L.ff, 0, n, st));
          FAM_TRY(KK_F32_PROJ, proj(m->p0, L.ff, L.w_down, L.ff, W, m->y, W, n));
          s.y = m->y;
        }
      } else {
        FAM_TRY(KK_F32_PROJ, proj(m->hn, W, L.w_up, W, L.ff, m->p0, L.ff, n));
        FAM_TRY(KK_GLU, launch_xielu(m->p0, L.ff, L.ff, L.act, n, st));
        FAM_TRY(KK_F32_PROJ, proj(m->p0, L.ff, L.w_down, L.ff, W, m->y, W, n));
        s.y = m->y;
      }
      FAM_TRY(KK_F32_NORM, launch_rms_step(s, st));
    } else if (L.kind == 2) {
      const int E = L.experts, top = L.top, ff = L.ff;
      FAM_TRY(KK_MOE_ROUTE, launch_moe_group(m->top_idx, n * top, top, E, m->grp_off, m->perm_row, m->slot_of, st));
      if (tc_ex) {
        FAM_TRY(KK_MOE_EXPERTS, launch_grouped_gemm_bf16(eg, st));
        FAM_TRY(KK_MOE_EXPERTS, launch_grouped_gemm_bf16(ed, st));
      } else {
        GemmF32 g;  // [gate | up] of every assignment, rows grouped by expert and gathered from hn
        g.A = m->hn, g.lda = W, g.W = L.w_egu, g.ldw = W, g.w_batch = (long)2 * ff * W, g.C = m->he, g.ldc = 2 * ff;
        g.M = n * top, g.N = 2 * ff, g.K = W, g.batches = E, g.grp_off = m->grp_off, g.row_idx = m->perm_row, g.round_a = rnd;
        FAM_TRY(KK_MOE_EXPERTS, launch_gemm_f32(g, st));
        FAM_TRY(KK_GLU, launch_silu_glu(m->he, 2 * ff, m->hg, ff, ff, n * top, st));
        GemmF32 g2;
        g2.A = m->hg, g2.lda = ff, g2.W = L.w_edown, g2.ldw = ff, g2.w_batch = (long)W * ff, g2.C = m->ye, g2.ldc = W;
        g2.M = n * top, g2.N = W, g2.K = ff, g2.batches = E, g2.grp_off = m->grp_off, g2.round_a = rnd;
        FAM_TRY(KK_MOE_EXPERTS, launch_gemm_f32(g2, st));
      }
      RmsStep s;  // the combine of the experts rides the output norm
      s.x = m->x, s.width = W, s.n = n, s.eps = m->eps, s.w_out = L.norm2b, s.mult = m->res_mult;
      s.mix.ye = m->ye, s.mix.slot_of = m->slot_of, s.mix.top_w = m->top_w, s.mix.top = top;
      if (L.shared_ff > 0) {
        const int sf = L.shared_ff;
        if (tc_sh) {
          FAM_TRY(KK_MOE_SHARED, m->tc.gemm_bf16(e, m->hb, L.w_sgu, W, 2 * sf, m->ub, n));
          FAM_TRY(KK_GLU, launch_silu_glu_bf16(m->ub, 2 * sf, m->ub2, sf, sf, n, st));
          FAM_TRY(KK_MOE_SHARED, m->tc.gemm_bf16(e, m->ub2, L.w_sdown, sf, W, m->ysb, n));
          s.ys_bf = m->ysb;
        } else {
          FAM_TRY(KK_MOE_SHARED, proj(m->hn, W, L.w_sgu, W, 2 * sf, m->hs, 2 * sf, n));
          FAM_TRY(KK_GLU, launch_silu_glu(m->hs, 2 * sf, m->hs, 2 * sf, sf, n, st));
          FAM_TRY(KK_MOE_SHARED, proj(m->hs, 2 * sf, L.w_sdown, sf, W, m->ys, W, n));
          s.mix.ys = m->ys;
        }
      }
      FAM_TRY(KK_F32_NORM, launch_rms_step(s, st));
    }
    if (m->dump_layers)
      if (cudaMemcpyAsync(m->layer_dump + li * (size_t)e->opts.max_batch_tokens * W, m->x, (size_t)n * W * sizeof(float), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return cudaErrorUnknown;
  }
  if (n_out <= 0) return cudaSuccess;
  {
    RmsStep s;
    s.x = m->x, s.width = W, s.n = n_out, s.eps = m->eps, s.w_in = m->final_norm, s.h = m->xo, s.gather = outs;
    FAM_TRY(KK_F32_NORM, launch_rms_step(s, st));
  }
  {  // the logits reuse the embedding table
    GemmF32 g;
    g.A = m->xo, g.lda = W, g.W = m->embed, g.ldw = W, g.C = m->logits, g.ldc = m->vocab, g.M = n_out, g.N = m->vocab, g.K = W, g.round_a = rnd;
    FAM_TRY(KK_LM_HEAD, launch_gemm_f32(g, st));
  }
  return sample_rows(e, n_out, temperature, advance);
}

}  // namespace qie
