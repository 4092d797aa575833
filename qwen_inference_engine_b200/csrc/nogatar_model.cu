// nogatar_model.cu -- the Nogatar family on the engine: configuration reader (config.json), weight loader
// (model.safetensors -> one device blob), rotary tables, the paged latent cache and the recurrent state slots, and
// the launch order of one forward over a batch of rows.  A row is (sequence slot, position) exactly as in the Qwen
// forward (engine.cu); rows of one sequence are consecutive and in position order, rows of different sequences may
// be portions of prompts next to single decoded tokens.  Every size and constant comes from the configuration.
#include "nogatar.h"

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

std::string parse_config(const JsonValue& root, NgModel* m) {
  NEED(root.kind == JsonValue::Object, "config.json: not an object");
  m->vocab = as_int(root.have("vocab"), 0);
  m->width = as_int(root.have("width"), 0);
  NEED(m->vocab > 0 && m->width > 0, "config.json: vocab / width missing");
  if (const JsonValue* e = root.have("embedding")) m->embed_scale = (float)(e->have("scale") ? e->have("scale")->number_or(1.0) : 1.0);
  if (const JsonValue* nm = root.have("norm")) m->eps = (float)(nm->have("eps") ? nm->have("eps")->number_or(1e-6) : 1e-6);
  m->res_mult = (float)(root.have("residual_mult") ? root.have("residual_mult")->number_or(1.0) : 1.0);
  m->softcap = (float)(root.have("logit_softcap") ? root.have("logit_softcap")->number_or(0.0) : 0.0);
  const JsonValue* layers = root.have("layers");
  NEED(layers && layers->kind == JsonValue::Array && !layers->arr.empty(), "config.json: layers missing");
  int n_attn = 0, n_state = 0;
  for (const JsonValue& jl : layers->arr) {
    NgLayer L;
    const JsonValue* type = jl.have("type");
    const JsonValue* mx = jl.have("mixer");
    NEED(type && type->kind == JsonValue::String && mx, "config.json: layer without type / mixer");
    L.heads = as_int(mx->have("heads"), 0);
    L.dim = as_int(mx->have("dim"), 0);
    L.vdim = as_int(mx->have("vdim"), 0);
    NEED(L.heads > 0 && L.dim > 0 && L.vdim > 0, "config.json: mixer heads / dim / vdim missing");
    if (type->str == "latent_attention") {
      L.type = 0;
      L.attn_id = n_attn++;
      L.rot_dim = as_int(mx->have("rot_dim"), 0);
      L.kv_rank = as_int(mx->have("kv_rank"), 0);
      NEED(L.kv_rank > 0 && L.rot_dim >= 0, "config.json: latent attention without kv_rank");
      NEED(mx->have("scale"), "config.json: latent attention without scale");
      L.scale = (float)mx->have("scale")->number_or(1.0);
      if (const JsonValue* mk = mx->have("mask")) L.window = as_int(mk->have("size"), 0);
      if (const JsonValue* rt = mx->have("rot")) {
        L.rot.dims = as_int(rt->have("dims"), L.rot_dim);
        L.rot.base = rt->have("base") ? rt->have("base")->number_or(10000.0) : 10000.0;
        if (const JsonValue* sc = rt->have("scaling")) {
          L.rot.scaled = true;
          L.rot.factor = sc->have("factor") ? sc->have("factor")->number_or(1.0) : 1.0;
          L.rot.original = sc->have("original") ? sc->have("original")->number_or(0.0) : 0.0;
          L.rot.fast = sc->have("fast") ? sc->have("fast")->number_or(32.0) : 32.0;
          L.rot.slow = sc->have("slow") ? sc->have("slow")->number_or(1.0) : 1.0;
          NEED(L.rot.original > 0 && L.rot.factor > 0, "config.json: rot.scaling needs factor and original");
        }
      }
      NEED(L.rot.dims % 2 == 0 && L.rot.dims <= L.rot_dim, "config.json: rot.dims must be even and <= rot_dim");
    } else if (type->str == "mlstm") {
      L.type = 1;
      L.state_id = n_state++;
      NEED(mx->have("gate_cap") && mx->have("gate_cap")->is_number() && mx->have("gate_cap")->num > 0, "config.json: mlstm without gate_cap");
      L.gate_cap = (float)mx->have("gate_cap")->num;
    } else {
      return "config.json: unknown layer type '" + type->str + "'";
    }
    if (const JsonValue* mlp = jl.have("mlp")) {
      const JsonValue* kind = mlp->have("kind");
      NEED(!kind || kind->str == "moe", "config.json: unknown mlp kind");
      const JsonValue* rt = mlp->have("router");
      const JsonValue* ex = mlp->have("expert");
      NEED(rt && ex, "config.json: mlp without router / expert");
      L.experts = as_int(rt->have("experts"), 0);
      L.top = as_int(rt->have("top"), 0);
      L.ff = as_int(ex->have("ff"), 0);
      NEED(L.experts > 0 && L.top > 0 && L.top <= L.experts && L.ff > 0, "config.json: bad router / expert sizes");
      if (const JsonValue* sh = mlp->have("shared")) L.shared_ff = as_int(sh->have("ff"), 0);
    }
    m->layers.push_back(L);
  }
  return "";
}

// tensors in blob order; tensors that one GEMM reads as a single matrix are adjacent (no padding between them)
std::vector<TensorSpec> build_layout(const NgModel& m) {
  BlobLayout bl;
  auto pad = [&]() { bl.pad(); };  // 256-byte boundaries between groups
  auto add = [&](const std::string& name, size_t rows, size_t cols, int kind) { bl.add(name, rows, cols, kind); };
  const size_t W = m.width;
  pad(), add("embed", m.vocab, W, 0);
  for (size_t i = 0; i < m.layers.size(); ++i) {
    const NgLayer& L = m.layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const size_t H = L.heads, d = L.dim, vd = L.vdim;
    pad(), add(p + "norm1", W, 0, 1);
    if (L.type == 0) {
      const size_t r = L.rot_dim, k = L.kv_rank;
      pad(), add(p + "mix.q", H * (d + r), W, 0), add(p + "mix.dkv", k + r, W, 0);
      pad(), add(p + "mix.dkv.norm", k, 0, 1);
      pad(), add(p + "mix.uk", H * d, k, 0);
      pad(), add(p + "mix.uv", H * vd, k, 0);
      pad(), add(p + "mix.sink", H, 0, 2);
      pad(), add(p + "mix.o", W, H * vd, 0);
    } else {
      pad(), add(p + "mix.q", H * d, W, 0), add(p + "mix.k", H * d, W, 0), add(p + "mix.v", H * vd, W, 0), add(p + "mix.g", H * vd, W, 0);
      pad(), add(p + "mix.i", H, W, 0), add(p + "mix.f", H, W, 0);
      pad(), add(p + "mix.i.b", H, 0, 2), add(p + "mix.f.b", H, 0, 2);
      pad(), add(p + "mix.norm", H * vd, 0, 1);
      pad(), add(p + "mix.o", W, H * vd, 0);
    }
    if (L.experts > 0) {
      pad(), add(p + "norm2", W, 0, 1);
      pad();
      for (int e = 0; e < L.experts; ++e) add(p + "mlp.e" + std::to_string(e) + ".up", L.ff, W, 0);
      pad();
      for (int e = 0; e < L.experts; ++e) add(p + "mlp.e" + std::to_string(e) + ".down", W, L.ff, 0);
      pad(), add(p + "mlp.router", L.experts, W, 0);
      if (L.shared_ff > 0) {
        add(p + "mlp.shared.sg", 1, W, 0);
        pad(), add(p + "mlp.shared.up", L.shared_ff, W, 0);
        pad(), add(p + "mlp.shared.down", W, L.shared_ff, 0);
      }
    }
  }
  pad(), add("final.norm", W, 0, 1);
  pad(), add("head", m.vocab, W, 0);
  return bl.t;
}

size_t layout_elems(const std::vector<TensorSpec>& t) { return t.empty() ? 0 : t.back().off + t.back().elems(); }


#define CUS(expr)                                                      \
  do {                                                                 \
    cudaError_t _e = (expr);                                           \
    if (_e != cudaSuccess) {                                           \
      *code = QIE_ECUDA;                                               \
      return std::string(#expr) + ": " + cudaGetErrorString(_e);       \
    }                                                                  \
  } while (0)

std::string finish_setup(qie_engine* e, const std::vector<TensorSpec>& t, const std::vector<uint16_t>& blob, int* code) {
  NgModel* m = e->ng;
  const qie_engine_opts& o = e->opts;
  m->f32 = o.compute_dtype == QIE_DTYPE_F32;
  m->blob_bytes = blob.size() * 2;
  CUS(cudaMalloc(&m->blob, m->blob_bytes));
  CUS(cudaMemcpy(m->blob, blob.data(), m->blob_bytes, cudaMemcpyHostToDevice));
  std::map<std::string, const bf16*> at;
  for (const TensorSpec& s : t) at[s.name] = m->blob + s.off;
  auto P = [&](const std::string& n) -> const bf16* {
    auto it = at.find(n);
    return it == at.end() ? nullptr : it->second;
  };
  m->embed = P("embed");
  m->final_norm = P("final.norm");
  m->head = P("head");
  e->cfg = qie_config{m->width, 0, (int)m->layers.size(), 0, 0, 0, m->vocab, o.context};
  size_t page_elems = 0, slot_floats = 0;
  size_t max_rank = 0;
  size_t w0 = 0, w1 = 0, w2 = 0, w3 = 0, w_zr = 1, w_he = 0, w_hs = 0, w_top = 1;
  for (size_t i = 0; i < m->layers.size(); ++i) {
    NgLayer& L = m->layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const size_t H = L.heads, d = L.dim, vd = L.vdim;
    L.norm1 = P(p + "norm1");
    L.wo = P(p + "mix.o");
    if (L.type == 0) {
      L.wq = P(p + "mix.q");
      L.wdkv = P(p + "mix.dkv");
      L.dkv_norm = P(p + "mix.dkv.norm");
      L.wuk = P(p + "mix.uk");
      L.wuv = P(p + "mix.uv");
      L.sink = P(p + "mix.sink");
      m->lat_off.push_back(page_elems);
      page_elems += (size_t)o.page_size * (L.kv_rank + L.rot_dim);
      size_t id = 0;
      while (id < m->rope_cfg.size() && !(m->rope_cfg[id] == L.rot)) ++id;
      if (id == m->rope_cfg.size()) m->rope_cfg.push_back(L.rot);
      L.rope_id = (int)id;
      w0 = std::max(w0, H * (d + L.rot_dim) + L.kv_rank + L.rot_dim);
      w1 = std::max(w1, H * (size_t)(L.kv_rank + L.rot_dim));
      w2 = std::max(w2, H * (size_t)L.kv_rank);
      max_rank = std::max(max_rank, (size_t)L.kv_rank);
      w3 = std::max(w3, H * vd);
    } else {
      L.wqkvg = P(p + "mix.q");
      L.wif = P(p + "mix.i");
      L.bif = P(p + "mix.i.b");
      L.out_norm = P(p + "mix.norm");
      m->state_off.push_back(slot_floats);
      slot_floats += mlstm_state_floats(L.heads, L.dim, L.vdim);
      w0 = std::max(w0, 2 * H * d + 2 * H * vd);
      w1 = std::max(w1, 2 * H);
      w2 = std::max(w2, H * vd);
    }
    if (L.experts > 0) {
      L.norm2 = P(p + "norm2");
      L.w_up = P(p + "mlp.e0.up");
      L.w_down = P(p + "mlp.e0.down");
      L.w_router = P(p + "mlp.router");
      if (L.shared_ff > 0) {
        L.w_sup = P(p + "mlp.shared.up");
        L.w_sdown = P(p + "mlp.shared.down");
      }
      w_zr = std::max(w_zr, (size_t)L.experts + 1);
      w_top = std::max(w_top, (size_t)L.top);
      w_he = std::max(w_he, (size_t)L.top * L.ff);
      w_hs = std::max(w_hs, (size_t)L.shared_ff);
      m->max_experts = std::max(m->max_experts, L.experts);
    }
  }
  // rotary tables
  for (const NgRot& r : m->rope_cfg) {
    std::vector<float> c, s;
    rotary_tables(r, o.context, &c, &s);
    float *cd = nullptr, *sd = nullptr;
    if (!c.empty()) {
      CUS(cudaMalloc(&cd, c.size() * sizeof(float)));
      CUS(cudaMalloc(&sd, s.size() * sizeof(float)));
      CUS(cudaMemcpy(cd, c.data(), c.size() * sizeof(float), cudaMemcpyHostToDevice));
      CUS(cudaMemcpy(sd, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    m->rope_cos.push_back(cd);
    m->rope_sin.push_back(sd);
  }
  // latent cache pages (a model without attention layers still counts positions in pages)
  m->page_elems = page_elems;
  const size_t elt = m->f32 ? 4 : 2;
  const size_t page_bytes = std::max<size_t>(page_elems * elt, 16);
  int n_pages = o.max_pages;
  if (n_pages <= 0) n_pages = (int)std::max<size_t>(1, (o.kv_bytes ? o.kv_bytes : ((size_t)1 << 30)) / page_bytes);
  CUS(cudaMalloc(&m->lat_pool, (size_t)n_pages * page_bytes));
  CUS(cudaMemsetAsync(m->lat_pool, 0, (size_t)n_pages * page_bytes, e->stream));
  e->kv = KvGeom{nullptr, n_pages, o.page_size, (int)m->lat_off.size(), 1, 0};
  CUS(engine_alloc_shared(e, n_pages, o.context));
  // recurrent state slots
  m->slot_floats = slot_floats;
  if (slot_floats) {
    CUS(cudaMalloc(&m->state, (size_t)o.max_seqs * slot_floats * sizeof(float)));
    CUS(cudaMemsetAsync(m->state, 0, (size_t)o.max_seqs * slot_floats * sizeof(float), e->stream));
  }
  // activations
  const size_t R = o.max_batch_tokens, W = m->width;
  auto fbuf = [&](float** p, size_t n) { return cudaMalloc(p, std::max<size_t>(n, 1) * sizeof(float)); };
  CUS(fbuf(&m->x, R * W));
  CUS(fbuf(&m->y, R * W));
  CUS(fbuf(&m->p0, R * w0));
  CUS(fbuf(&m->p1, R * w1));
  CUS(fbuf(&m->p2, R * w2));
  CUS(fbuf(&m->p3, R * w3));
  CUS(fbuf(&m->zr, R * w_zr));
  CUS(fbuf(&m->top_w, R * w_top));
  CUS(fbuf(&m->he, R * w_he));
  CUS(fbuf(&m->ye, R * w_top * W));
  CUS(fbuf(&m->hs, R * w_hs));
  CUS(fbuf(&m->ys, R * W));
  CUS(fbuf(&m->xo, R * W));
  m->attn_ws_floats = (size_t)4096 * (max_rank + 2);  // up to 4096 (row, head, split) partial results
  CUS(fbuf(&m->attn_ws, m->attn_ws_floats));
  if (!m->f32) {
    size_t maxk = W, maxn = std::max<size_t>(W, (size_t)m->vocab);
    maxk = std::max(maxk, std::max(w2, std::max(w3, w_hs)));
    maxn = std::max(maxn, std::max(w0, w_hs));
    CUS(m->tc.alloc(R, maxk, maxn, e->stream));
  }
  CUS(m->alloc_row_buffers(R));
  CUS(cudaMalloc(&m->top_idx, R * w_top * sizeof(int)));
  CUS(cudaMalloc(&m->perm_row, R * w_top * sizeof(int)));
  CUS(cudaMalloc(&m->slot_of, R * w_top * sizeof(int)));
  CUS(cudaMalloc(&m->grp_off, ((size_t)m->max_experts + 2) * sizeof(int)));
  e->logits_rows = (int)R;
  CUS(cudaStreamSynchronize(e->stream));
  return "";
}

std::string create_common(qie_engine* e, const std::string& cfg_text, const std::string* st_path, uint64_t seed, int* code) {
  *code = QIE_EIO;
  JsonValue root;
  std::string err;
  if (!JsonReader::parse(cfg_text.data(), cfg_text.data() + cfg_text.size(), &root, &err)) return "config.json: " + err;
  e->ng = new NgModel();
  e->fam = e->ng;
  err = parse_config(root, e->ng);
  if (!err.empty()) return err;
  const std::vector<TensorSpec> t = build_layout(*e->ng);
  std::vector<uint16_t> blob(layout_elems(t), 0);
  if (st_path) {
    err = load_safetensors_blob(*st_path, t, &blob);
    if (!err.empty()) return err;
  } else {
    fill_synthetic_blob(t, seed, &blob);
  }
  return finish_setup(e, t, blob, code);
}

}  // namespace

std::string nogatar_create(qie_engine* e, const std::string& dir, int* code) {
  std::string cfg;
  *code = QIE_EIO;
  if (!read_text_file(dir + "/config.json", &cfg)) return "cannot read " + dir + "/config.json";
  const std::string st = dir + "/model.safetensors";
  return create_common(e, cfg, &st, 0, code);
}

std::string nogatar_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code) {
  return create_common(e, cfg_json, nullptr, seed, code);
}

void NgModel::release() {
  NgModel* m = this;
  void* dev[] = {m->blob, m->lat_pool, m->state, m->x, m->y, m->p0, m->p1, m->p2, m->p3, m->zr, m->top_w, m->he, m->ye, m->hs, m->ys, m->xo,
                 m->top_idx, m->perm_row, m->slot_of, m->grp_off, m->attn_ws};
  m->tc.release();
  m->release_row_buffers();
  for (void* p : dev)
    if (p) cudaFree(p);
  for (float* p : m->rope_cos)
    if (p) cudaFree(p);
  for (float* p : m->rope_sin)
    if (p) cudaFree(p);
}

void NgModel::reset_slot(qie_engine* e, int seq) {
  if (state) cudaMemsetAsync(state + (size_t)seq * slot_floats, 0, slot_floats * sizeof(float), e->stream);
}

#define NG_TRY FAM_TRY

cudaError_t NgModel::forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) {
  NgModel* m = this;
  cudaStream_t st = e->stream;
  const int W = m->width;
  const int rnd = m->f32 ? 0 : 1;  // bf16 serving precision: operands and results of the projections are bf16 values
  const int* seg_start = advance ? m->iota : m->seg_start;
  const int* seg_slot = advance ? e->slot_d : m->seg_slot;
  const int* out_rows = advance ? m->iota : m->out_rows;
  auto gemm = [&](const float* A, int lda, const bf16* Wt, int K, int N, float* C, int ldc, int act, int round) {
    GemmF32 g;
    g.A = A, g.lda = lda, g.W = Wt, g.ldw = K, g.C = C, g.ldc = ldc, g.M = n, g.N = N, g.K = K, g.act = act;
    g.round_a = round, g.round_c = round;
    return g;
  };
  // plain projection: the tcgen05 GEMM when the shape and the precision allow, else the fp32-accumulate kernels
  auto proj = [&](const float* A, int lda, const bf16* Wt, int K, int N, float* C, int ldc, int act, int rows) {
    if (!m->f32 && m->tc.fits(rows, K, N, Wt)) return m->tc.gemm(e, A, lda, Wt, K, N, C, ldc, act, rows);
    GemmF32 g = gemm(A, lda, Wt, K, N, C, ldc, act, rnd);
    g.M = rows;
    return launch_gemm_f32(g, st);
  };
  if (m->dump_layers && !m->layer_dump)
    if (cudaMalloc(&m->layer_dump, m->layers.size() * (size_t)e->opts.max_batch_tokens * W * sizeof(float)) != cudaSuccess) return cudaErrorMemoryAllocation;
  NG_TRY(KK_EMBED, launch_embed_scale_f32(m->x, m->embed, e->ids_d, W, n, m->embed_scale, st));
  for (size_t li = 0; li < m->layers.size(); ++li) {
    const NgLayer& L = m->layers[li];
    const int H = L.heads, d = L.dim, vd = L.vdim;
    if (L.type == 0) {
      const int r = L.rot_dim, k = L.kv_rank, Nq = H * (d + r), Nd = k + r, ld0 = Nq + Nd, D = k + r;
      NG_TRY(KK_F32_PROJ, proj(m->x, W, L.wq, W, ld0, m->p0, ld0, 0, n));
      LatentCache c;
      c.pool = m->lat_pool, c.elt_bytes = m->f32 ? 4 : 2, c.page_size = e->kv.page_size, c.page_elems = m->page_elems;
      c.layer_off = m->lat_off[L.attn_id], c.rank = k, c.rot = r;
      RopeTable rope{m->rope_cos[L.rope_id], m->rope_sin[L.rope_id], L.rot.dims};
      QueryRope qr;  // the rotated part of the query heads goes behind the absorbed part of qa
      if (r > 0) qr.src = m->p0 + d, qr.ld_src = ld0, qr.hs_src = d + r, qr.dst = m->p1 + k, qr.ld_dst = H * D, qr.hs_dst = D, qr.heads = H;
      NG_TRY(KK_LATENT_STORE, launch_latent_store(c, m->p0 + Nq, ld0, L.dkv_norm, m->eps, rope, e->pos_d, e->slot_d, e->block_table_d, e->max_pages_per_seq, n, st, qr));
      {  // the key up-projection folded into the query: qa[:, h, 0:k] = W_uk,h^T q_h (unrotated part)
        GemmF32 g;
        g.A = m->p0, g.lda = ld0, g.a_batch = d + r;
        g.W = L.wuk, g.ldw = k, g.w_batch = (long)d * k, g.w_trans = 1;
        g.C = m->p1, g.ldc = H * D, g.c_batch = D;
        g.M = n, g.N = k, g.K = d, g.batches = H, g.round_a = rnd;
        NG_TRY(KK_F32_PROJ, launch_gemm_f32(g, st));
      }
      NG_TRY(KK_LATENT_ATTN, launch_latent_attention(c, m->p1, m->p2, L.sink, L.scale, L.window, H, e->pos_d, e->slot_d, e->block_table_d, e->max_pages_per_seq, n, max_kv_len, m->attn_ws, m->attn_ws_floats, st));
      {  // value up-projection of the attended latent, head by head
        GemmF32 g;
        g.A = m->p2, g.lda = H * k, g.a_batch = k;
        g.W = L.wuv, g.ldw = k, g.w_batch = (long)vd * k;
        g.C = m->p3, g.ldc = H * vd, g.c_batch = vd;
        g.M = n, g.N = vd, g.K = k, g.batches = H, g.round_a = rnd, g.round_c = rnd;
        NG_TRY(KK_F32_PROJ, launch_gemm_f32(g, st));
      }
      NG_TRY(KK_F32_PROJ, proj(m->p3, H * vd, L.wo, H * vd, W, m->y, W, 0, n));
    } else {
      const int N0 = 2 * H * d + 2 * H * vd;
      NG_TRY(KK_F32_PROJ, proj(m->x, W, L.wqkvg, W, N0, m->p0, N0, 0, n));
      {
        GemmF32 g = gemm(m->x, W, L.wif, W, 2 * H, m->p1, 2 * H, 0, 0);  // gate pre-activations: fp32
        g.bias = L.bif;
        NG_TRY(KK_F32_PROJ, launch_gemm_f32(g, st));
      }
      MlstmArgs a;
      a.qkvg = m->p0, a.ld = N0, a.gates = m->p1;
      a.state = m->state + m->state_off[L.state_id], a.slot_stride = m->slot_floats;
      a.out = m->p2, a.w_norm = L.out_norm, a.heads = H, a.dim = d, a.vdim = vd, a.gate_cap = L.gate_cap, a.eps = m->eps;
      a.seg_start = seg_start, a.seg_slot = seg_slot, a.n_seg = n_seg, a.n_rows = n;
      NG_TRY(KK_MLSTM, launch_mlstm_scan(a, st));
      NG_TRY(KK_F32_PROJ, proj(m->p2, H * vd, L.wo, H * vd, W, m->y, W, 0, n));
    }
    NG_TRY(KK_F32_NORM, launch_layernorm_f32(m->y, L.norm1, m->x, m->x, nullptr, W, n, m->eps, m->res_mult, st));
    if (L.experts > 0) {
      const int E = L.experts, top = L.top, ldz = E + (L.shared_ff > 0 ? 1 : 0);
      NG_TRY(KK_MOE_ROUTE, launch_gemm_f32(gemm(m->x, W, L.w_router, W, ldz, m->zr, ldz, 0, 0), st));  // router (+ shared gate): fp32
      NG_TRY(KK_MOE_ROUTE, launch_moe_route(m->zr, ldz, E, top, m->top_idx, m->top_w, n, st));
      NG_TRY(KK_MOE_ROUTE, launch_moe_group(m->top_idx, n * top, top, E, m->grp_off, m->perm_row, m->slot_of, st));
      {
        GemmF32 g = gemm(m->x, W, L.w_up, W, L.ff, m->he, L.ff, 1, rnd);
        g.M = n * top, g.batches = E, g.w_batch = (long)L.ff * W, g.grp_off = m->grp_off, g.row_idx = m->perm_row;
        NG_TRY(KK_MOE_EXPERTS, launch_gemm_f32(g, st));
        GemmF32 g2 = gemm(m->he, L.ff, L.w_down, L.ff, W, m->ye, W, 0, rnd);
        g2.M = n * top, g2.batches = E, g2.w_batch = (long)W * L.ff, g2.grp_off = m->grp_off;
        NG_TRY(KK_MOE_EXPERTS, launch_gemm_f32(g2, st));
      }
      if (L.shared_ff > 0) {
        NG_TRY(KK_MOE_SHARED, proj(m->x, W, L.w_sup, W, L.shared_ff, m->hs, L.shared_ff, 1, n));
        NG_TRY(KK_MOE_SHARED, proj(m->hs, L.shared_ff, L.w_sdown, L.shared_ff, W, m->ys, W, 0, n));
      }
      {  // combine folded into the output norm
        MoeMix mix;
        mix.ye = m->ye, mix.slot_of = m->slot_of, mix.top_w = m->top_w, mix.top = top, mix.ys = L.shared_ff > 0 ? m->ys : nullptr;
        mix.z = m->zr, mix.ldz = ldz, mix.gate_col = E;
        NG_TRY(KK_F32_NORM, launch_layernorm_f32(nullptr, L.norm2, m->x, m->x, nullptr, W, n, m->eps, m->res_mult, st, mix));
      }
    }
    if (m->dump_layers)
      if (cudaMemcpyAsync(m->layer_dump + li * (size_t)e->opts.max_batch_tokens * W, m->x, (size_t)n * W * sizeof(float), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return cudaErrorUnknown;
  }
  if (n_out <= 0) return cudaSuccess;
  NG_TRY(KK_F32_NORM, launch_layernorm_f32(m->x, m->final_norm, m->xo, nullptr, out_rows, W, n_out, m->eps, 1.0f, st));
  {
    GemmF32 g = gemm(m->xo, W, m->head, W, m->vocab, m->logits, m->vocab, 0, rnd);
    g.M = n_out;
    g.round_c = 0;
    NG_TRY(KK_LM_HEAD, launch_gemm_f32(g, st));
  }
  if (m->softcap > 0.f) NG_TRY(KK_LM_HEAD, launch_softcap_f32(m->logits, (size_t)n_out * m->vocab, m->softcap, st));
  return sample_rows(e, n_out, temperature, advance);
}

}  // namespace qie
