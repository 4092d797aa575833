// dedunex_model.cu -- the Dedunex family on the engine: configuration reader (config.json), weight loader
// (model.safetensors -> one device blob), the page pool shared by the key/value rows of the differential attention and the
// latent rows of the latent attention, the minGRU state slots, and the launch order of one forward over a batch of rows.
// A row is (sequence slot, position) exactly as in the other families; rows of one sequence are consecutive and in
// position order, rows of different sequences may be portions of prompts next to single decoded tokens.  Every size and
// constant comes from the configuration.  A layer inside the loop appears once per pass in `runs`, with cache rows or a
// state of its own.
#include "dedunex.h"

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
int up8(int v) { return (v + 7) & ~7; }

std::string parse_rot(const JsonValue* rt, int max_dims, RotaryCfg* r) {
  if (!rt) return "";  // no rotation
  r->dims = as_int(rt->have("dims"), 0);
  NEED(r->dims >= 0 && r->dims % 2 == 0 && r->dims <= max_dims, "config.json: rot.dims must be even and at most the rotated size");
  r->base = rt->have("base") ? rt->have("base")->num : 10000.0;
  NEED(r->base > 0.0, "config.json: rot.base");
  if (const JsonValue* sc = rt->have("scaling")) {
    r->scaled = true;
    r->factor = sc->have("factor") ? sc->have("factor")->num : 1.0;
    r->original = sc->have("original") ? sc->have("original")->num : 0.0;
    r->fast = sc->have("fast") ? sc->have("fast")->num : 0.0;
    r->slow = sc->have("slow") ? sc->have("slow")->num : 0.0;
    NEED(r->factor > 0.0 && r->original > 0.0 && r->fast > 0.0 && r->slow > 0.0, "config.json: rot.scaling needs factor, original, fast, slow");
  }
  return "";
}

std::string parse_config(const JsonValue& root, DdModel* m) {
  NEED(root.kind == JsonValue::Object, "config.json: not an object");
  m->vocab = as_int(root.have("vocab"), 0);
  m->width = as_int(root.have("width"), 0);
  NEED(m->vocab > 0 && m->width > 0, "config.json: vocab / width missing");
  if (const JsonValue* nm = root.have("norm")) {
    m->eps = as_float(nm->have("eps"), 1e-6f);
    m->groups = as_int(nm->have("groups"), 1);
  }
  NEED(m->groups > 0 && m->width % m->groups == 0, "config.json: norm.groups must divide the width");
  const JsonValue* layers = root.have("layers");
  NEED(layers && layers->kind == JsonValue::Array && !layers->arr.empty(), "config.json: layers missing");
  for (const JsonValue& jl : layers->arr) {
    DdLayer L;
    const JsonValue* type = jl.have("type");
    const JsonValue* mx = jl.have("mixer");
    NEED(type && type->kind == JsonValue::String && mx && mx->kind == JsonValue::Object, "config.json: layer without type / mixer");
    if (type->str == "attention") {
      L.type = 0;
      L.heads = as_int(mx->have("heads"), 0);
      L.kv_heads = as_int(mx->have("kv_heads"), L.heads);
      L.dim = as_int(mx->have("dim"), 0);
      L.vdim = as_int(mx->have("vdim"), L.dim);
      NEED(L.heads > 0 && L.kv_heads > 0 && L.dim > 0 && L.vdim > 0, "config.json: attention heads / kv_heads / dim / vdim missing");
      NEED(L.heads % L.kv_heads == 0, "config.json: heads must be a multiple of kv_heads");
      NEED(mx->have("scale") && mx->have("scale")->is_number(), "config.json: attention without scale");
      L.scale = (float)mx->have("scale")->num;
      L.softcap = as_float(mx->have("softcap"), 0.f);
      L.diff = as_float(mx->have("diff"), 0.f);
      if (const JsonValue* mk = mx->have("mask")) L.window = as_int(mk->have("size"), 0);
      const std::string err = parse_rot(mx->have("rot"), L.dim, &L.rot);
      if (!err.empty()) return err;
    } else if (type->str == "latent_attention") {
      L.type = 1;
      L.heads = as_int(mx->have("heads"), 0);
      L.dim = as_int(mx->have("dim"), 0);
      L.vdim = as_int(mx->have("vdim"), L.dim);
      L.rot_dim = as_int(mx->have("rot_dim"), 0);
      L.kv_rank = as_int(mx->have("kv_rank"), 0);
      L.q_rank = as_int(mx->have("q_rank"), 0);
      NEED(L.heads > 0 && L.dim > 0 && L.vdim > 0 && L.kv_rank > 0 && L.q_rank > 0 && L.rot_dim >= 0, "config.json: latent attention sizes missing");
      NEED(mx->have("scale") && mx->have("scale")->is_number(), "config.json: latent attention without scale");
      L.scale = (float)mx->have("scale")->num;
      const std::string err = parse_rot(mx->have("rot"), L.rot_dim, &L.rot);
      if (!err.empty()) return err;
    } else if (type->str == "mingru") {
      L.type = 2;
      L.gru_width = as_int(mx->have("width"), 0);
      NEED(L.gru_width > 0, "config.json: mingru without width");
    } else {
      return "config.json: unknown layer type '" + type->str + "'";
    }
    if (const JsonValue* mlp = jl.have("mlp")) {
      const JsonValue* kind = mlp->have("kind");
      NEED(kind && kind->kind == JsonValue::String && kind->str == "dense", "config.json: mlp.kind must be dense");
      L.ff = as_int(mlp->have("ff"), 0);
      NEED(L.ff > 0, "config.json: dense mlp without ff");
    }
    // the parts of the input projection, each starting at a multiple of 8 columns
    int a = 0, b = 0, c = 0;
    if (L.type == 0) a = L.heads * 2 * L.dim, b = L.kv_heads * 2 * L.dim, c = L.kv_heads * L.vdim;
    else if (L.type == 1) a = L.q_rank, b = L.kv_rank + L.rot_dim, c = L.heads;
    else a = b = c = L.gru_width;
    L.o_a = 0, L.o_b = up8(a), L.o_c = L.o_b + up8(b), L.o_gate = L.o_c + up8(c), L.o_up = L.o_gate + up8(L.ff), L.n_in = L.o_up + up8(L.ff);
    m->layers.push_back(L);
  }
  const int NL = (int)m->layers.size();
  m->loop_start = m->loop_stop = 0, m->loop_times = 1;
  if (const JsonValue* lp = root.have("loop")) {
    m->loop_start = as_int(lp->have("start"), 0);
    m->loop_stop = as_int(lp->have("stop"), m->loop_start);
    m->loop_times = as_int(lp->have("times"), 1);
    NEED(m->loop_start >= 0 && m->loop_start <= m->loop_stop && m->loop_stop <= NL && m->loop_times >= 1, "config.json: loop start / stop / times");
  }
  for (int i = 0; i < m->loop_start; ++i) m->runs.push_back(DdRun{i, -1, 0, 0});
  if (m->loop_stop > m->loop_start)
    for (int t = 0; t < m->loop_times; ++t)
      for (int i = m->loop_start; i < m->loop_stop; ++i) m->runs.push_back(DdRun{i, i == m->loop_start ? t : -1, 0, 0});
  for (int i = m->loop_stop; i < NL; ++i) m->runs.push_back(DdRun{i, -1, 0, 0});
  return "";
}

// tensors in blob order.  A layer's input projections and the feed-forward's gate and up are ONE matrix (one GEMM of the
// normed input); its parts start at multiples of 8 rows, the rows between them stay zero (kind 3: not in the file).
std::vector<TensorSpec> build_layout(const DdModel& m) {
  BlobLayout bl;
  auto pad = [&]() { bl.pad(); };
  auto add = [&](const std::string& name, size_t rows, size_t cols, int kind) { bl.add(name, rows, cols, kind); };
  const size_t W = m.width;
  pad(), add("embed", m.vocab, W, 0);
  pad(), add("embed.norm", W, 0, 1);
  if (m.loop_stop > m.loop_start) pad(), add("loop.step", m.loop_times, W, 2);
  for (size_t i = 0; i < m.layers.size(); ++i) {
    const DdLayer& L = m.layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    int at = 0;
    auto part = [&](const std::string& name, int rows, int off) {  // zero rows up to the part's offset, then the part
      if (off > at) add(p + "zero" + std::to_string(off), off - at, W, 3);
      add(name, rows, W, 0);
      at = off + rows;
    };
    pad(), add(p + "norm1", W, 0, 1);
    pad();
    if (L.type == 0) {
      part(p + "mix.q", L.heads * 2 * L.dim, L.o_a), part(p + "mix.k", L.kv_heads * 2 * L.dim, L.o_b), part(p + "mix.v", L.kv_heads * L.vdim, L.o_c);
    } else if (L.type == 1) {
      part(p + "mix.dq", L.q_rank, L.o_a), part(p + "mix.dkv", L.kv_rank + L.rot_dim, L.o_b), part(p + "mix.g", L.heads, L.o_c);
    } else {
      part(p + "mix.z", L.gru_width, L.o_a), part(p + "mix.x", L.gru_width, L.o_b), part(p + "mix.g", L.gru_width, L.o_c);
    }
    if (L.ff > 0) part(p + "mlp.gate", L.ff, L.o_gate), part(p + "mlp.up", L.ff, L.o_up);
    if (L.n_in > at) add(p + "zero" + std::to_string(L.n_in), L.n_in - at, W, 3);
    if (L.type == 0) {
      const size_t d = L.dim;
      pad(), add(p + "mix.q.b", L.heads * 2 * d, 0, 2);
      pad(), add(p + "mix.k.b", L.kv_heads * 2 * d, 0, 2);
      pad(), add(p + "mix.v.b", L.kv_heads * L.vdim, 0, 2);
      pad(), add(p + "mix.q.norm", d, 0, 1);
      pad(), add(p + "mix.k.norm", d, 0, 1);
      pad(), add(p + "mix.lq1", d, 0, 2), add(p + "mix.lk1", d, 0, 2), add(p + "mix.lq2", d, 0, 2), add(p + "mix.lk2", d, 0, 2);
      pad(), add(p + "mix.o", W, (size_t)L.heads * L.vdim, 0);
    } else if (L.type == 1) {
      pad(), add(p + "mix.dq.norm", L.q_rank, 0, 1);
      pad(), add(p + "mix.dkv.norm", L.kv_rank, 0, 1);
      pad(), add(p + "mix.uq", (size_t)L.heads * (L.dim + L.rot_dim), L.q_rank, 0);
      pad(), add(p + "mix.uk", (size_t)L.heads * L.dim, L.kv_rank, 0);
      pad(), add(p + "mix.uv", (size_t)L.heads * L.vdim, L.kv_rank, 0);
      pad(), add(p + "mix.o", W, (size_t)L.heads * L.vdim, 0);
    } else {
      pad(), add(p + "mix.z.b", L.gru_width, 0, 2);
      pad(), add(p + "mix.x.b", L.gru_width, 0, 2);
      pad(), add(p + "mix.o", W, L.gru_width, 0);
    }
    if (L.ff > 0) pad(), add(p + "mlp.down", W, L.ff, 0);
  }
  pad(), add("final.norm", W, 0, 1);
  pad(), add("head", m.vocab, W, 0);
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
  DdModel* m = e->dd;
  const qie_engine_opts& o = e->opts;
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
  m->embed = P("embed"), m->embed_norm = P("embed.norm"), m->loop_step = P("loop.step"), m->final_norm = P("final.norm"), m->head = P("head");
  e->cfg = qie_config{m->width, 0, (int)m->runs.size(), 0, 0, 0, m->vocab, o.context};
  const size_t W = m->width;
  size_t w0 = 1, w1 = 1, w2 = 1, w3 = 1, wff = 1, wq = 1, hmv = 1, maxk = W, maxn = W, max_gru = 1;
  for (size_t i = 0; i < m->layers.size(); ++i) {
    DdLayer& L = m->layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const size_t H = L.heads, G = L.kv_heads, d = L.dim, vd = L.vdim;
    L.norm1 = P(p + "norm1"), L.wo = P(p + "mix.o"), L.w_down = P(p + "mlp.down");
    w0 = std::max(w0, (size_t)L.n_in), maxn = std::max(maxn, (size_t)L.n_in);
    if (L.ff > 0) wff = std::max(wff, (size_t)L.ff), maxk = std::max(maxk, (size_t)L.ff);
    if (L.type == 0) {
      L.w_in = P(p + "mix.q");
      L.q_b = P(p + "mix.q.b"), L.k_b = P(p + "mix.k.b"), L.v_b = P(p + "mix.v.b"), L.q_norm = P(p + "mix.q.norm"), L.k_norm = P(p + "mix.k.norm");
      double s1 = 0.0, s2 = 0.0;  // lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number of the layer
      const TensorSpec *a1 = at[p + "mix.lq1"], *b1 = at[p + "mix.lk1"], *a2 = at[p + "mix.lq2"], *b2 = at[p + "mix.lk2"];
      for (size_t k = 0; k < d; ++k) {
        s1 += (double)bits_to_float(blob[a1->off + k]) * bits_to_float(blob[b1->off + k]);
        s2 += (double)bits_to_float(blob[a2->off + k]) * bits_to_float(blob[b2->off + k]);
      }
      L.lam = (float)(exp(s1) - exp(s2) + (double)L.diff);
      w1 = std::max(w1, H * vd), maxk = std::max(maxk, H * vd);
      hmv = std::max(hmv, H * 2 * (vd + 2));
    } else if (L.type == 1) {
      const size_t r = L.rot_dim, kr = L.kv_rank;
      L.w_in = P(p + "mix.dq");
      L.dq_norm = P(p + "mix.dq.norm"), L.dkv_norm = P(p + "mix.dkv.norm"), L.wuq = P(p + "mix.uq"), L.wuk = P(p + "mix.uk"), L.wuv = P(p + "mix.uv");
      w1 = std::max(w1, H * (kr + r));
      w2 = std::max(w2, std::max(H * (d + r), H * vd));
      w3 = std::max(w3, std::max(H * kr, (size_t)L.q_rank));
      wq = std::max(wq, (size_t)L.q_rank);
      maxk = std::max(maxk, std::max((size_t)L.q_rank, H * vd));
      maxn = std::max(maxn, H * (d + r));
      hmv = std::max(hmv, H * (kr + 2));
    } else {
      L.w_in = P(p + "mix.z");
      L.z_b = P(p + "mix.z.b"), L.x_b = P(p + "mix.x.b");
      w1 = std::max(w1, (size_t)L.gru_width), maxk = std::max(maxk, (size_t)L.gru_width);
      max_gru = std::max(max_gru, (size_t)L.gru_width);
    }
    if (L.type != 2 && L.rot.dims > 0) {
      size_t id = 0;
      while (id < m->rope_cfg.size() && !(m->rope_cfg[id] == L.rot)) ++id;
      if (id == m->rope_cfg.size()) m->rope_cfg.push_back(L.rot);
      L.rope_id = (int)id;
    }
  }
  for (const RotaryCfg& r : m->rope_cfg) {
    std::vector<float> c, s;
    rotary_tables(r, o.context, &c, &s);
    float *cd = nullptr, *sd = nullptr;
    CUS(cudaMalloc(&cd, std::max<size_t>(c.size(), 1) * sizeof(float)));
    CUS(cudaMalloc(&sd, std::max<size_t>(s.size(), 1) * sizeof(float)));
    CUS(cudaMemcpy(cd, c.data(), c.size() * sizeof(float), cudaMemcpyHostToDevice));
    CUS(cudaMemcpy(sd, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice));
    m->rope_cos.push_back(cd), m->rope_sin.push_back(sd);
  }
  // cache rows and state of every run: a page holds page_size positions of every caching run, each run's block of rows
  // starting at a multiple of 8 elements
  size_t page_elems = 0, slot_floats = 0;
  for (DdRun& r : m->runs) {
    const DdLayer& L = m->layers[r.layer];
    if (L.type == 0) r.kv_off = page_elems, page_elems += ((size_t)o.page_size * (L.kv_heads * 2 * L.dim + L.kv_heads * L.vdim) + 7) / 8 * 8;
    else if (L.type == 1) r.kv_off = page_elems, page_elems += ((size_t)o.page_size * (L.kv_rank + L.rot_dim) + 7) / 8 * 8;
    else r.state_off = slot_floats, slot_floats += ((size_t)L.gru_width + 3) / 4 * 4;
  }
  m->page_elems = page_elems;
  const size_t elt = m->f32 ? 4 : 2;
  const size_t page_bytes = std::max<size_t>(page_elems * elt, 16);
  int n_pages = o.max_pages;
  if (n_pages <= 0) n_pages = (int)std::max<size_t>(1, (o.kv_bytes ? o.kv_bytes : ((size_t)1 << 30)) / page_bytes);
  CUS(cudaMalloc(&m->kv_pool, (size_t)n_pages * page_bytes));
  CUS(cudaMemsetAsync(m->kv_pool, 0, (size_t)n_pages * page_bytes, e->stream));
  e->kv = KvGeom{nullptr, n_pages, o.page_size, (int)m->runs.size(), 1, 0};
  CUS(engine_alloc_shared(e, n_pages, o.context));
  m->slot_floats = std::max<size_t>(slot_floats, 4);
  CUS(cudaMalloc(&m->state, (size_t)o.max_seqs * m->slot_floats * sizeof(float)));
  CUS(cudaMemsetAsync(m->state, 0, (size_t)o.max_seqs * m->slot_floats * sizeof(float), e->stream));
  // activations
  const size_t R = o.max_batch_tokens;
  auto fbuf = [&](float** p, size_t n) { return cudaMalloc(p, std::max<size_t>(n, 4) * sizeof(float)); };
  CUS(fbuf(&m->x, R * W));
  CUS(fbuf(&m->hn, R * W));
  CUS(fbuf(&m->p0, R * w0));
  CUS(fbuf(&m->p1, R * w1));
  CUS(fbuf(&m->p2, R * std::max(w2, wff)));  // the feed-forward's hidden rows share it with the latent attention's queries
  CUS(fbuf(&m->p3, R * w3));
  CUS(fbuf(&m->y1, R * W));
  CUS(fbuf(&m->y2, R * W));
  CUS(fbuf(&m->xo, R * W));
  m->attn_ws_floats = (R + 2048) * hmv;  // room for key splits when a step has few rows
  CUS(fbuf(&m->attn_ws, m->attn_ws_floats));
  m->scan_ws_floats = mingru_ws_floats(R, (size_t)o.max_seqs, (int)max_gru);
  CUS(fbuf(&m->scan_ws, m->scan_ws_floats));
  if (!m->f32) {
    CUS(m->tc.alloc(R, maxk, std::max(maxn, (size_t)m->vocab), e->stream));
    auto bbuf = [&](bf16** p, size_t n) { return cudaMalloc(p, std::max<size_t>(n, 8) * sizeof(bf16)); };
    CUS(bbuf(&m->hb, R * W));
    CUS(bbuf(&m->mb, R * w1));
    CUS(bbuf(&m->fb, R * wff));
    CUS(bbuf(&m->qb, R * wq));
    CUS(bbuf(&m->y1b, R * W));
    CUS(bbuf(&m->y2b, R * W));
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
  e->dd = new DdModel();
  e->fam = e->dd;
  err = parse_config(root, e->dd);
  if (!err.empty()) return err;
  const std::vector<TensorSpec> t = build_layout(*e->dd);
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

std::string dedunex_create(qie_engine* e, const std::string& dir, int* code) {
  std::string cfg;
  *code = QIE_EIO;
  if (!read_text_file(dir + "/config.json", &cfg)) return "cannot read " + dir + "/config.json";
  const std::string st = dir + "/model.safetensors";
  return create_common(e, cfg, &st, 0, code);
}

std::string dedunex_create_synthetic(qie_engine* e, const std::string& cfg_json, uint64_t seed, int* code) {
  return create_common(e, cfg_json, nullptr, seed, code);
}

void DdModel::release() {
  void* dev[] = {blob, kv_pool, state, x, hn, p0, p1, p2, p3, y1, y2, xo, attn_ws, scan_ws, hb, mb, fb, qb, y1b, y2b};
  tc.release();
  release_row_buffers();
  for (void* p : dev)
    if (p) cudaFree(p);
  for (float* p : rope_cos)
    if (p) cudaFree(p);
  for (float* p : rope_sin)
    if (p) cudaFree(p);
}

void DdModel::reset_slot(qie_engine* e, int seq) {
  if (state) cudaMemsetAsync(state + (size_t)seq * slot_floats, 0, slot_floats * sizeof(float), e->stream);
}

cudaError_t DdModel::forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) {
  DdModel* m = this;
  cudaStream_t st = e->stream;
  const int W = m->width;
  const int rnd = m->f32 ? 0 : 1;  // bf16 serving precision: the operands of the projections are bf16 values
  const int* segs = advance ? m->iota : m->seg_start;
  const int* seg_sl = advance ? e->slot_d : m->seg_slot;
  const int* outs = advance ? m->iota : m->out_rows;
  const size_t R = e->opts.max_batch_tokens;
  // plain projection C[rows, N] = A[rows, K] Wt[N, K]^T on the fp32-accumulate kernels (tensor cores on bf16 operands,
  // plain fp32 in 32-bit mode, a warp-per-column GEMV for a decode step)
  auto proj = [&](const float* A, int lda, const bf16* Wt, int K, int N, float* C, int ldc, int rows) {
    GemmF32 g;
    g.A = A, g.lda = lda, g.W = Wt, g.ldw = K, g.C = C, g.ldc = ldc, g.M = rows, g.N = N, g.K = K, g.round_a = rnd;
    return launch_gemm_f32(g, st);
  };
  // bf16 precision and a GEMM the tcgen05 kernel takes: its producer writes bf16 rows and its consumer reads them
  auto tcfit = [&](int K, int N, const bf16* Wt) { return !m->f32 && m->tc.fits(n, K, N, Wt); };
  if (m->dump_layers && !m->layer_dump)
    if (cudaMalloc(&m->layer_dump, m->runs.size() * R * W * sizeof(float)) != cudaSuccess) return cudaErrorMemoryAllocation;
  // the two sublayer outputs of the run before, waiting to be added to the stream by the next norm step
  const float *py1 = nullptr, *py2 = nullptr;
  const bf16 *py1b = nullptr, *py2b = nullptr;
  for (size_t ri = 0; ri < m->runs.size(); ++ri) {
    const DdRun& run = m->runs[ri];
    const DdLayer& L = m->layers[run.layer];
    const int ld = L.n_in;
    const bool tc_in = tcfit(W, L.n_in, L.w_in);
    {  // x += outputs of the run before (first run: the normed embedding row); the pass vector; h = norm(x)
      GroupNormStep s;
      s.x = m->x, s.width = W, s.groups = m->groups, s.n = n, s.eps = m->eps;
      if (ri == 0) s.ids = e->ids_d, s.embed = m->embed, s.w_pre = m->embed_norm;
      s.y1 = py1, s.y2 = py2, s.y1_bf = py1b, s.y2_bf = py2b;
      if (ri > 0 && m->dump_layers) s.dump = m->layer_dump + (ri - 1) * R * W;
      if (run.pass >= 0) s.step = m->loop_step + (size_t)run.pass * W;
      s.w_in = L.norm1;
      if (tc_in) s.h_bf = m->hb;
      else s.h = m->hn;
      FAM_TRY(KK_F32_NORM, launch_group_norm_step(s, st));
    }
    py1 = py2 = nullptr, py1b = py2b = nullptr;
    // one GEMM of the normed input: the mixer's projections and the feed-forward's gate and up
    GatedAct ga;
    ga.ff = L.ff, ga.act = 1, ga.n = n;
    if (tc_in) {
      FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, m->hb, L.w_in, W, L.n_in, m->tc.cb, n));
      if (L.type != 2)  // the mixer's part as fp32 rows (the minGRU scan reads the bf16 rows themselves)
        FAM_TRY(KK_F32_PROJ, launch_rows_bf16_to_f32_ld(m->tc.cb, ld, L.o_gate, m->p0, ld, n, st));
      ga.g_bf = m->tc.cb + L.o_gate, ga.u_bf = m->tc.cb + L.o_up, ga.ld_bf = ld;
    } else {
      FAM_TRY(KK_F32_PROJ, proj(m->hn, W, L.w_in, W, L.n_in, m->p0, ld, n));
      ga.g = m->p0 + L.o_gate, ga.u = m->p0 + L.o_up, ga.ld = ld;
    }
    // feed-forward first: the mixer's GEMMs reuse the buffer the input projection's bf16 result lies in
    if (L.ff > 0) {
      if (tc_in && tcfit(L.ff, W, L.w_down)) {
        ga.out_bf = m->fb, ga.ldo_bf = L.ff;
        FAM_TRY(KK_GLU, launch_gated_act(ga, st));
        FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, m->fb, L.w_down, L.ff, W, m->y2b, n));
        py2b = m->y2b;
      } else {
        float* fh = m->p2;
        ga.out = fh, ga.ldo = L.ff;
        FAM_TRY(KK_GLU, launch_gated_act(ga, st));
        FAM_TRY(KK_F32_PROJ, proj(fh, L.ff, L.w_down, L.ff, W, m->y2, W, n));
        py2 = m->y2;
      }
    }
    // the mixer's output rows [n, Km] -> y1 = W_o rows: bf16 rows straight into the tcgen05 GEMM where it fits
    int Km = 0;
    const float* mix_f = nullptr;  // fp32 rows of the mixer's output (row stride Km); null: they are in mb as bf16
    if (L.type == 0) {
      const int H = L.heads, G = L.kv_heads, d = L.dim, vd = L.vdim;
      KvRowCache c;
      c.pool = m->kv_pool, c.elt_bytes = m->f32 ? 4 : 2, c.page_size = e->kv.page_size, c.page_elems = m->page_elems;
      c.layer_off = run.kv_off, c.kw = G * 2 * d, c.vw = G * vd;
      RopeTable rope;
      if (L.rope_id >= 0) rope = RopeTable{m->rope_cos[L.rope_id], m->rope_sin[L.rope_id], L.rot.dims, 1};
      {  // keys (bias, norm per head and map, rotation) and values (bias) -> cache rows; the queries alike, in place
        KvStoreArgs ks;
        ks.c = c, ks.k = m->p0 + L.o_b, ks.ldk = ld, ks.v = m->p0 + L.o_c, ks.ldv = ld;
        ks.k_bias = L.k_b, ks.v_bias = L.v_b, ks.k_norm = L.k_norm, ks.norm_dim = d, ks.eps = m->eps;
        ks.q = m->p0 + L.o_a, ks.ldq = ld, ks.q_heads = H * 2, ks.q_norm = L.q_norm, ks.q_bias = L.q_b, ks.rope = rope;
        ks.pos = e->pos_d, ks.slot = e->slot_d, ks.block_table = e->block_table_d, ks.max_pages = e->max_pages_per_seq, ks.n = n;
        FAM_TRY(KK_KV_STORE, launch_kv_store_rows(ks, st));
      }
      GqaAttnArgs g;
      g.c = c, g.q = m->p0 + L.o_a, g.ldq = ld, g.out = m->p1, g.ldo = H * vd;
      g.heads = H, g.kv_heads = G, g.dim = d, g.vdim = vd, g.maps = 2, g.scale = L.scale, g.softcap = L.softcap, g.window = L.window;
      g.finish = 2, g.lam = L.lam, g.post = 1.0f - L.diff, g.eps = m->eps;
      g.pos = e->pos_d, g.slot = e->slot_d, g.block_table = e->block_table_d, g.max_pages = e->max_pages_per_seq, g.n = n, g.max_keys = max_kv_len;
      g.ws = m->attn_ws, g.ws_floats = m->attn_ws_floats, g.num_sms = e->num_sms;
      g.seg_start = segs, g.seg_slot = seg_sl, g.n_seg = n_seg;
      const bool tc_o = tcfit(H * vd, W, L.wo);
      if (tc_o) g.out_bf = m->mb, g.ldo_bf = H * vd;  // bf16 rows for the output projection (the fp32 rows hold the first map meanwhile)
      int nl = 0;
      FAM_TRY(KK_GQA_ATTN, launch_gqa_attention(g, st, &nl));
      e->launches += nl > 0 ? nl - 1 : 0;
      Km = H * vd, mix_f = tc_o ? nullptr : m->p1;
    } else if (L.type == 1) {
      const int H = L.heads, d = L.dim, vd = L.vdim, r = L.rot_dim, kr = L.kv_rank, D = kr + r, Nq = H * (d + r), qk = L.q_rank;
      LatentCache c;
      c.pool = m->kv_pool, c.elt_bytes = m->f32 ? 4 : 2, c.page_size = e->kv.page_size, c.page_elems = m->page_elems;
      c.layer_off = run.kv_off, c.rank = kr, c.rot = r;
      RopeTable rope;
      if (L.rope_id >= 0) rope = RopeTable{m->rope_cos[L.rope_id], m->rope_sin[L.rope_id], L.rot.dims, 1};
      const bool tc_uq = tcfit(qk, Nq, L.wuq);
      {  // normed latent and rotated shared key -> cache row; the query latent is normed by the same launch
        RowNorm qn;
        qn.src = m->p0 + L.o_a, qn.ld_src = ld, qn.width = qk, qn.w = L.dq_norm;
        if (tc_uq) qn.dst_bf = m->qb, qn.ld_dst_bf = qk;
        else qn.dst = m->p3, qn.ld_dst = qk;
        FAM_TRY(KK_LATENT_STORE, launch_latent_store(c, m->p0 + L.o_b, ld, L.dkv_norm, m->eps, rope, e->pos_d, e->slot_d, e->block_table_d,
                                                     e->max_pages_per_seq, n, st, QueryRope(), qn));
      }
      if (tc_uq) {
        FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, m->qb, L.wuq, qk, Nq, m->tc.cb, n));
        FAM_TRY(KK_F32_PROJ, launch_rows_bf16_to_f32(m->tc.cb, Nq, m->p2, Nq, 0, n, st));
      } else {
        FAM_TRY(KK_F32_PROJ, proj(m->p3, qk, L.wuq, qk, Nq, m->p2, Nq, n));
      }
      // qa[:, h] = [W_uk,h^T q_h (unrotated part) | rotated part of q_h]: the score against a cached row is one dot product
      if (r > 0) FAM_TRY(KK_LATENT_STORE, launch_rope_heads_f32(m->p2 + d, Nq, d + r, m->p1 + kr, H * D, D, H, r, rope, e->pos_d, n, st));
      {
        GemmF32 g;
        g.A = m->p2, g.lda = Nq, g.a_batch = d + r;
        g.W = L.wuk, g.ldw = kr, g.w_batch = (long)d * kr, g.w_trans = 1;
        g.C = m->p1, g.ldc = H * D, g.c_batch = D;
        g.M = n, g.N = kr, g.K = d, g.batches = H, g.round_a = rnd;
        FAM_TRY(KK_F32_PROJ, launch_gemm_f32(g, st));
      }
      HeadGate hg;
      hg.z = m->p0 + L.o_c, hg.ld = ld;
      FAM_TRY(KK_LATENT_ATTN, launch_latent_attention(c, m->p1, m->p3, nullptr, L.scale, 0, H, e->pos_d, e->slot_d, e->block_table_d,
                                                       e->max_pages_per_seq, n, max_kv_len, m->attn_ws, m->attn_ws_floats, st, hg));
      {  // value up-projection of the attended (and gated) latent, head by head
        GemmF32 g;
        g.A = m->p3, g.lda = H * kr, g.a_batch = kr;
        g.W = L.wuv, g.ldw = kr, g.w_batch = (long)vd * kr;
        g.C = m->p2, g.ldc = H * vd, g.c_batch = vd;
        g.M = n, g.N = vd, g.K = kr, g.batches = H, g.round_a = rnd;
        FAM_TRY(KK_F32_PROJ, launch_gemm_f32(g, st));
      }
      Km = H * vd, mix_f = m->p2;
    } else {
      const int C = L.gru_width;
      const bool tc_o = tcfit(C, W, L.wo);
      MinGruArgs a;
      if (tc_in) a.zp_bf = m->tc.cb + L.o_a, a.up_bf = m->tc.cb + L.o_b, a.gp_bf = m->tc.cb + L.o_c, a.ld_bf = ld;  // the scan reads the GEMM's bf16 result
      else a.zp = m->p0 + L.o_a, a.up = m->p0 + L.o_b, a.gp = m->p0 + L.o_c, a.ld = ld;
      a.z_bias = L.z_b, a.u_bias = L.x_b, a.channels = C;
      if (tc_o) a.out_bf = m->mb, a.ldo_bf = C;
      else a.out = m->p1, a.ldo = C;
      a.state = m->state + run.state_off, a.slot_stride = m->slot_floats;
      a.seg_start = segs, a.seg_slot = seg_sl, a.n_seg = n_seg, a.n_rows = n;
      a.ws = m->scan_ws, a.ws_floats = m->scan_ws_floats;
      FAM_TRY(KK_LRU_SCAN, launch_mingru_scan(a, st));
      Km = C, mix_f = tc_o ? nullptr : m->p1;
    }
    if (tcfit(Km, W, L.wo)) {
      const bf16* A = m->mb;
      if (mix_f) {
        FAM_TRY(KK_F32_PROJ, launch_rows_f32_to_bf16(mix_f, Km, nullptr, m->tc.ab, Km, n, st));
        A = m->tc.ab;
      }
      FAM_TRY(KK_F32_PROJ, m->tc.gemm_bf16(e, A, L.wo, Km, W, m->y1b, n));
      py1b = m->y1b;
    } else {
      FAM_TRY(KK_F32_PROJ, proj(mix_f, Km, L.wo, Km, W, m->y1, W, n));
      py1 = m->y1;
    }
  }
  if (m->dump_layers) {  // the last run's outputs meet the stream in every row, not only in the output rows
    GroupNormStep s;
    s.x = m->x, s.width = W, s.groups = m->groups, s.n = n, s.eps = m->eps;
    s.y1 = py1, s.y2 = py2, s.y1_bf = py1b, s.y2_bf = py2b;
    s.dump = m->layer_dump + (m->runs.size() - 1) * R * W;
    FAM_TRY(KK_F32_NORM, launch_group_norm_step(s, st));
    py1 = py2 = nullptr, py1b = py2b = nullptr;
  }
  if (n_out <= 0) return cudaSuccess;
  {
    GroupNormStep s;
    s.x = m->x, s.width = W, s.groups = m->groups, s.n = n_out, s.eps = m->eps;
    s.y1 = py1, s.y2 = py2, s.y1_bf = py1b, s.y2_bf = py2b;
    s.w_in = m->final_norm, s.h = m->xo, s.gather = outs;
    FAM_TRY(KK_F32_NORM, launch_group_norm_step(s, st));
  }
  {
    GemmF32 g;
    g.A = m->xo, g.lda = W, g.W = m->head, g.ldw = W, g.C = m->logits, g.ldc = m->vocab, g.M = n_out, g.N = m->vocab, g.K = W, g.round_a = rnd;
    FAM_TRY(KK_LM_HEAD, launch_gemm_f32(g, st));
  }
  return sample_rows(e, n_out, temperature, advance);
}

}  // namespace qie
