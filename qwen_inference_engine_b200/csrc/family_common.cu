// family_common.cu -- see family.h: weight blob helpers and the tcgen05 projection helper of the row-forward families.
#include "family.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>

#include "engine.h"
#include "json_min.h"

namespace qie {

bool read_text_file(const std::string& path, std::string* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  fseek(f, 0, SEEK_END);
  const long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  out->resize(n > 0 ? (size_t)n : 0);
  const size_t got = n > 0 ? fread(&(*out)[0], 1, (size_t)n, f) : 0;
  fclose(f);
  return got == out->size();
}

uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// counter hash -> uniform in [-1, 1)
static float hash_uniform(uint64_t seed, uint64_t i) {
  uint64_t z = seed + 0x9e3779b97f4a7c15ull * (i + 1);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  return (float)((double)(z >> 11) * (1.0 / 9007199254740992.0) * 2.0 - 1.0);
}

void fill_synthetic_blob(const std::vector<TensorSpec>& t, uint64_t seed, std::vector<uint16_t>* blob) {
  for (size_t k = 0; k < t.size(); ++k) {
    const TensorSpec& s = t[k];
    if (s.kind == 3) continue;  // zero rows between the parts of a fused matrix
    const float a = s.kind == 0 ? sqrtf(3.0f / (float)s.cols) : 0.f;
    for (size_t i = 0; i < s.elems(); ++i) {
      const float u = hash_uniform(seed + 1315423911ull * k, i);
      const float v = s.kind == 0 ? a * u : (s.kind == 1 ? 1.0f + 0.1f * u : 0.5f * u);
      (*blob)[s.off + i] = f32_to_bf16_bits(v);
    }
  }
}

std::string load_safetensors_blob(const std::string& path, const std::vector<TensorSpec>& t, std::vector<uint16_t>* blob) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return "cannot open " + path;
  unsigned char lenb[8];
  if (fread(lenb, 1, 8, f) != 8) return fclose(f), "short safetensors file " + path;
  uint64_t hl = 0;
  for (int i = 7; i >= 0; --i) hl = (hl << 8) | lenb[i];
  if (hl == 0 || hl > ((uint64_t)1 << 30)) return fclose(f), "bad safetensors header length in " + path;
  std::string hdr((size_t)hl, '\0');
  if (fread(&hdr[0], 1, (size_t)hl, f) != (size_t)hl) return fclose(f), "short safetensors header in " + path;
  JsonValue root;
  std::string err;
  if (!JsonReader::parse(hdr.data(), hdr.data() + hdr.size(), &root, &err)) return fclose(f), path + ": " + err;
  const size_t data0 = 8 + (size_t)hl;
  for (const TensorSpec& s : t) {
    if (s.kind == 3) continue;  // not in the file: zero rows between the parts of a fused matrix
    const JsonValue* rec = root.have(s.name.c_str());
    if (!rec) return fclose(f), "tensor " + s.name + " missing in " + path;
    const JsonValue* dt = rec->have("dtype");
    const JsonValue* sh = rec->have("shape");
    const JsonValue* of = rec->have("data_offsets");
    if (!dt || !sh || !of || of->arr.size() != 2) return fclose(f), "tensor " + s.name + ": malformed record";
    if (dt->str != "BF16") return fclose(f), "tensor " + s.name + ": dtype " + dt->str + " (only BF16 weights are loaded)";
    size_t n = 1;
    for (const JsonValue& dv : sh->arr) n *= (size_t)llround(dv.num);
    const size_t b0 = (size_t)llround(of->arr[0].num), b1 = (size_t)llround(of->arr[1].num);
    if (n != s.elems() || b1 - b0 != 2 * n) return fclose(f), "tensor " + s.name + ": shape does not fit the configuration";
    if (fseek(f, (long)(data0 + b0), SEEK_SET) != 0 || fread(&(*blob)[s.off], 2, n, f) != n) return fclose(f), "tensor " + s.name + ": short read";
  }
  fclose(f);
  return "";
}

cudaError_t RowFamily::alloc_row_buffers(size_t R) {
  cudaError_t r;
  if ((r = cudaMalloc(&logits, R * (size_t)vocab * sizeof(float))) != cudaSuccess) return r;
  if ((r = cudaMalloc(&logits_bf, R * (size_t)vocab * sizeof(bf16))) != cudaSuccess) return r;
  if ((r = cudaMalloc(&seg_start, (R + 1) * sizeof(int))) != cudaSuccess) return r;
  if ((r = cudaMalloc(&seg_slot, (R + 1) * sizeof(int))) != cudaSuccess) return r;
  if ((r = cudaMalloc(&out_rows, (R + 1) * sizeof(int))) != cudaSuccess) return r;
  if ((r = cudaMalloc(&iota, (R + 1) * sizeof(int))) != cudaSuccess) return r;
  std::vector<int> io(R + 1);
  for (size_t i = 0; i <= R; ++i) io[i] = (int)i;
  return cudaMemcpy(iota, io.data(), (R + 1) * sizeof(int), cudaMemcpyHostToDevice);
}

void RowFamily::release_row_buffers() {
  void* dev[] = {logits, logits_bf, seg_start, seg_slot, out_rows, iota, layer_dump};
  for (void* p : dev)
    if (p) cudaFree(p);
  logits = nullptr, logits_bf = nullptr, seg_start = seg_slot = out_rows = iota = nullptr, layer_dump = nullptr;
}

cudaError_t RowFamily::sample_rows(qie_engine* e, int n_out, float temperature, bool advance) {
  cudaStream_t st = e->stream;
  if (e->topk <= 1) {
    FAM_TRY(KK_SAMPLE, launch_argmax_f32(logits, e->sampled_d, n_out, vocab, st));
  } else {
    FAM_TRY(KK_SAMPLE, launch_cast_f32_bf16(logits, logits_bf, (size_t)n_out * vocab, st));
    FAM_TRY(KK_SAMPLE, launch_sample_topk(logits_bf, e->sampled_d, n_out, vocab, temperature, e->topk, e->seed, 0, e->add_step ? e->rowstep_d : nullptr, st));
  }
  if (advance) FAM_TRY(KK_ADVANCE, launch_advance(e->pos_d, e->ids_d, e->sampled_d, n_out, e->rowstep_d, st));
  return cudaSuccess;
}

void rotary_tables(const RotaryCfg& r, int context, std::vector<float>* c, std::vector<float>* s) {
  const int half = r.dims / 2;
  std::vector<double> f(half);
  double mag = 1.0;
  for (int i = 0; i < half; ++i) f[i] = pow(r.base, -2.0 * i / r.dims);
  if (r.scaled) {
    const double PI = 3.14159265358979323846;
    auto corr = [&](double turns) { return r.dims * log(r.original / (2.0 * PI * turns)) / (2.0 * log(r.base)); };
    const double lo = std::max(floor(corr(r.fast)), 0.0), hi = std::min(ceil(corr(r.slow)), (double)(r.dims - 1));
    for (int i = 0; i < half; ++i) {
      const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
      f[i] = f[i] / r.factor * ramp + f[i] * (1.0 - ramp);
    }
    mag = 0.1 * log(r.factor) + 1.0;
  }
  c->resize((size_t)context * half);
  s->resize((size_t)context * half);
  for (int p = 0; p < context; ++p)
    for (int i = 0; i < half; ++i) {
      (*c)[(size_t)p * half + i] = (float)(cos(p * f[i]) * mag);
      (*s)[(size_t)p * half + i] = (float)(sin(p * f[i]) * mag);
    }
}

cudaError_t TcProjector::alloc(size_t rows, size_t max_k, size_t max_n, cudaStream_t st) {
  cudaError_t r;
  if ((r = cudaMalloc(&ab, rows * max_k * sizeof(bf16))) != cudaSuccess) return r;
  if ((r = cudaMalloc(&cb, rows * max_n * sizeof(bf16))) != cudaSuccess) return r;
  ws_bytes = (size_t)64 << 20;
  if ((r = cudaMalloc(&ws, ws_bytes)) != cudaSuccess) return r;
  if ((r = cudaMalloc(&counters, 8192 * sizeof(int))) != cudaSuccess) return r;
  if ((r = cudaMemsetAsync(counters, 0, 8192 * sizeof(int), st)) != cudaSuccess) return r;
  maps = new std::map<const bf16*, TensorMap2D>();
  const char* v = getenv("QIE_NG_TC");
  use = !(v && v[0] == '0');
  return cudaSuccess;
}

void TcProjector::release() {
  delete static_cast<std::map<const bf16*, TensorMap2D>*>(maps);
  maps = nullptr;
  void* dev[] = {ab, cb, ws, counters};
  for (void* p : dev)
    if (p) cudaFree(p);
  ab = cb = nullptr, ws = nullptr, counters = nullptr;
}

bool TcProjector::fits(int n, int K, int N, const bf16* W) const {
  return use && maps && n > 16 && K >= 64 && K % 64 == 0 && N >= 128 && N % 8 == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0;
}

cudaError_t TcProjector::gemm(qie_engine* e, const float* A, int lda, const bf16* W, int K, int N, float* C, int ldc, int act, int n) {
  cudaError_t r = launch_rows_f32_to_bf16(A, lda, nullptr, ab, K, n, e->stream);
  if (r != cudaSuccess) return r;
  if ((r = gemm_bf16(e, ab, W, K, N, cb, n)) != cudaSuccess) return r;
  ++e->launches;
  return launch_rows_bf16_to_f32(cb, N, C, ldc, act, n, e->stream);
}

cudaError_t TcProjector::gemm_bf16(qie_engine* e, const bf16* A, const bf16* W, int K, int N, bf16* C, int n) {
  cudaStream_t st = e->stream;
  auto* mp = static_cast<std::map<const bf16*, TensorMap2D>*>(maps);
  auto it = mp->find(W);
  if (it == mp->end()) {
    TensorMap2D wm;
    cudaError_t r = make_tensor_map_2d(&wm, W, N, K, 128);
    if (r != cudaSuccess) return r;
    it = mp->emplace(W, wm).first;
  }
  cudaError_t r;
  TensorMap2D xmap;
  // many rows but few output columns (N = 1024 at 2048 rows: 64 tiles of 128 x 256): half-size token tiles fill the SMs without
  // the split over K and its reduction through the cluster
  int tile = tc_token_tile(n);
  static const bool small_on = [] { const char* v = getenv("QIE_TC_TILE128"); return !(v && v[0] == '0'); }();
  if (small_on && tile == 256 && (long)((N + 127) / 128) * ((n + 255) / 256) * 2 <= e->num_sms) tile = 128;
  if ((r = make_tensor_map_2d(&xmap, A, n, K, tile)) != cudaSuccess) return r;
  TcGemm t{};
  t.w[0] = &it->second;
  t.rows[0] = N;
  t.x = &xmap;
  t.nseg = 1;
  t.M = n;
  t.K = K;
  t.epi = EPI_STORE;
  t.out = C;
  t.ld_out = N;
  t.ws = ws;
  t.ws_bytes = ws_bytes;
  t.max_splits = (int)std::max<size_t>(1, ws_bytes / ((size_t)n * N * sizeof(float)));
  t.counters = counters;
  t.n_counters = 8192;
  t.token_tile = tile;
  t.w_static = 0;  // the operand comes from the kernel in front
  int nl = 0;
  if ((r = launch_gemm_tcgen05(t, e->num_sms, st, &nl)) != cudaSuccess) return r;
  e->launches += nl > 0 ? nl - 1 : 0;  // the caller counts one
  return cudaSuccess;
}

}  // namespace qie
