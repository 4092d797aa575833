// family.h -- what the model families with a general row forward share (Nogatar, Fosavik, Ditenex, Dedunex): the interface the engine
// drives them through (forward over rows, slot reset, release), the weight blob helpers (tensor layout, safetensors
// reader, synthetic fill), the rotary tables and the projection helper that puts a plain GEMM on the tcgen05 kernel when
// precision and shape allow.  A row is (sequence slot, position); rows of one sequence are consecutive and in position order
// (a "segment"); rows of different sequences may be portions of prompts next to single decoded tokens.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "common.cuh"

struct qie_engine;

namespace qie {

struct RowFamily {
  virtual ~RowFamily() {}
  virtual const char* family_name() const = 0;
  // one forward over n rows (ids_d / pos_d / slot_d staged; segments and output rows staged in seg_start / seg_slot /
  // out_rows, or one row per sequence when `advance`) -> logits [n_out, vocab] and sampled_d[0..n_out);
  // max_kv_len bounds position + 1 over the rows
  virtual cudaError_t forward(qie_engine* e, int n, int n_seg, int n_out, int max_kv_len, float temperature, bool advance) = 0;
  // a sequence slot is handed out again: recurrent state of its previous user is cleared
  virtual void reset_slot(qie_engine* e, int seq) = 0;
  // frees the device memory; the object itself is deleted by the caller
  virtual void release() = 0;
  virtual size_t layer_runs() const = 0;
  // logits (fp32 + the bf16 copy the top-k sampler reads), segment / output row lists and iota for `rows` rows
  cudaError_t alloc_row_buffers(size_t rows);
  void release_row_buffers();
  // the end of every forward: greedy arg-max on the fp32 logits (the bf16 sampler flips near-ties) or the engine's
  // top-k sampler on a bf16 copy; with `advance` the sampled tokens become the next step's inputs
  cudaError_t sample_rows(qie_engine* e, int n_out, float temperature, bool advance);

  int vocab = 0, width = 0;
  bool f32 = false;  // true 32-bit arithmetic everywhere; false: bf16 products / bf16 cache rows
  float* logits = nullptr;
  bf16* logits_bf = nullptr;
  int *seg_start = nullptr, *seg_slot = nullptr, *out_rows = nullptr;
  int* iota = nullptr;  // 0, 1, 2, ...: segments and output rows of a decode step (one row per sequence)
  // parity hook: residual stream after every layer of the last forward [layer runs, max_batch_tokens, width]
  float* layer_dump = nullptr;
  bool dump_layers = false;
};

// ---------------------------------------------------------------- weight blob
struct TensorSpec {
  std::string name;
  size_t rows = 0, cols = 0;  // cols 0 = vector of `rows`
  size_t off = 0;             // element offset in the blob
  int kind = 0;               // synthetic fill: 0 matrix (uniform, variance 1/cols), 1 norm weight (about 1), 2 small vector; 3: zeros that no file holds
  size_t elems() const { return rows * (cols ? cols : 1); }
};
// appends tensors to a layout; pad() starts the next group on a 256-byte boundary (tensors that one GEMM reads as a
// single matrix are added without a pad between them)
struct BlobLayout {
  std::vector<TensorSpec> t;
  size_t off = 0;
  void pad() { off = (off + 127) / 128 * 128; }
  void add(const std::string& name, size_t rows, size_t cols, int kind) {
    TensorSpec s;
    s.name = name, s.rows = rows, s.cols = cols, s.off = off, s.kind = kind;
    off += s.elems();
    t.push_back(s);
  }
  size_t elems() const { return t.empty() ? 0 : t.back().off + t.back().elems(); }
};
bool read_text_file(const std::string& path, std::string* out);
uint16_t f32_to_bf16_bits(float f);
void fill_synthetic_blob(const std::vector<TensorSpec>& t, uint64_t seed, std::vector<uint16_t>* blob);
// reads every tensor of the layout from a safetensors file (BF16 only; shapes are checked by element count) -> "" or the error
std::string load_safetensors_blob(const std::string& path, const std::vector<TensorSpec>& t, std::vector<uint16_t>* blob);

// ---------------------------------------------------------------- rotary positions
// Rotation angles of position p: a_i = p * f_i, f_i = base^(-2i / dims), i < dims / 2.  With `scaled` (YaRN) the
// frequencies are blended: with corr(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(corr(fast)), 0),
// hi = min(ceil(corr(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is
// f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1.
struct RotaryCfg {
  int dims = 0;
  double base = 10000.0;
  bool scaled = false;
  double factor = 1.0, original = 0.0, fast = 0.0, slow = 0.0;
  bool operator==(const RotaryCfg& o) const {
    return dims == o.dims && base == o.base && scaled == o.scaled && factor == o.factor && original == o.original && fast == o.fast &&
           slow == o.slow;
  }
};
// cos / sin tables [context, dims / 2], worked out in double, the magnitude factor folded in
void rotary_tables(const RotaryCfg& r, int context, std::vector<float>* c, std::vector<float>* s);
// what the kernels read: the tables on the device and how the rotated dimensions pair up
struct RopeTable {
  const float* cos_t = nullptr;  // [context, dims/2], scaled by the magnitude factor
  const float* sin_t = nullptr;
  int dims = 0;         // rotated leading dimensions
  int half_layout = 0;  // 0: pairs (2i, 2i+1); 1: pairs (i, i + dims/2)
};

// ---------------------------------------------------------------- projections on the tcgen05 GEMM
// C[n, N] = A[n, K] W[N, K]^T in bf16 serving precision and for more than 16 rows: A rows -> dense bf16, the tcgen05
// GEMM (gemm_tcgen05.cu), result bf16 -> fp32 rows of C (optional relu^2).  The operands and the result are the same
// bf16 values as on the fp32-accumulate path with round_a / round_c; only the summation order differs.
struct TcProjector {
  bool use = false;
  bf16 *ab = nullptr, *cb = nullptr;
  float* ws = nullptr;
  size_t ws_bytes = 0;
  int* counters = nullptr;
  void* maps = nullptr;  // std::map<const bf16*, TensorMap2D>*: weight descriptors by pointer
  cudaError_t alloc(size_t rows, size_t max_k, size_t max_n, cudaStream_t st);
  void release();
  bool fits(int n, int K, int N, const bf16* W) const;
  cudaError_t gemm(qie_engine* e, const float* A, int lda, const bf16* W, int K, int N, float* C, int ldc, int act, int n);
  // the GEMM alone, for callers whose producers write bf16 rows and whose consumers read them: A dense [n, K] -> C dense [n, N]
  cudaError_t gemm_bf16(qie_engine* e, const bf16* A, const bf16* W, int K, int N, bf16* C, int n);
};

}  // namespace qie

// launch + count + (when profiling) an event pair per launch, summed per kernel class by qie_profile_end
#define FAM_TRY(kind, expr)                                  \
  do {                                                       \
    qie_engine::ProfRec _r{kind, nullptr, nullptr};          \
    if (e->prof_on) {                                        \
      cudaEventCreate(&_r.a);                                \
      cudaEventCreate(&_r.b);                                \
      cudaEventRecord(_r.a, e->stream);                      \
    }                                                        \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return _e;                        \
    if (e->prof_on) {                                        \
      cudaEventRecord(_r.b, e->stream);                      \
      e->prof.push_back(_r);                                 \
    }                                                        \
    ++e->launches;                                           \
  } while (0)
