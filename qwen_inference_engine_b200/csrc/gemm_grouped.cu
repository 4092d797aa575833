// gemm_grouped.cu -- the expert GEMMs of a mixture of experts on tensor cores over bf16 rows (nogatar.h: GroupedGemmBf16):
// rows grouped by expert (grp_off), optionally gathered (row_idx), one weight matrix [N, K] per expert.  A CTA owns a
// 128 x 128 tile of one expert: 8 warps as 2 x 4, each 64 rows x 32 columns of mma.sync m16n8k16 with fp32 accumulators,
// operands staged through a 3-stage cp.async ring of 32 k-elements (rows padded to 40 elements: conflict-free ldmatrix).
// In the gated mode the expert's matrix is [gate rows | up rows] (N = 2 ff) and the tile's 128 weight rows are 64 gate
// rows interleaved in runs of 16 with the 64 up rows of the same columns, so that a thread holds silu's argument and
// its factor side by side and writes silu(gate) * up as bf16 -- the [gate | up] rows never go to memory.
// k ascends per output whatever the tile, so a row's result does not depend on the rows around it.
#include "launch.h"
#include "nogatar.h"

namespace qie {
namespace {

constexpr int BM = 128, BN = 128, BK = 32, BKP = 40, STAGES = 3;

__global__ void __launch_bounds__(256) grouped_gemm_bf16_kernel(const GroupedGemmBf16 g) {
  extern __shared__ __align__(16) unsigned char gg_smem[];
  typedef bf16 Tile[BM][BKP];
  Tile* As = reinterpret_cast<Tile*>(gg_smem);
  Tile* Bs = reinterpret_cast<Tile*>(gg_smem + STAGES * sizeof(Tile));
  __shared__ int a_row[BM];  // source row of each tile row (clamped to a valid one: rows past the group are computed and dropped)
  __shared__ int b_row[BN];  // weight row of each tile column
  pdl_wait();
  pdl_trigger();
  const int z = blockIdx.z;
  const int row_base = g.grp_off[z], Mz = g.grp_off[z + 1] - row_base;
  const int m0 = blockIdx.y * BM;
  if (m0 >= Mz) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_out = g.gated ? g.N / 2 : g.N;                      // output columns
  const int c0 = blockIdx.x * (g.gated ? BN / 2 : BN);            // first output column of the tile
  if (tid < BM) {
    const int m = min(m0 + tid, Mz - 1);
    a_row[tid] = g.row_idx ? g.row_idx[row_base + m] : row_base + m;
  } else {
    const int j = tid - BM;
    int r;
    if (g.gated) {  // runs of 16: gate columns, then the up rows of the same columns
      const int run = j >> 5, in = j & 31;
      const int col = min(c0 + run * 16 + (in & 15), n_out - 1);
      r = in < 16 ? col : n_out + col;
    } else {
      r = min(c0 + j, g.N - 1);
    }
    b_row[j] = r;
  }
  __syncthreads();
  const bf16* W = g.W + (size_t)z * g.w_batch;
  // a thread stages two 16-byte pieces of A and two of B per stage
  const int sr = tid >> 2, sc = (tid & 3) * 8;
  const bf16* a_src0 = g.A + (size_t)a_row[sr] * g.lda + sc;
  const bf16* a_src1 = g.A + (size_t)a_row[sr + 64] * g.lda + sc;
  const bf16* b_src0 = W + (size_t)b_row[sr] * g.K + sc;
  const bf16* b_src1 = W + (size_t)b_row[sr + 64] * g.K + sc;
  auto load = [&](int stage, int kt) {
    const int k = kt * BK;
    cp_async16(smem_u32(&As[stage][sr][sc]), a_src0 + k);
    cp_async16(smem_u32(&As[stage][sr + 64][sc]), a_src1 + k);
    cp_async16(smem_u32(&Bs[stage][sr][sc]), b_src0 + k);
    cp_async16(smem_u32(&Bs[stage][sr + 64][sc]), b_src1 + k);
  };
  const int KT = g.K / BK;
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < KT) load(s, s);
    cp_async_commit();
  }
  const int wm = (warp & 1) * 64, wn = (warp >> 1) * 32;
  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();  // stage kt has landed for every thread; stage kt - 1 is consumed and may be refilled
    const int nk = kt + STAGES - 1;
    if (nk < KT) load(nk % STAGES, nk);
    cp_async_commit();
    const int st = kt % STAGES;
#pragma unroll
    for (int ks = 0; ks < BK; ks += 16) {
      uint32_t a[4][4], b[4][2];
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
        ldmatrix_x4(a[mt][0], a[mt][1], a[mt][2], a[mt][3], smem_u32(&As[st][wm + mt * 16 + (lane & 15)][ks + (lane >> 4) * 8]));
#pragma unroll
      for (int np = 0; np < 2; ++np)
        ldmatrix_x4(b[2 * np][0], b[2 * np][1], b[2 * np + 1][0], b[2 * np + 1][1],
                    smem_u32(&Bs[st][wn + np * 16 + (lane >> 4) * 8 + (lane & 7)][ks + ((lane >> 3) & 1) * 8]));
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma_bf16_16816(acc[mt][nt], a[mt], b[nt][0], b[nt][1]);
    }
  }
  cp_async_wait<0>();
  const int gq = lane >> 2, tq = lane & 3;
  if (g.gated) {
    // the warp's 32 tile columns are [gate c .. c + 15 | up c .. c + 15]: n-tiles 0, 1 against 2, 3
    const int cw = c0 + (wn >> 5) * 16;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int m = m0 + wm + mt * 16 + gq + (u >> 1) * 8;
        if (m >= Mz) continue;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = cw + nt * 8 + 2 * tq + (u & 1);
          if (col >= n_out) continue;
          const float gate = acc[mt][nt][u], up = acc[mt][nt + 2][u];
          g.out_bf[(size_t)(row_base + m) * g.ldo + col] = f2bf(gate / (1.0f + expf(-gate)) * up);
        }
      }
  } else {
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int m = m0 + wm + mt * 16 + gq + (u >> 1) * 8;
        if (m >= Mz) continue;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int col = c0 + wn + nt * 8 + 2 * tq + (u & 1);
          if (col >= g.N) continue;
          g.out[(size_t)(row_base + m) * g.ldo + col] = acc[mt][nt][u];
        }
      }
  }
}

}  // namespace

bool grouped_gemm_bf16_fits(const GroupedGemmBf16& g) {
  return g.K >= BK && g.K % BK == 0 && g.lda % 8 == 0 && g.w_batch % 8 == 0 && (reinterpret_cast<uintptr_t>(g.A) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(g.W) & 15) == 0 && g.N > 0 && (!g.gated || g.N % 2 == 0);
}

cudaError_t launch_grouped_gemm_bf16(const GroupedGemmBf16& g, cudaStream_t st) {
  if (g.rows <= 0 || g.groups <= 0) return cudaSuccess;
  if (!grouped_gemm_bf16_fits(g) || !g.grp_off || (g.gated ? !g.out_bf : !g.out)) return cudaErrorInvalidValue;
  const size_t smem = (size_t)2 * STAGES * BM * BKP * sizeof(bf16);  // 60 KB
  static PerDeviceOnce set;
  if (set.need()) {
    cudaError_t r = cudaFuncSetAttribute(grouped_gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (r != cudaSuccess) return r;
    set.done();
  }
  const int n_out = g.gated ? g.N / 2 : g.N, per = g.gated ? BN / 2 : BN;
  const dim3 grid((n_out + per - 1) / per, (g.rows + BM - 1) / BM, g.groups);  // rows: the upper bound of any group; empty tiles leave at once
  return launch_k(grouped_gemm_bf16_kernel, grid, dim3(256), smem, st, g);
}

}  // namespace qie
