// Plain matrix product on the CUDA cores, true 32-bit: out[m,n] = sum_k A[m,k] * W[n,k].
//
// This is the product of the float32 path and the reference twin of the tensor-core
// kernels.  Every output element is one chain of FFMAs over k in ascending order that
// starts from zero, whatever M is and whichever tile the element falls into, so a row's
// result does not depend on what else is in the batch.  (The reference's kernel sums
// 16-wide k tiles in ascending order too: src/hip_ops.hip:43-64.)
//
// Options, all of them orthogonal:
//   a_rows    gather: row m of A is A[a_rows[m], :]
//   grouped   W is [E, Nw, K]; M-tiles are listed in (tile_expert, tile_row0, tile_rows) and
//             each uses its own expert's matrix; rows are positions in an expert-sorted list
//   swiglu    W holds 2N rows, gate rows [0,N) then up rows [N,2N); out = silu(g) * u
//   bias      fp32 or bf16 vector of N, added after the sum
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

struct GemmArgs {
  const void* A;
  const void* W;
  const void* bias;
  void* out;
  const int* a_rows;
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tiles;  // device scalar (grouped) or null
  long long lda, ldo;
  long long w_expert_stride;  // elements between experts' matrices
  int M, N, K;
  int bias_dt, out_dt;
  int swiglu;
};

template <typename TA, typename TW, bool SWIGLU>
__global__ void __launch_bounds__(256) gemm_plain_kernel(GemmArgs g) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  __shared__ float B2s[SWIGLU ? BK : 1][BN + 4];

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  int row0, rows_here;
  const TW* W = (const TW*)g.W;
  if (g.tile_expert) {
    if ((int)blockIdx.y >= *g.num_tiles) return;
    row0 = g.tile_row0[blockIdx.y];
    rows_here = g.tile_rows[blockIdx.y];
    W += (size_t)g.tile_expert[blockIdx.y] * g.w_expert_stride;
  } else {
    row0 = blockIdx.y * BM;
    rows_here = min(BM, g.M - row0);
  }
  const int col0 = blockIdx.x * BN;
  const TA* A = (const TA*)g.A;

  // which rows of A this thread stages: 64 rows x 16 k = 1024 elements, 4 per thread
  float acc[TM][TN] = {};
  float acc2[SWIGLU ? TM : 1][TN] = {};

  const int lr = tid / 4;         // 0..63 : row (of A) or column (of W) staged by this thread
  const int lk = (tid % 4) * 4;   // 0,4,8,12
  long long a_off = -1;
  if (lr < rows_here) {
    int r = row0 + lr;
    if (g.a_rows) r = g.a_rows[r];
    a_off = (long long)r * g.lda;
  }
  const int wn = col0 + lr;
  const bool w_ok = wn < g.N;

  for (int k0 = 0; k0 < g.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int k = k0 + lk + i;
      float av = 0.f, bv = 0.f, b2v = 0.f;
      if (k < g.K) {
        if (a_off >= 0) av = to_f32(A[a_off + k]);
        if (w_ok) {
          bv = to_f32(W[(size_t)wn * g.K + k]);
          if (SWIGLU) b2v = to_f32(W[(size_t)(wn + g.N) * g.K + k]);
        }
      }
      As[lk + i][lr] = av;
      Bs[lk + i][lr] = bv;
      if (SWIGLU) B2s[lk + i][lr] = b2v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      if (SWIGLU) {
#pragma unroll
        for (int j = 0; j < TN; ++j) b[j] = B2s[k][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc2[i][j] = fmaf(a[i], b[j], acc2[i][j]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int lrow = ty * TM + i;
    if (lrow >= rows_here) continue;
    size_t orow = (size_t)(row0 + lrow) * g.ldo;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int n = col0 + tx * TN + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (SWIGLU) v = silu_mul(v, acc2[i][j]);
      if (g.bias) v += ld_dt(g.bias, g.bias_dt, n);
      st_dt(g.out, g.out_dt, orow + n, v);
    }
  }
}

template <typename TA, typename TW>
int launch(const GemmArgs& g, int m_tiles, cudaStream_t s) {
  dim3 grid((g.N + BN - 1) / BN, m_tiles);
  if (grid.x == 0 || grid.y == 0) return NV_OK;
  if (grid.y > 65535) return NV_ERR_BAD_SIZE;
  if (g.swiglu) gemm_plain_kernel<TA, TW, true><<<grid, 256, 0, s>>>(g);
  else gemm_plain_kernel<TA, TW, false><<<grid, 256, 0, s>>>(g);
  NV_RETURN_LAST();
}

}  // namespace

// Rows per M-tile of the grouped form; the tile list given to nv_gemm_plain must be cut by this.
NV_API int nv_gemm_plain_tile_m() { return BM; }

NV_API int nv_gemm_plain(const void* A, int a_dt, long long lda, const int* a_rows,
                         const void* W, int w_dt, long long w_expert_stride,
                         const void* bias, int bias_dt,
                         void* out, int out_dt, long long ldo,
                         int M, int N, int K, int swiglu,
                         const int* tile_expert, const int* tile_row0, const int* tile_rows,
                         const int* num_tiles, int max_tiles, cudaStream_t stream) {
  if (!dt_ok(a_dt) || !dt_ok(w_dt) || !dt_ok(out_dt) || (bias && !dt_ok(bias_dt))) return NV_ERR_BAD_DTYPE;
  if (M < 0 || N <= 0 || K <= 0) return NV_ERR_BAD_SIZE;
  GemmArgs g;
  g.A = A; g.W = W; g.bias = bias; g.out = out; g.a_rows = a_rows;
  g.tile_expert = tile_expert; g.tile_row0 = tile_row0; g.tile_rows = tile_rows; g.num_tiles = num_tiles;
  g.lda = lda; g.ldo = ldo; g.w_expert_stride = w_expert_stride;
  g.M = M; g.N = N; g.K = K; g.bias_dt = bias_dt; g.out_dt = out_dt; g.swiglu = swiglu;
  int m_tiles = tile_expert ? max_tiles : (M + BM - 1) / BM;
  if (a_dt == NV_DT_F32 && w_dt == NV_DT_F32) return launch<float, float>(g, m_tiles, stream);
  if (a_dt == NV_DT_F32 && w_dt == NV_DT_BF16) return launch<float, bf16>(g, m_tiles, stream);
  if (a_dt == NV_DT_BF16 && w_dt == NV_DT_F32) return launch<bf16, float>(g, m_tiles, stream);
  return launch<bf16, bf16>(g, m_tiles, stream);
}
