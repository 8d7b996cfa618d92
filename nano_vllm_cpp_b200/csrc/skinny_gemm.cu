// Products of a handful of rows with bfloat16 weights: out[r, n] = sum_k x[r, k] * W[n, k].
//
// With one to eight rows a product is nothing but a stream of W from memory, and what decides its time is how soon
// every multiprocessor has loads in flight and how many.  The tensor-core kernel (tc_gemm.cu) pays for its set-up
// here: a weight tile of 128 rows per CTA leaves a 2,048 x 2,048 matrix with 16 tiles for 148 multiprocessors, so
// it splits K and needs a second kernel to add the parts, and an expert's matrix for one row is 11 tiles that each
// pull 1 MB through one CTA's ring.  This kernel has no tiles: a warp takes four output features at a time
// (consecutive rows of W, 16-byte loads, a lane's eight elements of every row in registers), multiplies them with
// the rows of x (read through L1, where they stay) and adds the lanes up with shuffles; the grid covers the GPU
// with sixteen warps per multiprocessor whatever the matrix is.  Sums are float32.  Forms:
//
//   dense      W [N, K]; rows 0 .. R-1 of x; optional bias; out bfloat16 or float32
//   grouped    W [E, rows, K]; a tile list (expert, first row, rows <= 8) over an expert-sorted row list as built by
//              the routing kernels; a tile's row j is x[a_rows[row0 + j]], or x[(row0 + j - x_sub) % x_mod] for
//              experts that all take the same few rows, or x[row0 + j]
//   swiglu     W holds gate rows [0, N) and up rows [N, 2N) (per expert); out = silu(gate) * up
//
// The reference computes these products row by row on the vector units too (src/hip_ops.hip:43-64, 861-893).
#include "common.cuh"

namespace {

constexpr int SK_WARPS = 16;          // warps per block
constexpr int SK_NF = 4;              // output features a warp works on at once
constexpr int SK_MAX_ROWS = 8;

struct SkArgs {
  const bf16* x;
  const bf16* w;
  const void* bias;
  void* out;
  const int* a_rows;        // grouped: source row of every sorted row (nullptr: see x_mod)
  const int* tile_expert;   // grouped: tile list; nullptr = dense
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tiles;
  int* err;
  long long ldx, ldo, w_expert_stride;   // elements
  int R;                    // dense: rows
  int N, K, swiglu, out_dt, bias_dt, x_sub, x_mod, x_rows_total;
};

__device__ __forceinline__ void fma8(float (&acc), const uint4& wv, const uint4& xv) {
  const __nv_bfloat162* wp = (const __nv_bfloat162*)&wv;
  const __nv_bfloat162* xp = (const __nv_bfloat162*)&xv;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(wp[i]), b = __bfloat1622float2(xp[i]);
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
  }
}

// One warp, one tile (up to RMAX rows), SK_NF features from feature n0 on (swiglu: gate and up rows of SK_NF / 2
// features).  wrow[f] points at the f-th weight row; a row that does not exist points at row 0 and is not stored.
template <int RMAX>
__device__ __forceinline__ void warp_unit(const SkArgs& a, const bf16* const (&wrow)[SK_NF], const bf16* const (&xrow)[RMAX],
                                          int rows, int lane, float (&sum)[SK_NF][RMAX]) {
#pragma unroll
  for (int f = 0; f < SK_NF; ++f)
#pragma unroll
    for (int r = 0; r < RMAX; ++r) sum[f][r] = 0.f;
  const int chunks = a.K / 8;                     // 16-byte pieces of a row
  // two pieces per lane and step: eight weight loads in flight per lane
  for (int c0 = lane; c0 < chunks; c0 += 64) {
    const int c1 = c0 + 32;
    const bool two = c1 < chunks;
    uint4 wv0[SK_NF], wv1[SK_NF];
#pragma unroll
    for (int f = 0; f < SK_NF; ++f) {
      wv0[f] = __ldcs((const uint4*)wrow[f] + c0);          // streamed once: no reason to keep it in L1 or early in L2
      wv1[f] = two ? __ldcs((const uint4*)wrow[f] + c1) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      if (r < rows) {
        const uint4 xv0 = __ldg((const uint4*)xrow[r] + c0);
        const uint4 xv1 = two ? __ldg((const uint4*)xrow[r] + c1) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int f = 0; f < SK_NF; ++f) {
          fma8(sum[f][r], wv0[f], xv0);
          fma8(sum[f][r], wv1[f], xv1);
        }
      }
    }
  }
#pragma unroll
  for (int f = 0; f < SK_NF; ++f)
#pragma unroll
    for (int r = 0; r < RMAX; ++r)
      if (r < rows) sum[f][r] = warp_sum(sum[f][r]);
}

template <int RMAX, bool SWIGLU>
__global__ void __launch_bounds__(SK_WARPS * 32) skinny_kernel(SkArgs a) {
  grid_dep_wait();            // x is the output of the kernel before
  grid_dep_launch();
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int gwarp = blockIdx.x * SK_WARPS + warp, nwarps = gridDim.x * SK_WARPS;
  constexpr int fpu = SWIGLU ? SK_NF / 2 : SK_NF;                 // output features per unit
  const int units_n = (a.N + fpu - 1) / fpu;
  const int tiles = a.tile_expert ? *a.num_tiles : 1;
  const long long total = (long long)tiles * units_n;
  for (long long u = gwarp; u < total; u += nwarps) {
    const int y = (int)(u / units_n), n0 = (int)(u % units_n) * fpu;
    int row0 = 0, rows = a.R;
    const bf16* wbase = a.w;
    if (a.tile_expert) {
      row0 = a.tile_row0[y];
      rows = a.tile_rows[y];
      if (rows > RMAX) {                              // the list was cut for another kernel: flag it, do what fits
        if (a.err && lane == 0) atomicExch(a.err, 1 + row0);
        rows = RMAX;
      }
      if (rows <= 0) continue;
      wbase += (size_t)a.tile_expert[y] * a.w_expert_stride;
    }
    const bf16* xrow[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      int src = row0 + min(r, rows - 1);
      if (a.tile_expert) {
        if (a.a_rows) src = a.a_rows[src];
        else if (a.x_mod) src = (src - a.x_sub) % a.x_mod;
      }
      if (src < 0 || src >= a.x_rows_total) {          // a bad permutation: flag it and read row 0
        if (a.err && lane == 0) atomicExch(a.err, 1 + row0 + r);
        src = 0;
      }
      xrow[r] = a.x + (size_t)src * a.ldx;
    }
    const bf16* wrow[SK_NF];
    bool ok[SK_NF];
#pragma unroll
    for (int f = 0; f < SK_NF; ++f) {
      // swiglu: features n0, n0 + 1 as (gate, gate, up, up); else features n0 .. n0 + 3
      const int n = SWIGLU ? n0 + (f % fpu) : n0 + f;
      ok[f] = n < a.N;
      const int wr = ok[f] ? (SWIGLU && f >= fpu ? a.N + n : n) : 0;
      wrow[f] = wbase + (size_t)wr * a.K;
    }
    float sum[SK_NF][RMAX];
    warp_unit<RMAX>(a, wrow, xrow, rows, lane, sum);
    // lane r stores row r (every lane holds every sum)
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      if (r < rows && lane == r) {
        const size_t o = (size_t)(row0 + r) * a.ldo;
        if (SWIGLU) {
#pragma unroll
          for (int f = 0; f < SK_NF / 2; ++f)
            if (ok[f]) st_dt(a.out, a.out_dt, o + n0 + f, silu_mul(sum[f][r], sum[f + SK_NF / 2][r]));
        } else {
#pragma unroll
          for (int f = 0; f < SK_NF; ++f)
            if (ok[f]) {
              float v = sum[f][r];
              if (a.bias) v += ld_dt(a.bias, a.bias_dt, n0 + f);
              st_dt(a.out, a.out_dt, o + n0 + f, v);
            }
        }
      }
    }
  }
}

int sk_blocks() {
  static int blocks = 0;
  if (!blocks) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    blocks = sms * 2;           // two blocks of sixteen warps per multiprocessor
  }
  return blocks;
}

}  // namespace

NV_API int nv_skinny_gemm_max_rows() { return SK_MAX_ROWS; }

// Whether the kernel takes these sizes: K a multiple of 8 (16-byte loads), rows of x and W 16-byte aligned.
NV_API int nv_skinny_gemm_usable(int rows, int K, long long ldx, const void* x, const void* w) {
  return rows >= 1 && rows <= SK_MAX_ROWS && K > 0 && K % 8 == 0 && ldx % 8 == 0 && !((uintptr_t)x & 15) &&
         !((uintptr_t)w & 15);
}

// Dense (tile_expert == nullptr: rows 0 .. R-1 of x, R <= 8) or grouped (tiles of at most `max_tile_rows` <= 8 rows;
// rows of W per expert = N, or 2N with swiglu; max_tiles bounds the list, whose length is read on the device).
// x has x_rows_total rows.  out row = sorted row (grouped) or row (dense).
NV_API int nv_skinny_gemm(const void* x, long long ldx, int x_rows_total, int R, const void* w, int N, int K,
                          const void* bias, int bias_dt, void* out, int out_dt, long long ldo, int swiglu,
                          const int* a_rows, const int* tile_expert, const int* tile_row0, const int* tile_rows,
                          const int* num_tiles, int max_tiles, int max_tile_rows, int x_sub, int x_mod, int* err,
                          cudaStream_t stream) {
  if (!dt_ok(out_dt) || (bias && !dt_ok(bias_dt))) return NV_ERR_BAD_DTYPE;
  const bool grouped = tile_expert != nullptr;
  const int rmax = grouped ? max_tile_rows : R;
  if (!nv_skinny_gemm_usable(rmax, K, ldx, x, w) || N <= 0 || x_rows_total <= 0) return NV_ERR_UNSUPPORTED;
  if (x_mod < 0 || x_sub < 0 || (bias && (swiglu || grouped))) return NV_ERR_BAD_SIZE;
  if (grouped && max_tiles <= 0) return NV_OK;
  SkArgs a;
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.bias = bias; a.out = out; a.a_rows = a_rows;
  a.tile_expert = tile_expert; a.tile_row0 = tile_row0; a.tile_rows = tile_rows; a.num_tiles = num_tiles; a.err = err;
  a.ldx = ldx; a.ldo = ldo; a.w_expert_stride = (long long)(swiglu ? 2 * N : N) * K;
  a.R = R; a.N = N; a.K = K; a.swiglu = swiglu ? 1 : 0; a.out_dt = out_dt; a.bias_dt = bias_dt;
  a.x_sub = x_sub; a.x_mod = x_mod; a.x_rows_total = x_rows_total;
  const int fpu = swiglu ? SK_NF / 2 : SK_NF;
  const long long units = (long long)(grouped ? max_tiles : 1) * ((N + fpu - 1) / fpu);
  long long blocks = (units + SK_WARPS - 1) / SK_WARPS;
  if (blocks > sk_blocks()) blocks = sk_blocks();
  const dim3 grid((unsigned)blocks), block(SK_WARPS * 32);
  cudaError_t e;
  if (swiglu) {
    if (rmax <= 1) e = launch_dep(skinny_kernel<1, true>, grid, block, 0, stream, a);
    else if (rmax <= 2) e = launch_dep(skinny_kernel<2, true>, grid, block, 0, stream, a);
    else if (rmax <= 4) e = launch_dep(skinny_kernel<4, true>, grid, block, 0, stream, a);
    else e = launch_dep(skinny_kernel<8, true>, grid, block, 0, stream, a);
  } else {
    if (rmax <= 1) e = launch_dep(skinny_kernel<1, false>, grid, block, 0, stream, a);
    else if (rmax <= 2) e = launch_dep(skinny_kernel<2, false>, grid, block, 0, stream, a);
    else if (rmax <= 4) e = launch_dep(skinny_kernel<4, false>, grid, block, 0, stream, a);
    else e = launch_dep(skinny_kernel<8, false>, grid, block, 0, stream, a);
  }
  NV_RETURN_IF(e);
  NV_RETURN_LAST();
}
