// Small fast kernels around the big products.
#include "common.cuh"
#include "moe_route.cuh"

namespace {

// out[t, n] = sum_k a[t, k] * w[n, k] for float32 rows a and a short, wide matrix w (router logits,
// the shared expert's gate): one block per (row, four outputs); its 8 warps take the 128-element
// chunks of k in turn (warp w: chunks w, w + 8, ...), a lane sums its 4 elements of each chunk in
// ascending order, lanes are added by a fixed xor tree and the 8 warp sums in warp order.  The order
// is the same whatever the batch is, so a row's result does not depend on it.  Float32 throughout
// (src/model.cpp:797 computes the router logits in float32 too).
template <typename TW>
__global__ void __launch_bounds__(256) rowdot_kernel(const float* __restrict__ a, long long lda,
                                                     const TW* __restrict__ w, float* __restrict__ out,
                                                     long long ldo, int N, int K) {
  __shared__ float part[8][4];
  grid_dep_wait();
  grid_dep_launch();
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t = blockIdx.x, n0 = blockIdx.y * 4;
  const float* ar = a + (size_t)t * lda;
  float s[4] = {0.f, 0.f, 0.f, 0.f};
  const TW* wr[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) wr[i] = w + (size_t)min(n0 + i, N - 1) * K;
  if (K % 4 == 0 && ((uintptr_t)ar & 15) == 0 && ((uintptr_t)w & 15) == 0) {
    for (int k = warp * 128 + lane * 4; k < K; k += 1024) {
      const float4 av = *(const float4*)(ar + k);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float w0, w1, w2, w3;
        if (sizeof(TW) == 4) {
          const float4 wv = *(const float4*)((const float*)wr[i] + k);
          w0 = wv.x; w1 = wv.y; w2 = wv.z; w3 = wv.w;
        } else {
          const uint2 raw = *(const uint2*)((const bf16*)wr[i] + k);
          const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
          const float2 hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
          w0 = lo.x; w1 = lo.y; w2 = hi.x; w3 = hi.y;
        }
        s[i] = fmaf(av.x, w0, s[i]); s[i] = fmaf(av.y, w1, s[i]);
        s[i] = fmaf(av.z, w2, s[i]); s[i] = fmaf(av.w, w3, s[i]);
      }
    }
  } else {
    for (int k0 = warp * 128; k0 < K; k0 += 1024)
      for (int k = k0 + lane; k < min(K, k0 + 128); k += 32) {
        const float av = ar[k];
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] = fmaf(av, to_f32(wr[i][k]), s[i]);
      }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    s[i] = warp_sum(s[i]);
    if (lane == 0) part[warp][i] = s[i];
  }
  __syncthreads();
  if (threadIdx.x < 4 && n0 + threadIdx.x < N) {
    float v = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) v += part[wi][threadIdx.x];
    out[(size_t)t * ldo + n0 + threadIdx.x] = v;
  }
}

// The same product for many rows: one block keeps WT rows in shared memory and its 8 warps walk the outputs
// four at a time, each warp summing its k for the WT rows at once, so a weight row is read once per
// WT rows.  Fewer, fatter blocks and a fraction of the loads; the order of the sum differs from
// rowdot_kernel's, so a run uses one of the two for a given op and batch shape only where rounding-level
// differences between batch shapes are accepted (bfloat16 runs).
// A warp's walk along k is a chain of trips to L2 for the weights, one per 128 elements, so a long K is cut into
// ranges of ROWDOT_K_RANGE elements (blockIdx.y): every range is a block of its own, writes its sums to part[range],
// and rowdot_finish_kernel adds the ranges in order.  The cut depends on K alone, so a row's value does not depend
// on the batch.  Measured for 2,048 rows: K = 3,584 and 65 outputs, 147 us in one range (84 trips one after the
// other) and 72 us in seven; K = 2,048 and 61 outputs, 31 us in one range and 40 us in four (the second kernel and
// the blocks' set-up cost more than the shorter chain gains): K is cut from ROWDOT_CUT_FROM elements on.
constexpr int ROWDOT_K_RANGE = 512;
constexpr int ROWDOT_CUT_FROM = 3072;
template <typename TW, int WT>
__global__ void __launch_bounds__(256) rowdot_wide_kernel(const float* __restrict__ a, long long lda,
                                                          const TW* __restrict__ w, float* __restrict__ out,
                                                          long long ldo, int T, int N, int K_all,
                                                          float* __restrict__ part) {
  extern __shared__ float row_s[];                 // [WT][K]
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t0 = blockIdx.x * WT;
  const int nt = min(WT, T - t0);
  // this block's range of k; from here on a, w and K are the range's
  const int kb = gridDim.y > 1 ? (int)blockIdx.y * ROWDOT_K_RANGE : 0;
  const int K = gridDim.y > 1 ? min(ROWDOT_K_RANGE, K_all - kb) : K_all;
  a += kb;
  w += kb;
  if (gridDim.y > 1) {
    out = part + (size_t)blockIdx.y * T * N;
    ldo = N;
  }
  if (K_all % 4 == 0 && lda % 4 == 0 && ((uintptr_t)a & 15) == 0) {
    // 16-byte loads, four in flight per thread: one scalar load at a time made this copy the kernel's time
    // (the rows of the tile are walked as one run of WT * K / 4 loads, eight in flight per thread: row by row a
    // thread had only K / 1024 loads under way at a time)
    const int k4 = K / 4, total = WT * k4;
    for (int i0 = threadIdx.x; i0 < total; i0 += 8 * 256) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * 256;
        const int r = i / k4, c = i - r * k4;
        v[u] = (i < total && r < nt) ? ((const float4*)(a + (size_t)(t0 + r) * lda))[c] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * 256;
        if (i < total) ((float4*)row_s)[i] = v[u];
      }
    }
  } else {
    for (int i = threadIdx.x; i < WT * K; i += 256) {
      const int r = i / K, k = i - r * K;
      row_s[i] = r < nt ? a[(size_t)(t0 + r) * lda + k] : 0.f;
    }
  }
  __syncthreads();
  const bool vec = K_all % 4 == 0 && ((uintptr_t)w & 15) == 0;
  for (int n0 = warp * 4; n0 < N; n0 += 32) {
    float s[WT][4];
#pragma unroll
    for (int r = 0; r < WT; ++r) s[r][0] = s[r][1] = s[r][2] = s[r][3] = 0.f;
    const TW* wr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wr[i] = w + (size_t)min(n0 + i, N - 1) * K_all;
    if (vec) {
      // (few rows per block: unrolled, so that a warp has the weight loads of several steps under way; with four or
      // eight rows the accumulators leave no registers for that and the unrolled loop was slower)
#pragma unroll (WT <= 2 ? 8 : 1)
      for (int k = lane * 4; k < K; k += 128) {
        float4 av[WT];
#pragma unroll
        for (int r = 0; r < WT; ++r) av[r] = *(const float4*)(row_s + r * K + k);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float w0, w1, w2, w3;
          if (sizeof(TW) == 4) {
            const float4 wv = *(const float4*)((const float*)wr[i] + k);
            w0 = wv.x; w1 = wv.y; w2 = wv.z; w3 = wv.w;
          } else {
            const uint2 raw = *(const uint2*)((const bf16*)wr[i] + k);
            const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
            const float2 hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
            w0 = lo.x; w1 = lo.y; w2 = hi.x; w3 = hi.y;
          }
#pragma unroll
          for (int r = 0; r < WT; ++r) {
            s[r][i] = fmaf(av[r].x, w0, s[r][i]); s[r][i] = fmaf(av[r].y, w1, s[r][i]);
            s[r][i] = fmaf(av[r].z, w2, s[r][i]); s[r][i] = fmaf(av[r].w, w3, s[r][i]);
          }
        }
      }
    } else {
      for (int k = lane; k < K; k += 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float wv = to_f32(wr[i][k]);
#pragma unroll
          for (int r = 0; r < WT; ++r) s[r][i] = fmaf(row_s[r * K + k], wv, s[r][i]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < WT; ++r)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float v = warp_sum(s[r][i]);
        if (lane == 0 && r < nt && n0 + i < N) out[(size_t)(t0 + r) * ldo + n0 + i] = v;
      }
  }
}

// out[t, n] = part[0][t][n] + part[1][t][n] + ... in that order.
__global__ void rowdot_finish_kernel(const float* __restrict__ part, int ranges, float* __restrict__ out, long long ldo,
                                     int T, int N) {
  grid_dep_wait();
  grid_dep_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T * N) return;
  float v = 0.f;
  for (int r = 0; r < ranges; ++r) v += part[(size_t)r * T * N + i];
  out[(i / N) * ldo + i % N] = v;
}

// Routing of a small batch in one launch: top-k of every row, the expert permutation, and the
// expert-sorted copy of the (bfloat16) activations.  One block of 1024 threads; for batches whose
// T * (K + C) pairs and rows fit one block's reach (the launcher checks).
__global__ void __launch_bounds__(1024) moe_route_small_kernel(
    const float* __restrict__ logits, long long ld, int T, int E, int K, int renorm, int C,
    const float* __restrict__ gate_logit, long long gate_ld, int* __restrict__ idx, float* __restrict__ score,
    int tile_m, int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ sorted_token,
    int* __restrict__ pair_pos, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
    int* __restrict__ tile_rows, int* __restrict__ num_tiles, int* __restrict__ err,
    const bf16* __restrict__ x, bf16* __restrict__ x_sorted, int H, int n_static, int* __restrict__ zero,
    int n_zero) {
  extern __shared__ double rs_smem[];
  grid_dep_wait();
  grid_dep_launch();
  if ((int)threadIdx.x < n_zero) zero[threadIdx.x] = 0;      // (tile counters of the products that follow)
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int KT = K + C;
  for (int t = warp; t < T; t += 32)
    route_row(logits + (size_t)t * ld, E, K, renorm, rs_smem + (size_t)warp * E, lane, idx + (size_t)t * KT,
              score + (size_t)t * KT, C, C ? gate_logit + (size_t)t * gate_ld : nullptr);
  __threadfence_block();
  __syncthreads();
  int* al_s = (int*)(rs_smem + (size_t)32 * E);
  align_block(idx, T * KT, KT, E + C, tile_m, counts, offsets, sorted_token, pair_pos, tile_expert, tile_row0,
              tile_rows, num_tiles, err, al_s, 0, nullptr, nullptr, nullptr, nullptr, n_static);
  if (!x_sorted) return;
  __threadfence_block();
  __syncthreads();
  // flat copy of T*KT rows of H/8 16-byte chunks; four loads in flight per thread before the stores
  const int cpr = H / 8, total = T * KT * cpr;
  for (int base = threadIdx.x; base < total; base += 4 * 1024) {
    uint4 v[4];
    int idx4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      idx4[u] = base + u * 1024;
      if (idx4[u] < total) {
        const int p = idx4[u] / cpr, c = idx4[u] - p * cpr;
        v[u] = *((const uint4*)(x + (size_t)sorted_token[p] * H) + c);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (idx4[u] < total) *((uint4*)x_sorted + idx4[u]) = v[u];
  }
}

}  // namespace

// Floats of scratch that the many-rows kernel needs for its ranges of k (0: it does not cut K).
NV_API long long nv_rowdot_scratch_floats(int T, int N, int K, int wide) {
  if (!wide || K < ROWDOT_CUT_FROM) return 0;
  return (long long)((K + ROWDOT_K_RANGE - 1) / ROWDOT_K_RANGE) * T * N;
}

NV_API int nv_rowdot(const float* a, long long lda, const void* w, int w_dt, float* out, long long ldo, int T,
                     int N, int K, int wide, float* scratch, cudaStream_t s) {
  if (!dt_ok(w_dt)) return NV_ERR_BAD_DTYPE;
  if (T == 0 || N == 0) return NV_OK;
  // many rows: WT of them per block in shared memory.  Every block reads the matrix's columns of its range of k (from
  // L2), so fat blocks save traffic, but there must be blocks enough to hide a warp's chain of loads: WT = T / 256
  // (1, 2, 4 or 8), i.e. 256 blocks or more per range.  (Measured at 256 rows, 61 outputs, K = 2,048: 60 us with
  // 64 blocks of four rows.)  A row's sum does not depend on WT.
  if (wide) {
    const int ranges = scratch && K >= ROWDOT_CUT_FROM ? (K + ROWDOT_K_RANGE - 1) / ROWDOT_K_RANGE : 1;
    if (ranges > 1 && nv_rowdot_scratch_floats(T, N, K, 1) == 0) return NV_ERR_BAD_SIZE;
    const int k_block = ranges > 1 ? ROWDOT_K_RANGE : K;
    int wt = 8;
    while (wt > 1 && (T < 256 * wt || (size_t)wt * k_block * 4 > 96 * 1024)) wt >>= 1;
    const size_t smem = (size_t)wt * k_block * 4;
    if (smem <= 96 * 1024 && ranges <= 65535) {
      static bool attr_done = false;
      if (!attr_done) {
        const void* fns[8] = {(const void*)rowdot_wide_kernel<float, 1>, (const void*)rowdot_wide_kernel<bf16, 1>,
                              (const void*)rowdot_wide_kernel<float, 2>, (const void*)rowdot_wide_kernel<bf16, 2>,
                              (const void*)rowdot_wide_kernel<float, 4>, (const void*)rowdot_wide_kernel<bf16, 4>,
                              (const void*)rowdot_wide_kernel<float, 8>, (const void*)rowdot_wide_kernel<bf16, 8>};
        for (const void* f : fns) {
          const cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
          if (e != cudaSuccess) return (int)e;
        }
        attr_done = true;
      }
      const dim3 blocks((unsigned)((T + wt - 1) / wt), (unsigned)ranges);
      const bool f32 = w_dt == NV_DT_F32;
#define NV_ROWDOT_WIDE(WT)                                                                                           \
  if (f32)                                                                                                           \
    rowdot_wide_kernel<float, WT><<<blocks, 256, smem, s>>>(a, lda, (const float*)w, out, ldo, T, N, K, scratch);   \
  else                                                                                                               \
    rowdot_wide_kernel<bf16, WT><<<blocks, 256, smem, s>>>(a, lda, (const bf16*)w, out, ldo, T, N, K, scratch)
      if (wt == 8) { NV_ROWDOT_WIDE(8); }
      else if (wt == 4) { NV_ROWDOT_WIDE(4); }
      else if (wt == 2) { NV_ROWDOT_WIDE(2); }
      else { NV_ROWDOT_WIDE(1); }
#undef NV_ROWDOT_WIDE
      NV_RETURN_IF(cudaGetLastError());
      if (ranges > 1) {
        const long long outputs = (long long)T * N;
        NV_RETURN_IF(launch_dep(rowdot_finish_kernel, dim3((unsigned)((outputs + 255) / 256)), dim3(256), 0, s,
                                (const float*)scratch, ranges, out, ldo, T, N));
      }
      NV_RETURN_LAST();
    }
  }
  if ((N + 3) / 4 > 65535) return NV_ERR_BAD_SIZE;
  dim3 grid(T, (N + 3) / 4);
  if (w_dt == NV_DT_F32) NV_RETURN_IF(launch_dep(rowdot_kernel<float>, grid, dim3(256), 0, s, a, lda, (const float*)w, out, ldo, N, K));
  else NV_RETURN_IF(launch_dep(rowdot_kernel<bf16>, grid, dim3(256), 0, s, a, lda, (const bf16*)w, out, ldo, N, K));
  NV_RETURN_LAST();
}

// Largest batch the fused routing kernel takes: rows and pairs one block can walk in a few microseconds.
NV_API int nv_moe_route_small_usable(int T, int E, int K, int C, int H) {
  const size_t smem = (size_t)32 * E * sizeof(double) + (size_t)4 * (E + C) * sizeof(int);
  return T <= 64 && T * (K + C) <= 1024 && smem <= 48 * 1024 && H % 8 == 0 && K <= 32 && C <= 32;
}

NV_API int nv_moe_route_small(const float* logits, long long ld, int T, int E, int K, int renorm, int C,
                              const float* gate_logit, long long gate_ld, int* idx, float* score, int tile_m,
                              int* counts, int* offsets, int* sorted_token, int* pair_pos, int* tile_expert,
                              int* tile_row0, int* tile_rows, int* num_tiles, int* err, const void* x,
                              void* x_sorted, int H, int n_static, int* zero, int n_zero, cudaStream_t s) {
  if (!nv_moe_route_small_usable(T, E, K, C, H) || K < 1 || K > E || (C > 0 && !gate_logit)) return NV_ERR_UNSUPPORTED;
  if (n_zero < 0 || n_zero > 1024 || (n_zero && !zero)) return NV_ERR_BAD_SIZE;
  if (n_static != 0 && n_static != C) return NV_ERR_UNSUPPORTED;
  if (T == 0) return NV_OK;
  const size_t smem = (size_t)32 * E * sizeof(double) + (size_t)4 * (E + C) * sizeof(int);
  NV_RETURN_IF(launch_dep(moe_route_small_kernel, dim3(1), dim3(1024), smem, s, logits, ld, T, E, K, renorm, C,
                          gate_logit, gate_ld, idx, score, tile_m, counts, offsets, sorted_token, pair_pos, tile_expert,
                          tile_row0, tile_rows, num_tiles, err, (const bf16*)x, (bf16*)x_sorted, H, n_static, zero,
                          n_zero));
  NV_RETURN_LAST();
}
