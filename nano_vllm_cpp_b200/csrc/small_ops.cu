// Small fast kernels around the big products.
#include "common.cuh"

namespace {

// out[t, n] = sum_k a[t, k] * w[n, k] for float32 rows a and a short, wide matrix w (router logits,
// the shared expert's gate): one warp per (row, four outputs).  A lane sums its strided elements in
// ascending order, then the lanes are added by a fixed xor tree, so a row's result does not
// depend on the batch.  Float32 throughout (src/model.cpp:797 computes the router logits in float32 too).
template <typename TW>
__global__ void __launch_bounds__(256) rowdot_kernel(const float* __restrict__ a, long long lda,
                                                     const TW* __restrict__ w, float* __restrict__ out, int T,
                                                     int N, int K) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32;
  const int nq = (N + 3) / 4;
  if (warp >= T * nq) return;
  const int t = warp / nq, n0 = (warp % nq) * 4;
  const float* ar = a + (size_t)t * lda;
  float s[4] = {0.f, 0.f, 0.f, 0.f};
  const TW* wr[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) wr[i] = w + (size_t)min(n0 + i, N - 1) * K;
  if (K % 4 == 0 && ((uintptr_t)ar & 15) == 0 && ((uintptr_t)w & 15) == 0) {
    for (int k = lane * 4; k < K; k += 128) {
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
    for (int k = lane; k < K; k += 32) {
      const float av = ar[k];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(av, to_f32(wr[i][k]), s[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    s[i] = warp_sum(s[i]);
    if (lane == 0 && n0 + i < N) out[(size_t)t * N + n0 + i] = s[i];
  }
}

}  // namespace

NV_API int nv_rowdot(const float* a, long long lda, const void* w, int w_dt, float* out, int T, int N, int K,
                     cudaStream_t s) {
  if (!dt_ok(w_dt)) return NV_ERR_BAD_DTYPE;
  if (T == 0 || N == 0) return NV_OK;
  const long long warps = (long long)T * ((N + 3) / 4);
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (w_dt == NV_DT_F32) rowdot_kernel<float><<<blocks, 256, 0, s>>>(a, lda, (const float*)w, out, T, N, K);
  else rowdot_kernel<bf16><<<blocks, 256, 0, s>>>(a, lda, (const bf16*)w, out, T, N, K);
  NV_RETURN_LAST();
}
