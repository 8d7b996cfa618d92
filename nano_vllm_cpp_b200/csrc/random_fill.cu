// Random weights whose values are a function of (key, element index) alone, in integer arithmetic up to one
// exactly rounded multiply and add, so that the host (numpy, weights/random_values.py) and this kernel produce
// the same bits.  The reference has no random-weights mode (TODO.md:108-109 only mentions a synthesised model).
//
//   c  = key + i * 0x9E3779B97F4A7C15                       (64-bit, wrapping)
//   h0 = mix(c), h1 = mix(c ^ 0xD6E8FEB86659FD93), h2 = mix(c ^ 0xA0761D6478BD642F)
//   S  = sum of the twelve 16-bit fields of h0, h1, h2      (0 .. 12 * 65535)
//   z  = float(S - 393210) * 2^-16                          (mean 0, variance 1.0000: twelve uniforms)
//   v  = mean + z * std                                      (multiply, then add, each rounded once)
//
// mix is the finishing function of splitmix64.  The sum of twelve uniform numbers is bell-shaped with tails cut at
// six standard deviations, which is all that weights drawn "N(0, std)" for tests and benchmarks need.
#include "common.cuh"

__host__ __device__ __forceinline__ uint64_t rf_mix(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ int rf_fields(uint64_t h) {
  return (int)(h & 0xFFFF) + (int)((h >> 16) & 0xFFFF) + (int)((h >> 32) & 0xFFFF) + (int)(h >> 48);
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long n, uint64_t key, float mean, float std) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const uint64_t c = key + (uint64_t)i * 0x9E3779B97F4A7C15ull;
    const int S = rf_fields(rf_mix(c)) + rf_fields(rf_mix(c ^ 0xD6E8FEB86659FD93ull)) +
                  rf_fields(rf_mix(c ^ 0xA0761D6478BD642Full));
    const float z = __fmul_rn((float)(S - 393210), 1.0f / 65536.0f);
    out[i] = from_f32<T>(__fadd_rn(mean, __fmul_rn(z, std)));
  }
}

// out[i] = mean + z_i(key) * std for i < n, rounded once to the output type.
NV_API int nv_random_fill(void* out, int dt, long long n, unsigned long long key, float mean, float std,
                          cudaStream_t stream) {
  if (!dt_ok(dt)) return NV_ERR_BAD_DTYPE;
  if (n < 0) return NV_ERR_BAD_SIZE;
  if (n == 0) return NV_OK;
  const int block = 256;
  const long long want = (n + block - 1) / block;
  const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dt == NV_DT_F32) random_fill_kernel<float><<<grid, block, 0, stream>>>((float*)out, n, key, mean, std);
  else random_fill_kernel<bf16><<<grid, block, 0, stream>>>((bf16*)out, n, key, mean, std);
  NV_RETURN_LAST();
}
