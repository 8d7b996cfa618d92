// Dense products of a handful of rows with bfloat16 weights: out[r, n] = sum_k x[r, k] * W[n, k], r < 8 (r < 32
// without SwiGLU).
//
// With one to eight rows a product is nothing but a stream of W from memory, and what decides its time is how soon
// the whole matrix is on its way.  The tcgen05 kernel (tc_gemm.cu) pays for its set-up here: a weight tile of 128
// rows per CTA leaves a 2,048 x 2,048 matrix with 16 tiles for 148 multiprocessors, so it splits K and needs a
// second kernel to add the parts.  This kernel has no ring and no set-up: a block of sixteen warps takes sixteen
// output features at a time (sixteen rows of W; with swiglu sixteen gate rows and their sixteen up rows), its warps
// share out K in steps of 32 elements, and every lane asks for its pieces of W, 16 bytes each, a round ahead of the
// one it works on, the first of them before it waits for the kernel before it, whose output (x) it reads last.
// The sums run on the tensor cores all the same: one mma.sync.m16n8k16 takes sixteen weight rows as A and up to
// eight rows of x as B.  A lane's 16 bytes are eight consecutive k of one weight row; they are used as the lane's
// slots of two instructions' A fragments, and the lane's 16 bytes of the x row at the same k as its B slots, so each
// instruction sums 16 values of k that are not the 16 the fragment layout names, but the same 16 in A and in B, and
// all of them exactly once.  Warps' partial sums are added in warp order in shared memory.  A row's result depends
// on no other row.  More than eight rows (up to 32, without SwiGLU) are NT groups of eight: the same weight
// fragments go through NT instructions, each with its own eight rows of x, which come from the first-level cache (x is
// a few hundred KB at most) while the weights come from memory.
// Options: bias; swiglu (W holds gate rows [0, N) and up rows [N, 2N); out = silu(gate) * up).
//
// It is for small streams: one block per multiprocessor with a round of loads ahead tops out near 4.5 TB/s, so
// matrices beyond about a hundred MB stay with the tcgen05 kernel, whose ring is deeper; and inside a decode step
// it pays for the dense projections only (measured: the experts' grouped products were no faster on it than on
// the tcgen05 kernel, which fetches its first weights while the kernel before it still runs).
//
// The reference computes these products row by row on the vector units (src/hip_ops.hip:43-64).
#include "common.cuh"

namespace {

constexpr int SK_WARPS = 16;          // warps per block: the block's share of K is cut into this many
constexpr int SK_MAX_ROWS = 32;        // without SwiGLU; 8 with it.  (64 rows as eight groups were slower inside a step
                                       // than the tcgen05 kernel: batch 64 6,209 -> 6,030 tokens/s; 16 and 32 rows gain 1.5 %)
constexpr int SK_LOADS = 8;           // 16-byte weight loads of a lane per round; two rounds are in flight

struct SkArgs {
  const bf16* x;
  const bf16* w;
  const void* bias;
  void* out;
  long long ldx, ldo;       // elements
  int R, N, K, groups_n, out_dt, bias_dt;
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool SWIGLU, int NT>
__global__ void __launch_bounds__(SK_WARPS * 32, 1) skinny_kernel(SkArgs a) {
  constexpr int NA = SWIGLU ? 2 : 1;                  // accumulators: gate and up
  constexpr int SK_BATCH = SK_LOADS / (2 * NA);       // steps of 32 elements of K per round of loads
  extern __shared__ __align__(16) float part_s[];     // [2][SK_WARPS][NA][NT][32][4]
  typedef float (*PartPtr)[NA][NT][32][4];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int g = lane / 4, c = lane % 4;               // fragment row / column group of this lane
  const int total = a.groups_n;                       // groups of sixteen features
  const int steps = a.K / 32;                         // this warp takes steps warp, warp + 16, ...
  const int my_steps = steps > warp ? (steps - warp + SK_WARPS - 1) / SK_WARPS : 0;
  const int rounds = max(1, ((steps + SK_WARPS - 1) / SK_WARPS + SK_BATCH - 1) / SK_BATCH);   // the same for every warp

  // asks for this lane's pieces of W of round r of the group of features from n0 on: its two weight rows (features
  // n0 + g and n0 + g + 8, clamped to rows that exist), steps warp + 16 * (r * SK_BATCH + b)
  auto issue = [&](int n0, int r, uint4 (&wl)[SK_BATCH][NA], uint4 (&wh)[SK_BATCH][NA]) {
    const int f_lo = min(n0 + g, a.N - 1), f_hi = min(n0 + g + 8, a.N - 1);
#pragma unroll
    for (int b = 0; b < SK_BATCH; ++b) {
      const int i = r * SK_BATCH + b;
      if (i < my_steps) {
        const int st = warp + i * SK_WARPS;
#pragma unroll
        for (int s = 0; s < NA; ++s) {
          wl[b][s] = __ldcs((const uint4*)(a.w + ((size_t)s * a.N + f_lo) * a.K) + c + st * 4);   // streamed once
          wh[b][s] = __ldcs((const uint4*)(a.w + ((size_t)s * a.N + f_hi) * a.K) + c + st * 4);
        }
      }
    }
  };
  float acc[NA][NT][4];
  auto clear = [&]() {
#pragma unroll
    for (int s = 0; s < NA; ++s)
#pragma unroll
      for (int t = 0; t < NT; ++t) acc[s][t][0] = acc[s][t][1] = acc[s][t][2] = acc[s][t][3] = 0.f;
  };
  // this lane's rows of x (column g of the B operand of each group of eight rows); lanes beyond the rows multiply zeros
  const uint4* xp = (const uint4*)(a.x + (size_t)(g < a.R ? g : 0) * a.ldx) + c;
  const size_t x_tile = (size_t)8 * a.ldx / 8;        // uint4s from one group of eight rows to the next
  int done = 0;                                       // groups this block has finished: which half of `part` is next
  auto compute = [&](int n0, int r, const uint4 (&wl)[SK_BATCH][NA], const uint4 (&wh)[SK_BATCH][NA]) {
    if (NT == 1) {
      uint4 xv[SK_BATCH];
#pragma unroll
      for (int b = 0; b < SK_BATCH; ++b) {
        const int i = r * SK_BATCH + b;
        xv[b] = (i < my_steps && g < a.R) ? __ldg(xp + (warp + i * SK_WARPS) * 4) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int b = 0; b < SK_BATCH; ++b) {
        if (r * SK_BATCH + b < my_steps) {
#pragma unroll
          for (int s = 0; s < NA; ++s) {
            mma_bf16_16816(acc[s][0], wl[b][s].x, wh[b][s].x, wl[b][s].y, wh[b][s].y, xv[b].x, xv[b].y);
            mma_bf16_16816(acc[s][0], wl[b][s].z, wh[b][s].z, wl[b][s].w, wh[b][s].w, xv[b].z, xv[b].w);
          }
        }
      }
    } else {
#pragma unroll
      for (int b = 0; b < SK_BATCH; ++b) {
        const int i = r * SK_BATCH + b;
        if (i < my_steps) {
          constexpr int XT = NT < 4 ? NT : 4;         // row groups whose x is in registers at a time
#pragma unroll
          for (int t0 = 0; t0 < NT; t0 += XT) {
            uint4 xv[XT];
#pragma unroll
            for (int t = 0; t < XT; ++t)
              xv[t] = ((t0 + t) * 8 + g < a.R) ? __ldg(xp + (t0 + t) * x_tile + (warp + i * SK_WARPS) * 4)
                                               : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int t = 0; t < XT; ++t)
#pragma unroll
              for (int s = 0; s < NA; ++s) {
                mma_bf16_16816(acc[s][t0 + t], wl[b][s].x, wh[b][s].x, wl[b][s].y, wh[b][s].y, xv[t].x, xv[t].y);
                mma_bf16_16816(acc[s][t0 + t], wl[b][s].z, wh[b][s].z, wl[b][s].w, wh[b][s].w, xv[t].z, xv[t].w);
              }
          }
        }
      }
    }
    if (r + 1 < rounds) return;
    // the group is complete: the warps' sums are added in warp order.  The halves of `part` take turns, so one
    // barrier per group is enough: a half is written again only after the barrier of the group in between.
    PartPtr p = (PartPtr)(part_s + (size_t)(done & 1) * SK_WARPS * NA * NT * 32 * 4);
    ++done;
#pragma unroll
    for (int s = 0; s < NA; ++s)
#pragma unroll
      for (int t = 0; t < NT; ++t)
        *(float4*)p[warp][s][t][lane] = make_float4(acc[s][t][0], acc[s][t][1], acc[s][t][2], acc[s][t][3]);
    clear();
    __syncthreads();
    // accumulator element j of lane l of row group t: feature (l / 4) + 8 * (j / 2), row 8 * t + 2 * (l % 4) + (j % 2)
    for (int o = threadIdx.x; o < 128 * NT; o += SK_WARPS * 32) {
      const int t = o / 128, l = (o % 128) / 4, j = o % 4;
      float v[NA];
#pragma unroll
      for (int s = 0; s < NA; ++s) {
        v[s] = 0.f;
#pragma unroll
        for (int wi = 0; wi < SK_WARPS; ++wi) v[s] += p[wi][s][t][l][j];
      }
      const int feat = n0 + l / 4 + 8 * (j / 2), row = 8 * t + 2 * (l % 4) + (j % 2);
      if (feat < a.N && row < a.R) {
        float out = SWIGLU ? silu_mul(v[0], v[NA - 1]) : v[0];
        if (!SWIGLU && a.bias) out += ld_dt(a.bias, a.bias_dt, feat);
        st_dt(a.out, a.out_dt, (size_t)row * a.ldo + feat, out);
      }
    }
  };

  // The block's work is the rounds of its groups (blockIdx.x, + gridDim.x, ...), one after the other; the loads of
  // the round after are asked for before a round is worked on (two sets of registers taking turns), so a lane
  // always has loads in flight, also across the sum of a group.
  uint4 wl0[SK_BATCH][NA], wh0[SK_BATCH][NA], wl1[SK_BATCH][NA], wh1[SK_BATCH][NA];
  int q0 = blockIdx.x, q1, r0 = 0, r1;
  clear();
  auto advance = [&](int q, int r, int& qn, int& rn) {
    if (r + 1 < rounds) { qn = q; rn = r + 1; }
    else { qn = q + gridDim.x; rn = 0; }
  };
  if (q0 < total) issue(q0 * 16, r0, wl0, wh0);
  grid_dep_wait();                                    // the first weights are on their way: now wait for x
  grid_dep_launch();
  while (q0 < total) {
    advance(q0, r0, q1, r1);
    if (q1 < total) issue(q1 * 16, r1, wl1, wh1);
    compute(q0 * 16, r0, wl0, wh0);
    if (q1 >= total) break;
    advance(q1, r1, q0, r0);
    if (q0 < total) issue(q0 * 16, r0, wl0, wh0);
    compute(q1 * 16, r1, wl1, wh1);
  }
}

template <bool SWIGLU, int NT>
cudaError_t launch_skinny(const SkArgs& a, int blocks, cudaStream_t stream) {
  constexpr size_t smem = (size_t)2 * SK_WARPS * (SWIGLU ? 2 : 1) * NT * 32 * 4 * sizeof(float);
  static bool attr_done = false;
  if (!attr_done && smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(skinny_kernel<SWIGLU, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  return launch_dep(skinny_kernel<SWIGLU, NT>, dim3(blocks), dim3(SK_WARPS * 32), smem, stream, a);
}

}  // namespace

NV_API int nv_skinny_gemm_max_rows(int swiglu) { return swiglu ? 8 : SK_MAX_ROWS; }

// Whether the kernel takes these sizes: K a multiple of 32 (a warp's step), rows of x and W 16-byte aligned.
NV_API int nv_skinny_gemm_usable(int rows, int K, long long ldx, const void* x, const void* w) {
  return rows >= 1 && rows <= SK_MAX_ROWS && K > 0 && K % 32 == 0 && ldx % 8 == 0 && !((uintptr_t)x & 15) &&
         !((uintptr_t)w & 15);
}

// out[r, :] for rows r < R of x (R <= 32, or 8 with swiglu); W is [N, K], or [2N, K] with swiglu.
NV_API int nv_skinny_gemm(const void* x, long long ldx, int R, const void* w, int N, int K, const void* bias, int bias_dt,
                          void* out, int out_dt, long long ldo, int swiglu, cudaStream_t stream) {
  if (!dt_ok(out_dt) || (bias && !dt_ok(bias_dt))) return NV_ERR_BAD_DTYPE;
  if (!nv_skinny_gemm_usable(R, K, ldx, x, w) || N <= 0 || R > nv_skinny_gemm_max_rows(swiglu)) return NV_ERR_UNSUPPORTED;
  if (bias && swiglu) return NV_ERR_BAD_SIZE;
  SkArgs a;
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.bias = bias; a.out = out;
  a.ldx = ldx; a.ldo = ldo; a.R = R; a.N = N; a.K = K; a.out_dt = out_dt; a.bias_dt = bias_dt;
  a.groups_n = (N + 15) / 16;
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  const int blocks = a.groups_n < num_sms ? a.groups_n : num_sms;   // one block per multiprocessor walks the groups
  cudaError_t e;
  if (swiglu) e = launch_skinny<true, 1>(a, blocks, stream);
  else if (R <= 8) e = launch_skinny<false, 1>(a, blocks, stream);
  else if (R <= 16) e = launch_skinny<false, 2>(a, blocks, stream);
  else e = launch_skinny<false, 4>(a, blocks, stream);
  NV_RETURN_IF(e);
  NV_RETURN_LAST();
}
