// Prefill attention: portions of prompts (any number of rows per request, any mix of requests) against
// the paged keys and values, bfloat16, on the tensor cores.
//
// grid = (row tiles, query heads).  A CTA takes 128 consecutive rows of one request (its portion is cut
// into tiles of 128; the CTA finds its tile by walking the entries' row offsets) and one query head;
// each of its 8 warps owns 16 rows.  Keys and values are gathered page by page into shared memory in
// tiles of 64 keys with cp.async (double-buffered), S = Q K^T and O += P V run as m16n8k16 bf16
// MMAs with float32 accumulators, and the softmax is the online form in float32 registers.
// Row at position p sees keys [max(0, p + 1 - window), p]; the mask is applied per element, so
// a tile may mix rows with different ranges.  The rows of this step are already in the cache when
// the kernel runs, so a portion sees its own earlier rows there.
//
// Reference twin: nv_paged_attention_plain.  (The reference's kernel: src/hip_ops.hip:473-551.)
#include "common.cuh"

#include <stdlib.h>

namespace {

constexpr int BN = 64;   // keys per shared-memory tile; a CTA is BM / 16 warps of 16 rows that share it (BM: 64 or 128)

struct PfArgs {
  const bf16* qkv;
  const bf16* kc;
  const bf16* vc;
  const int* block_table;
  const int* cu_rows;       // [S + 1]
  const int* entry_pos0;    // [S]
  bf16* out;
  float scale_log2;         // scale * log2(e)
  int S, q_stride, max_blocks, window, Hq, Hkv, D, page;
  int min_rows;             // entries with fewer rows are left to another kernel
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// DP: head dimension rounded up to 32, 64, 128 or 256 (sizes the shared memory and the accumulators).
template <int DP, int BM>
__global__ void __launch_bounds__(BM * 2, DP <= 128 ? 2 : 1) attention_prefill_kernel(PfArgs a) {
  constexpr int PF_THREADS = BM * 2;
  constexpr int LDS = DP + 8;                      // row stride (elements): 16 bytes of padding against bank conflicts
  extern __shared__ __align__(16) uint8_t pf_smem[];
  bf16* Qs = (bf16*)pf_smem;
  bf16* Ks = Qs + BM * LDS;                        // [2][BN][LDS]
  bf16* Vs = Ks + 2 * BN * LDS;                    // [2][BN][LDS]
  __shared__ int tile_info[3];                     // entry, first row (batch), rows

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int h = blockIdx.y, kvh = h / (a.Hq / a.Hkv);
  const int D = a.D, chunks = D / 8;

  if (tid == 0) {                                  // which (entry, tile of BM rows) is this CTA's?
    // later tiles of a portion see more keys: hand them out first so that the long ones start early
    int left = (int)(gridDim.x - 1 - blockIdx.x), e = 0, found = -1;
    for (; e < a.S; ++e) {
      int n = a.cu_rows[e + 1] - a.cu_rows[e];
      int tiles = n >= a.min_rows ? (n + BM - 1) / BM : 0;
      if (left < tiles) { found = e; break; }
      left -= tiles;
    }
    tile_info[0] = found;
    if (found >= 0) {
      tile_info[1] = a.cu_rows[found] + left * BM;
      tile_info[2] = min(BM, a.cu_rows[found + 1] - tile_info[1]);
    }
  }
  __syncthreads();
  const int e = tile_info[0];
  if (e < 0) return;
  const int row0 = tile_info[1], nrows = tile_info[2];
  const int pos0 = a.entry_pos0[e] + (row0 - a.cu_rows[e]);      // position of the tile's first row
  const int hi = pos0 + nrows;                                   // keys [.., hi) exist for this tile
  const int lo = a.window > 0 ? max(0, pos0 + 1 - a.window) : 0; // first key any row of the tile sees
  const int kv0 = lo / 16 * 16;
  const int n_tiles = (hi - kv0 + BN - 1) / BN;
  const int* bt = a.block_table + (size_t)e * a.max_blocks;
  const bool pow2_page = (a.page & (a.page - 1)) == 0;
  const int page_shift = 31 - __clz(a.page);

  // ---- Q tile -> shared memory (rows beyond nrows are zero)
  for (int c = tid; c < BM * chunks; c += PF_THREADS) {
    const int r = c / chunks, ch = c % chunks;
    bf16* dst = Qs + r * LDS + ch * 8;
    if (r < nrows) cp_async16(dst, a.qkv + (size_t)(row0 + r) * a.q_stride + (size_t)h * D + ch * 8);
    else *(uint4*)dst = make_uint4(0, 0, 0, 0);
  }
  auto load_kv = [&](int tile, int buf) {
    const int j0 = kv0 + tile * BN;
    bf16* kd = Ks + buf * BN * LDS;
    bf16* vd = Vs + buf * BN * LDS;
    for (int c = tid; c < BN * chunks; c += PF_THREADS) {
      const int r = c / chunks, ch = c - r * chunks;
      const int j = j0 + r;
      int blk = -1, slot = 0;
      if (j < hi) {
        const int pg = pow2_page ? (j >> page_shift) : j / a.page;
        slot = j - pg * a.page;
        blk = bt[pg];
      }
      if (blk >= 0) {
        const size_t off = (((size_t)blk * a.Hkv + kvh) * a.page + slot) * D + ch * 8;
        cp_async16(kd + r * LDS + ch * 8, a.kc + off);
        cp_async16(vd + r * LDS + ch * 8, a.vc + off);
      } else {
        *(uint4*)(kd + r * LDS + ch * 8) = make_uint4(0, 0, 0, 0);
        *(uint4*)(vd + r * LDS + ch * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_kv(0, 0);
  cp_commit();

  const int g = lane / 4, tq = lane % 4;
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;               // this thread's two rows in the tile
  const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;
  const int w_lo_lo = a.window > 0 ? p_lo + 1 - a.window : 0, w_lo_hi = a.window > 0 ? p_hi + 1 - a.window : 0;
  const bool live_lo = r_lo < nrows, live_hi = r_hi < nrows;

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) load_kv(t + 1, buf ^ 1);
    cp_commit();
    cp_wait<1>();                                   // tile t (and Q) have landed
    __syncthreads();
    const bf16* kb = Ks + buf * BN * LDS;
    const bf16* vb = Vs + buf * BN * LDS;
    const int j0 = kv0 + t * BN;

    // a warp whose 16 rows see none of this tile's keys (all later than its last row, or all before its
    // first row's window) only keeps the barriers
    const int warp_p_hi = pos0 + warp * 16 + 15, warp_p_lo = pos0 + warp * 16;
    const bool warp_sees = j0 <= warp_p_hi && (a.window <= 0 || j0 + BN - 1 >= warp_p_lo + 1 - a.window) &&
                           warp * 16 < nrows;
    if (warp_sees) {
    // ---- S = Q K^T for this warp's 16 rows x 64 keys
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      if (kk * 16 < D) {
        uint32_t qa[4];
        ldsm4(s_u32(Qs + (warp * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * LDS + kk * 16 + 8 * (lane / 16)), qa[0],
              qa[1], qa[2], qa[3]);
        // the four fragment loads of a k-block go out together, then their eight products
        uint32_t kf[BN / 16][4];
#pragma unroll
        for (int np = 0; np < BN / 16; ++np)
          ldsm4(s_u32(kb + (np * 16 + (lane % 8) + 8 * (lane / 16)) * LDS + kk * 16 + 8 * ((lane / 8) % 2)), kf[np][0],
                kf[np][1], kf[np][2], kf[np][3]);
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          mma16816(s[2 * np], qa, kf[np][0], kf[np][1]);
          mma16816(s[2 * np + 1], qa, kf[np][2], kf[np][3]);
        }
      }
    }
    // ---- mask (only on tiles that some row of the warp sees partly), online softmax
    const bool whole = j0 + BN - 1 <= warp_p_lo && (a.window <= 0 || j0 >= warp_p_hi + 1 - a.window) &&
                       warp * 16 + 15 < nrows;
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
    if (!whole) {
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = j0 + nt * 8 + 2 * tq + c;
          if (!(live_lo && j <= p_lo && j >= w_lo_lo)) s[nt][c] = -INFINITY;
          if (!(live_hi && j <= p_hi && j >= w_lo_hi)) s[nt][2 + c] = -INFINITY;
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo * a.scale_log2;
    const float ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi * a.scale_log2;
    const float al_lo = exp2f(m_lo * a.scale_log2 - ms_lo), al_hi = exp2f(m_hi * a.scale_log2 - ms_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      s[nt][0] = exp2f(s[nt][0] * a.scale_log2 - ms_lo);
      s[nt][1] = exp2f(s[nt][1] * a.scale_log2 - ms_lo);
      s[nt][2] = exp2f(s[nt][2] * a.scale_log2 - ms_hi);
      s[nt][3] = exp2f(s[nt][3] * a.scale_log2 - ms_hi);
      sum_lo += s[nt][0] + s[nt][1];
      sum_hi += s[nt][2] + s[nt][3];
    }
    l_lo = l_lo * al_lo + sum_lo;                   // per-thread partial sums; lanes are added at the end
    l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi;
    }
    // ---- O += P V
#pragma unroll
    for (int kb16 = 0; kb16 < BN / 16; ++kb16) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kb16][0], s[2 * kb16][1]);
      pa[1] = pack_bf16(s[2 * kb16][2], s[2 * kb16][3]);
      pa[2] = pack_bf16(s[2 * kb16 + 1][0], s[2 * kb16 + 1][1]);
      pa[3] = pack_bf16(s[2 * kb16 + 1][2], s[2 * kb16 + 1][3]);
#pragma unroll
      for (int d4 = 0; d4 < DP / 64; ++d4) {
        if (d4 * 64 < D) {
          uint32_t vf[4][4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int dp = d4 * 4 + u;
            if (dp * 16 < D)
              ldsm4_t(s_u32(vb + (kb16 * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * LDS + dp * 16 + 8 * (lane / 16)),
                      vf[u][0], vf[u][1], vf[u][2], vf[u][3]);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int dp = d4 * 4 + u;
            if (dp * 16 < D) {
              mma16816(o[2 * dp], pa, vf[u][0], vf[u][1]);
              mma16816(o[2 * dp + 1], pa, vf[u][2], vf[u][3]);
            }
          }
        }
      }
      if (DP < 64) {                                 // head sizes below 64: at most two 16-wide blocks
#pragma unroll
        for (int dp = 0; dp < DP / 16; ++dp) {
          if (dp * 16 < D) {
            uint32_t b0, b1, b2, b3;
            ldsm4_t(s_u32(vb + (kb16 * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * LDS + dp * 16 + 8 * (lane / 16)), b0, b1,
                    b2, b3);
            mma16816(o[2 * dp], pa, b0, b1);
            mma16816(o[2 * dp + 1], pa, b2, b3);
          }
        }
      }
    }
    }
    __syncthreads();                                // everyone is done with this buffer before it is refilled
  }
  cp_wait<0>();

  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) {
    const int d = i * 8 + 2 * tq;
    if (d < D) {
      if (live_lo)
        *(uint32_t*)(a.out + ((size_t)(row0 + r_lo) * a.Hq + h) * D + d) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
      if (live_hi)
        *(uint32_t*)(a.out + ((size_t)(row0 + r_hi) * a.Hq + h) * D + d) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
  }
}

template <int DP, int BM>
int launch_prefill_bm(const PfArgs& a, int max_tiles, cudaStream_t s) {
  const size_t smem = (size_t)(BM + 4 * BN) * (DP + 8) * sizeof(bf16);
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DP, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  dim3 grid(max_tiles, a.Hq);
  attention_prefill_kernel<DP, BM><<<grid, BM * 2, smem, s>>>(a);
  NV_RETURN_LAST();
}

// Tiles of 128 rows read every key once per 128 rows; tiles of 64 rows make twice as many, shorter blocks, which
// evens out a causal prompt (its last tile sees all keys, its first almost none) but leaves a multiprocessor
// with half the warps: measured slower (a 2,048-token prompt: 21.7 against 20.5 ms), so 128 it is.
template <int DP>
int launch_prefill(const PfArgs& a, int max_tiles64, int num_sms, cudaStream_t s) {
  (void)num_sms;
  return launch_prefill_bm<DP, 128>(a, max_tiles64, s);
}

}  // namespace

// bfloat16 only; head_dim a multiple of 16 up to 256.  `max_tiles` >= sum over entries of
// ceil(rows / nv_attention_prefill_tile_rows()), the smallest tile the launcher may choose; surplus CTAs leave at once.
// Entries with fewer than `min_rows` rows are skipped (their rows of `out` stay untouched): in a mixed step the
// single rows go to the decode kernel.
NV_API int nv_attention_prefill_tile_rows() { return 64; }

NV_API int nv_attention_prefill(const void* qkv, int q_stride, const void* kc, const void* vc,
                                const int* block_table, int max_blocks, const int* cu_rows, const int* entry_pos0,
                                int S, int max_tiles, float scale, int window, void* out, int Hq, int Hkv, int D,
                                int page, int min_rows, cudaStream_t stream) {
  if (D <= 0 || D > 256 || D % 16 || Hkv <= 0 || Hq % Hkv) return NV_ERR_UNSUPPORTED;
  if (q_stride % 8 || ((uintptr_t)qkv & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15)) return NV_ERR_UNSUPPORTED;
  if (S == 0 || max_tiles == 0) return NV_OK;
  PfArgs a;
  a.qkv = (const bf16*)qkv; a.kc = (const bf16*)kc; a.vc = (const bf16*)vc; a.block_table = block_table;
  a.cu_rows = cu_rows; a.entry_pos0 = entry_pos0; a.out = (bf16*)out;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.S = S; a.q_stride = q_stride; a.max_blocks = max_blocks; a.window = window; a.Hq = Hq; a.Hkv = Hkv; a.D = D;
  a.page = page;
  a.min_rows = min_rows;
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      num_sms = 148;
  }
  if (D <= 32) return launch_prefill<32>(a, max_tiles, num_sms, stream);
  if (D <= 64) return launch_prefill<64>(a, max_tiles, num_sms, stream);
  if (D <= 128) return launch_prefill<128>(a, max_tiles, num_sms, stream);
  return launch_prefill<256>(a, max_tiles, num_sms, stream);
}
