// Prefill attention on the 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05.mma with the
// accumulators in tensor memory, bfloat16 operands in shared memory.
//
// grid = (row tiles, query heads).  A CTA takes 128 consecutive rows of one request's portion and one query
// head, and walks the keys it can see in blocks of 64:
//   warp 0     one thread issues the TMA loads: the Q tile once, then per block the pages of K and of V
//              (boxes of one page x 64 elements, 128-byte swizzle, stacked into [64 keys][head_dim] tiles)
//   warp 1     allocates tensor memory; one thread issues the MMAs: S(i) = Q K(i)^T (both operands K-major),
//              and, once the softmax warps have written P(i), O += P(i) V(i) with V as an MN-major operand
//              (its tile is [key][d], d contiguous, exactly as the cache holds it)
//   warps 2-5  softmax: thread r of the four warps owns row r of the tile (tensor-memory lane r), so the row
//              maximum and sum need no exchange between threads.  It reads S(i) from tensor memory, masks by
//              position (causal, window), updates the running maximum, rescales O in tensor memory when the
//              maximum of some row of its warp moved (exactly: by exp2 of the difference), writes P(i) as
//              bfloat16 into shared memory in the swizzled K-major layout, and at the end reads O, divides by
//              the row sum and stores.
// S has two buffers in tensor memory and K two in shared memory: S(i+1) and S(i+2) are issued ahead, so the softmax
// warps go from block to block without waiting for the tensor core, and the tensor core computes S while they
// work.  Two CTAs share a multiprocessor and fill each other's gaps.  Every wait is bounded.
//
// Takes bfloat16, head_dim 64 or 128, pages of 16, 32 or 64 keys; everything else goes to the mma.sync kernel
// (attention_prefill.cu), which is also this kernel's twin in the tests.  (The reference's kernel:
// src/hip_ops.hip:473-551.)
#include "tcgen05.cuh"

#include <stdlib.h>

namespace {

constexpr int TQ = 128;          // rows per CTA: the M of the instruction, one tensor-memory lane per row
constexpr int TKB = 64;          // keys per block: one 128-byte swizzle row of P
constexpr int PT_THREADS = 192;
constexpr int BT_CAP = 1024;     // block-table entries kept in shared memory (16,384 keys with pages of 16)

struct PtArgs {
  const int* block_table;
  const int* cu_rows;       // [S + 1]
  const int* entry_pos0;    // [S]
  bf16* out;
  int* err;
  float scale_log2;         // scale * log2(e)
  int S, max_blocks, window, Hq, Hkv, page;
  int min_rows;             // entries with fewer rows are left to another kernel
  int first_wave;           // CTAs that start alone on a multiprocessor (their number), before the second ones join them
};

// 2^x by the special-function unit; exp2(-inf) = 0.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(PT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_v, PtArgs a) {
  constexpr int SL = D / 64;                       // 64-element slabs of the head dimension
  constexpr uint32_t Q_SLAB = TQ * 128, KV_SLAB = TKB * 128;
  extern __shared__ __align__(1024) uint8_t pt_smem_raw[];
  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full, v_empty, s_full[2], p_full, pv_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int tile_info[3];                     // entry, first row (batch), rows
  __shared__ int bt_s[BT_CAP];                     // the tile's block-table entries, fetched once up front

  uint8_t* smem = (uint8_t*)(((uintptr_t)pt_smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + SL * Q_SLAB;                  // two buffers
  uint8_t* Vs = Ks + 2 * SL * KV_SLAB;
  uint8_t* Ps = Vs + SL * KV_SLAB;                 // [128 rows][64 keys] bf16

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  // Which (tile, head) is this CTA's.  A causal tile's work grows with its place in the request, and two CTAs share
  // a multiprocessor: the CTAs that start alone on one (the first `first_wave` in launch order) take the tiles in
  // descending order of work, later tiles first and the heads of a tile side by side, and the CTAs that join them
  // take the rest in ascending order, so that a heavy tile shares its multiprocessor with a light one.  (Where a CTA
  // lands is the hardware's choice; the order only makes the even spread likely.  In launch order, tile by tile from
  // the heaviest, the 2,048-token prompt's attention took the time of its heaviest pair: 51 us a layer.)
  const int n_cta = (int)(gridDim.x * gridDim.y), cta = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  // (more CTAs than fit at once: plain descending order, the heaviest first, is the better schedule then)
  const int alone = n_cta <= 2 * a.first_wave ? min(n_cta, a.first_wave) : n_cta;
  const int rank = cta < alone ? cta : n_cta - 1 - (cta - alone);          // 0: the heaviest
  const int h = rank % a.Hq, kvh = h / (a.Hq / a.Hkv);

  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_v) : "memory");
    mbar_init(&q_full, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&k_full[b], 1);
      mbar_init(&k_empty[b], 1);
      mbar_init(&s_full[b], 1);
    }
    mbar_init(&v_full, 1);
    mbar_init(&v_empty, 1);
    mbar_init(&p_full, 4);                         // one arrival per softmax warp
    mbar_init(&pv_done, 1);
    mbar_fence_init();
  }
  // keys that a block never loads (beyond the last key, pages a window gave back) must still be finite numbers:
  // their probabilities are zero, and zero times whatever the shared memory held before must be zero
  for (int i = tid; i < (int)(3 * SL * KV_SLAB / 16); i += PT_THREADS) ((uint4*)Ks)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  if (warp == 1) tmem_alloc(&tmem_base_s, 256);
  grid_dep_wait();              // queries, and this step's keys and values, come from the kernel before
  grid_dep_launch();
  if (tid == 0) {               // which (entry, tile of 128 rows) is this CTA's?  later tiles (more keys) first
    int left = (int)gridDim.x - 1 - rank / a.Hq, e = 0, found = -1;
    for (; e < a.S; ++e) {
      const int n = a.cu_rows[e + 1] - a.cu_rows[e];
      const int tiles = n >= a.min_rows ? (n + TQ - 1) / TQ : 0;
      if (left < tiles) { found = e; break; }
      left -= tiles;
    }
    tile_info[0] = found;
    if (found >= 0) {
      tile_info[1] = a.cu_rows[found] + left * TQ;
      tile_info[2] = min(TQ, a.cu_rows[found + 1] - tile_info[1]);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const int e = tile_info[0];
  if (e >= 0) {
    const int row0 = tile_info[1], nrows = tile_info[2];
    const int pos0 = a.entry_pos0[e] + (row0 - a.cu_rows[e]);      // position of the tile's first row
    const int hi = pos0 + nrows;                                   // keys [.., hi) exist for this tile
    const int lo = a.window > 0 ? max(0, pos0 + 1 - a.window) : 0; // first key any row of the tile sees
    const int kv0 = lo / TKB * TKB;
    const int n_blocks = (hi - kv0 + TKB - 1) / TKB;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * TKB;     // S(even), S(odd), O
    const int* bt = a.block_table + (size_t)e * a.max_blocks;
    const int page_shift = 31 - __clz(a.page);                     // pages are 16, 32 or 64 keys
    const int pg0 = kv0 >> page_shift, n_pg = min(((hi - 1) >> page_shift) + 1 - pg0, BT_CAP);
    for (int i = tid; i < n_pg; i += PT_THREADS) bt_s[i] = bt[pg0 + i];
    __syncthreads();

    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      // The whole warp works: a tile of keys (or values) is pages x slabs boxes, and lane (page, slab) issues its
      // own box, so a tile costs one instruction's time and not a thread's walk over sixteen of them.
      if (lane == 0) {
        mbar_expect_tx(&q_full, SL * Q_SLAB);
#pragma unroll
        for (int s = 0; s < SL; ++s) tma_load_2d(Qs + s * Q_SLAB, &tm_q, &q_full, h * D + s * 64, row0);
      }
      const int pages = TKB >> page_shift;
      const uint32_t box = (uint32_t)a.page * 128;
      const int my_p = lane / SL, my_s = lane % SL;
      auto load = [&](int i, bool values) {
        const int j = kv0 + i * TKB + (my_p << page_shift);          // first key of this lane's page
        int blk = -1;
        if (my_p < pages && j < hi && j + a.page > lo) {               // a page some row can see
          const int pi = (j >> page_shift) - pg0;
          blk = pi < BT_CAP ? bt_s[pi] : bt[pg0 + pi];
          if (blk < 0) atomicExch(a.err, 1 + row0);                    // it should be there and is not
        }
        const uint32_t boxes = __popc(__ballot_sync(0xffffffffu, blk >= 0));
        uint64_t* full = values ? &v_full : &k_full[i & 1];
        if (lane == 0) {
          if (values) mbar_wait(&v_empty, (i & 1) ^ 1, a.err, 0x7202);
          else mbar_wait(&k_empty[i & 1], ((i >> 1) & 1) ^ 1, a.err, 0x7201);
          mbar_expect_tx(full, boxes * box);
        }
        __syncwarp();
        if (blk >= 0) {
          uint8_t* dst = (values ? Vs : Ks + (i & 1) * SL * KV_SLAB) + my_s * KV_SLAB + my_p * box;
          tma_load_2d(dst, values ? &tm_v : &tm_k, full, my_s * 64, (blk * a.Hkv + kvh) * a.page);
        }
      };
      load(0, false);
      for (int i = 0; i < n_blocks; ++i) {         // the next keys go out before these values: they are free earlier
        if (i + 1 < n_blocks) load(i + 1, false);
        load(i, true);
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        const uint32_t idesc_s = instr_desc(TKB), idesc_o = instr_desc_b_mn(D);
        const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Ks), v_addr = smem_u32(Vs), p_addr = smem_u32(Ps);
        // one thread issues everything, so its instruction count is on the critical path: the descriptors are
        // built once, a product costs an add and the instruction
        uint64_t dq[SL], dk[2][SL], dv[TKB / 16];
#pragma unroll
        for (int s = 0; s < SL; ++s) {
          dq[s] = smem_desc_sw128(q_addr + s * Q_SLAB);
          dk[0][s] = smem_desc_sw128(k_addr + s * KV_SLAB);
          dk[1][s] = smem_desc_sw128(k_addr + (SL + s) * KV_SLAB);
        }
#pragma unroll
        for (int kk = 0; kk < TKB / 16; ++kk) dv[kk] = smem_desc_sw128_mn(v_addr + kk * 2048, KV_SLAB, 1024);
        const uint64_t dp = smem_desc_sw128(p_addr);
        auto issue_s = [&](int i) {
          const int b = i & 1;
          mbar_wait(&k_full[b], (i >> 1) & 1, a.err, 0x7203);
          tc_fence_after();
#pragma unroll
          for (int s = 0; s < SL; ++s)           // the four 16-wide slices of a 64-element slab in one block
            umma_bf16_x4(tmem_s + b * TKB, dq[s], b ? dk[1][s] : dk[0][s], idesc_s, s ? 1u : 0u);
          umma_commit(&k_empty[b]);
          umma_commit(&s_full[b]);
        };
        mbar_wait(&q_full, 0, a.err, 0x7204);
        issue_s(0);
        if (n_blocks > 1) issue_s(1);
        for (int i = 0; i < n_blocks; ++i) {
          mbar_wait(&p_full, i & 1, a.err, 0x7205);  // P(i) is written, S(i) is read, O is rescaled
          mbar_wait(&v_full, i & 1, a.err, 0x7206);
          tc_fence_after();
          // 16 keys per product: 32 bytes (2 units) along P's rows, two 8-key groups (2,048 bytes = 128 units) of V
          umma_bf16_x4s(tmem_o, dp, dv[0], idesc_o, i ? 1u : 0u, 2, 128);
          umma_commit(&v_empty);
          umma_commit(&pv_done);
          if (i + 2 < n_blocks) issue_s(i + 2);      // into the buffer that S(i) has left
        }
      }
    } else {
      // ---------------------------------------------------------------- softmax: thread r owns row r
      const int q = warp % 4;                        // a warp may touch tensor-memory lanes [32q, 32q + 32) only
      const int r = q * 32 + lane;
      const int p_row = pos0 + r;
      const bool live = r < nrows;
      const int w_lo = a.window > 0 ? p_row + 1 - a.window : 0;
      const uint32_t lane_off = (uint32_t)(q * 32) << 16;
      float m = -INFINITY, l = 0.f;
      for (int i = 0; i < n_blocks; ++i) {
        const int j0 = kv0 + i * TKB;
        mbar_wait(&s_full[i & 1], (i >> 1) & 1, a.err, 0x7207);
        tc_fence_after();
        float s[TKB];
        tmem_ld32_nowait(tmem_s + (i & 1) * TKB + lane_off, s);
        tmem_ld32_nowait(tmem_s + (i & 1) * TKB + lane_off + 32, s + 32);
        tmem_ld_wait();
        tmem_ld_fence<64>(s);
        if (!live || j0 + TKB - 1 > p_row || j0 < w_lo) {
#pragma unroll
          for (int c = 0; c < TKB; ++c)
            if (!(live && j0 + c <= p_row && j0 + c >= w_lo)) s[c] = -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains instead of one of 64
#pragma unroll
        for (int c = 0; c < TKB; c += 4) {
          mx4[0] = fmaxf(mx4[0], s[c]); mx4[1] = fmaxf(mx4[1], s[c + 1]);
          mx4[2] = fmaxf(mx4[2], s[c + 2]); mx4[3] = fmaxf(mx4[3], s[c + 3]);
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // The exponent's reference m follows the running maximum only when that has moved by more than 2^8 in
        // the scaled (log2) units: P = exp2(s - m) may then be as large as 256, which costs bfloat16 and the
        // float32 sums nothing, O / l is the same quotient, and O in tensor memory is rescaled once in a long
        // while instead of at almost every block of a short prompt.
        float alpha = 1.f;
        if (mx > m && (m == -INFINITY || (mx - m) * a.scale_log2 > 8.f)) {
          alpha = m == -INFINITY ? 0.f : ex2_approx((m - mx) * a.scale_log2);
          m = mx;
        }
        const float ms = m == -INFINITY ? 0.f : m * a.scale_log2;
        // O += P(i-1) V(i-1) must have ended before O is rescaled and before P is overwritten
        if (i > 0) {
          mbar_wait(&pv_done, (i - 1) & 1, a.err, 0x7209);
          tc_fence_after();
        }
        if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            float o[32];
            tmem_ld32(tmem_o + lane_off + c * 32, o);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= alpha;
            tmem_st32(tmem_o + lane_off + c * 32, o);
          }
        }
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < TKB; c += 4) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            s[c + u] = ex2_approx(fmaf(s[c + u], a.scale_log2, -ms));
            sum4[u] += s[c + u];
          }
        }
        l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        // P row r: 8 chunks of 8 bfloat16, chunk c at physical chunk c ^ (r % 8) (the 128-byte swizzle)
        uint8_t* prow = Ps + (size_t)r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 v;
          __nv_bfloat162 t0 = __floats2bfloat162_rn(s[c * 8 + 0], s[c * 8 + 1]);
          __nv_bfloat162 t1 = __floats2bfloat162_rn(s[c * 8 + 2], s[c * 8 + 3]);
          __nv_bfloat162 t2 = __floats2bfloat162_rn(s[c * 8 + 4], s[c * 8 + 5]);
          __nv_bfloat162 t3 = __floats2bfloat162_rn(s[c * 8 + 6], s[c * 8 + 7]);
          v.x = *(uint32_t*)&t0; v.y = *(uint32_t*)&t1; v.z = *(uint32_t*)&t2; v.w = *(uint32_t*)&t3;
          *(uint4*)(prow + ((c ^ (r & 7)) << 4)) = v;
        }
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full);
      }
      // ---- the result: O / l
      mbar_wait(&pv_done, (n_blocks - 1) & 1, a.err, 0x7208);
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld32(tmem_o + lane_off + c * 32, o);
        if (live) {
          bf16* dst = a.out + ((size_t)(row0 + r) * a.Hq + h) * D + c * 32;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(o[j + 0] * inv, o[j + 1] * inv);
            __nv_bfloat162 t1 = __floats2bfloat162_rn(o[j + 2] * inv, o[j + 3] * inv);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(o[j + 4] * inv, o[j + 5] * inv);
            __nv_bfloat162 t3 = __floats2bfloat162_rn(o[j + 6] * inv, o[j + 7] * inv);
            v.x = *(uint32_t*)&t0; v.y = *(uint32_t*)&t1; v.z = *(uint32_t*)&t2; v.w = *(uint32_t*)&t3;
            *(uint4*)(dst + j) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

template <int D>
int launch_prefill_tc(const PtArgs& a, const void* qkv, int q_stride, int T, const void* kc, const void* vc,
                      int num_pages, int max_tiles, cudaStream_t s) {
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = nv_tensor_map_bf16(qkv, T, q_stride, q_stride, TQ, &tm_q);
  if (rc) return rc;
  const long long rows = (long long)num_pages * a.Hkv * a.page;
  rc = nv_tensor_map_bf16(kc, rows, D, D, a.page, &tm_k);
  if (rc) return rc;
  rc = nv_tensor_map_bf16(vc, rows, D, D, a.page, &tm_v);
  if (rc) return rc;
  constexpr int SL = D / 64;
  const size_t smem = (size_t)SL * TQ * 128 + 3 * (size_t)SL * TKB * 128 + (size_t)TQ * 128 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  dim3 grid(max_tiles > 0 ? max_tiles : 1, a.Hq);
  NV_RETURN_IF(launch_dep(attention_prefill_tc_kernel<D>, grid, dim3(PT_THREADS), smem, s, tm_q, tm_k, tm_v, a));
  NV_RETURN_LAST();
}

}  // namespace

NV_API int nv_attention_prefill_tc_usable(int D, int page) {
  return (D == 64 || D == 128) && (page == 16 || page == 32 || page == 64);
}

// Same contract as nv_attention_prefill (max_tiles counts tiles of nv_attention_prefill_tile_rows() = 64 rows, an
// upper bound), plus the number of rows T of qkv, the pages of the cache, and the error flag.  An entry of n rows
// has ceil(n / 128) <= (ceil(n / 64) + 1) / 2 tiles here, so (max_tiles + S + 1) / 2 CTAs per head are enough;
// surplus CTAs leave at once.
NV_API int nv_attention_prefill_tc(const void* qkv, int q_stride, int T, const void* kc, const void* vc, int num_pages,
                                   const int* block_table, int max_blocks, const int* cu_rows, const int* entry_pos0,
                                   int S, int max_tiles, float scale, int window, void* out, int Hq, int Hkv, int D,
                                   int page, int min_rows, int* err, cudaStream_t stream) {
  if (!nv_attention_prefill_tc_usable(D, page) || Hkv <= 0 || Hq % Hkv) return NV_ERR_UNSUPPORTED;
  if (q_stride % 8 || ((uintptr_t)qkv & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15)) return NV_ERR_UNSUPPORTED;
  if (S == 0 || max_tiles == 0 || T == 0) return NV_OK;
  PtArgs a;
  a.block_table = block_table; a.cu_rows = cu_rows; a.entry_pos0 = entry_pos0; a.out = (bf16*)out; a.err = err;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.S = S; a.max_blocks = max_blocks; a.window = window; a.Hq = Hq; a.Hkv = Hkv; a.page = page;
  a.min_rows = min_rows;
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  a.first_wave = num_sms;
  const int tiles = (max_tiles + S + 1) / 2;
  if (D == 64) return launch_prefill_tc<64>(a, qkv, q_stride, T, kc, vc, num_pages, tiles, stream);
  return launch_prefill_tc<128>(a, qkv, q_stride, T, kc, vc, num_pages, tiles, stream);
}
