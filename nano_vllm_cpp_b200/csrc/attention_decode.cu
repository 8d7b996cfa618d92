// Decode attention: one query row per request against its paged keys and values, split over the
// keys so that a few requests still fill the GPU.
//
// grid = (rows, kv heads x head groups, splits).  A block streams its share of one request's pages
// once, for up to GB query heads that share the kv head.  A page's rows of one kv head are
// contiguous in the cache, so a producer warp fetches them with bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier) into a ring of shared-memory stages, several pages
// ahead of the four consumer warps; that keeps tens of kilobytes in flight per SM, which is what the
// memory system needs to run at full speed.  Inside a consumer warp, groups of 8 lanes own one
// key each; a lane holds 8-element chunks of the head dimension, so a dot product needs three
// shuffles.  Every (warp, lane group) keeps its own running max / sum / output (online softmax,
// float32) and the partial results are merged at the end: lane groups by shuffles, warps through
// shared memory, splits by a second small kernel.  The merge order is fixed, so a row's result does
// not depend on the batch.  Keys of row t at position p: [max(0, p + 1 - window), p].
//
// Reference twin: nv_paged_attention_plain.  (The reference's kernel: src/hip_ops.hip:473-551.)
#include "pipeline.cuh"

#include <cstdlib>

namespace {

constexpr int WARPS = 4;                // consumer warps; one more warp produces
constexpr int MAX_STAGES = 16;
constexpr int BT_CACHE = 1024;           // block-table entries of a split kept in shared memory
constexpr int LPK = 8;                 // lanes per key
constexpr int KEYS_PER_WARP = 32 / LPK;
constexpr int KEYS_PER_PASS = WARPS * KEYS_PER_WARP;   // 16

template <typename T>
struct Chunk;                           // 8 consecutive elements as floats
template <>
struct Chunk<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float* v) {
    uint4 r = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&r;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};
template <>
struct Chunk<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

struct DecArgs {
  const void* qkv;
  const void* kc;
  const void* vc;
  const int* block_table;
  const int* row_entry;
  const int* positions;
  const int* rows;        // which batch rows to process (null: all, row = blockIdx.x)
  void* out;
  float* part_o;          // [rows, Hq, splits, D]
  float* part_ml;         // [rows, Hq, splits, 2]
  int* split_count;       // [rows, gridDim.y] zeros, or null: how many splits of a (row, group of heads) have finished
  int* err;
  float scale;
  int q_dt, out_dt, q_stride, max_blocks, window, Hq, Hkv, D, page, splits, stages;
};

// Called by every thread of a block once the block has written its split's partial results for the query heads
// h0 .. h0 + nh - 1 of row r (batch row t): the block that arrives last for this (row, group of heads) adds the splits
// up, in split order and with the arithmetic of attention_decode_merge_kernel, and writes the result; the others
// leave.  That saves the merge kernel's launch, which stands between the attention and the output projection of
// every layer.  The count goes back to zero for the next launch.
__device__ __forceinline__ void merge_when_last(const DecArgs& a, int r, int t, int h0, int nh, int D) {
  __shared__ int last_s;
  __threadfence();                      // this block's partial results are visible to every block ...
  __syncthreads();
  if (threadIdx.x == 0) {
    int* c = a.split_count + (size_t)r * gridDim.y + blockIdx.y;
    const int ticket = atomicAdd(c, 1); // ... before its arrival is
    last_s = ticket == a.splits - 1;
    if (last_s) *c = 0;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
    const int h = h0 + i / D, d = i % D;
    const size_t pi = ((size_t)r * a.Hq + h) * a.splits;
    float mm = -1e30f;
    for (int s = 0; s < a.splits; ++s) mm = fmaxf(mm, __ldcg(a.part_ml + (pi + s) * 2));
    float ll = 0.f, o = 0.f;
    for (int s = 0; s < a.splits; ++s) {
      const float sc = __expf(__ldcg(a.part_ml + (pi + s) * 2) - mm);
      ll = fmaf(__ldcg(a.part_ml + (pi + s) * 2 + 1), sc, ll);
      o = fmaf(__ldcg(a.part_o + (pi + s) * D + d), sc, o);
    }
    st_dt(a.out, a.out_dt, ((size_t)t * a.Hq + h) * D + d, o * (ll > 0.f ? 1.f / ll : 0.f));
  }
}

// CPL: chunks of 8 elements per lane (D <= 64 * CPL); GB: query heads per block.
template <typename TC, int CPL, int GB>
__global__ void __launch_bounds__((WARPS + 1) * 32) attention_decode_kernel(DecArgs a) {
  extern __shared__ __align__(128) uint8_t dec_smem[];
  __shared__ __align__(16) float q_s[GB][256];           // (read four floats at a time)
  __shared__ __align__(16) float mrg_o[WARPS][GB][256];
  __shared__ float mrg_m[WARPS][GB], mrg_l[WARPS][GB];
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
  __shared__ int bt_s[BT_CACHE];          // this split's block-table entries, fetched once up front

  const int r = blockIdx.x;
  const int t = a.rows ? a.rows[r] : r;
  const int G = a.Hq / a.Hkv;
  const int groups = (G + GB - 1) / GB;
  const int kvh = blockIdx.y / groups;
  const int g0 = (blockIdx.y % groups) * GB;          // first query head of the kv head handled here
  const int ng = min(GB, G - g0);
  const int split = blockIdx.z;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int sub = lane / LPK, li = lane % LPK;
  const int D = a.D, chunks = D / 8;

  const int n = a.positions[t] + 1;
  const int lo = a.window > 0 ? max(0, n - a.window) : 0;
  // this split's pages
  const int p_lo = lo / a.page, p_hi = (n - 1) / a.page + 1;
  const int per = (p_hi - p_lo + a.splits - 1) / a.splits;
  const int pb = p_lo + split * per;
  const int n_pages = max(0, min(p_hi, pb + per) - pb);
  const uint32_t chunk_bytes = (uint32_t)a.page * D * sizeof(TC);

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], WARPS);
    }
    mbar_fence_init();
  }
  grid_dep_wait();              // the queries and the newest keys come from the kernel before
  grid_dep_launch();
  for (int i = threadIdx.x; i < ng * D; i += (WARPS + 1) * 32) {
    int g = i / D, d = i % D;
    q_s[g][d] = ld_dt(a.qkv, a.q_dt, (size_t)t * a.q_stride + (size_t)(kvh * G + g0 + g) * D + d) * a.scale;
  }
  const int* bt = a.block_table + (size_t)a.row_entry[t] * a.max_blocks;
  // the producer must not wait for a block-table entry per page: that load's latency would bound the stream
  for (int i = threadIdx.x; i < min(n_pages, BT_CACHE); i += (WARPS + 1) * 32) bt_s[i] = bt[pb + i];
  __syncthreads();

  if (warp == WARPS) {
    // ---------------------------------------------------------------- producer: one lane issues the copies
    if (lane == 0) {
      for (int i = 0; i < n_pages; ++i) {
        const int s = i % a.stages;
        mbar_wait(&empty_bar[s], ((i / a.stages) & 1) ^ 1, a.err, 0x7101);
        const int blk = i < BT_CACHE ? bt_s[i] : bt[pb + i];
        uint8_t* st = dec_smem + (size_t)s * 2 * chunk_bytes;
        if (blk < 0) {                       // a page that should be there is not: report, let the consumers pass
          if (a.err) atomicExch(a.err, 1 + t);
          mbar_arrive(&full_bar[s]);
          continue;
        }
        const size_t off = ((size_t)blk * a.Hkv + kvh) * a.page * D;
        mbar_expect_tx(&full_bar[s], 2 * chunk_bytes);
        bulk_load(st, (const TC*)a.kc + off, chunk_bytes, &full_bar[s]);
        bulk_load(st + chunk_bytes, (const TC*)a.vc + off, chunk_bytes, &full_bar[s]);
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers
    float m[GB], l[GB], acc[GB][CPL][8];
#pragma unroll
    for (int g = 0; g < GB; ++g) {
      m[g] = -1e30f;
      l[g] = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][c][e] = 0.f;
    }
    // with one query head per block its chunks of q live in registers; otherwise they are read from shared memory
    float qr[GB == 1 ? CPL : 1][8];
    if (GB == 1) {
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = li + c * LPK;
#pragma unroll
        for (int e = 0; e < 8; ++e) qr[c][e] = ch < chunks ? q_s[0][ch * 8 + e] : 0.f;
      }
    }
    for (int i = 0; i < n_pages; ++i) {
      const int s = i % a.stages;
      mbar_wait(&full_bar[s], (i / a.stages) & 1, a.err, 0x7102);
      const TC* ks = (const TC*)(dec_smem + (size_t)s * 2 * chunk_bytes);
      const TC* vs = (const TC*)(dec_smem + (size_t)s * 2 * chunk_bytes + chunk_bytes);
      for (int slot = warp * KEYS_PER_WARP + sub; slot < a.page; slot += KEYS_PER_PASS) {
        const int j = (pb + i) * a.page + slot;
        const bool live = j >= lo && j < n;
        float kf[CPL][8], vf[CPL][8];
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          const int ch = li + c * LPK;
          if (ch < chunks) {
            Chunk<TC>::load(ks + (size_t)slot * D + ch * 8, kf[c]);
            Chunk<TC>::load(vs + (size_t)slot * D + ch * 8, vf[c]);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) kf[c][e] = vf[c][e] = 0.f;
          }
        }
#pragma unroll
        for (int g = 0; g < GB; ++g) {
          if (g >= ng) break;
          float sc = 0.f;
#pragma unroll
          for (int c = 0; c < CPL; ++c) {
            const int ch = li + c * LPK;
            if (GB == 1) {
#pragma unroll
              for (int e = 0; e < 8; ++e) sc = fmaf(qr[c][e], kf[c][e], sc);     // kf is zero beyond the head
            } else if (ch < chunks) {
              const float4 qa = *(const float4*)&q_s[g][ch * 8], qb = *(const float4*)&q_s[g][ch * 8 + 4];
              sc = fmaf(qa.x, kf[c][0], sc); sc = fmaf(qa.y, kf[c][1], sc); sc = fmaf(qa.z, kf[c][2], sc);
              sc = fmaf(qa.w, kf[c][3], sc); sc = fmaf(qb.x, kf[c][4], sc); sc = fmaf(qb.y, kf[c][5], sc);
              sc = fmaf(qb.z, kf[c][6], sc); sc = fmaf(qb.w, kf[c][7], sc);
            }
          }
          sc += __shfl_xor_sync(0xffffffffu, sc, 1);
          sc += __shfl_xor_sync(0xffffffffu, sc, 2);
          sc += __shfl_xor_sync(0xffffffffu, sc, 4);
          if (live) {
            if (sc > m[g]) {                       // a new maximum (rare after the first keys): rescale what was summed
              const float alpha = __expf(m[g] - sc);
              l[g] *= alpha;
#pragma unroll
              for (int c = 0; c < CPL; ++c)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][c][e] *= alpha;
              m[g] = sc;
            }
            const float p = __expf(sc - m[g]);
            l[g] += p;
#pragma unroll
            for (int c = 0; c < CPL; ++c)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[g][c][e] = fmaf(p, vf[c][e], acc[g][c][e]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);   // this warp is done with the stage
    }

    // merge the four lane groups of the warp (xor 8, 16), in a fixed order
#pragma unroll
    for (int g = 0; g < GB; ++g) {
#pragma unroll
      for (int off = LPK; off < 32; off <<= 1) {
        const float m_o = __shfl_xor_sync(0xffffffffu, m[g], off);
        const float l_o = __shfl_xor_sync(0xffffffffu, l[g], off);
        const float m_new = fmaxf(m[g], m_o);
        const float sa = __expf(m[g] - m_new), sb = __expf(m_o - m_new);
        l[g] = l[g] * sa + l_o * sb;
#pragma unroll
        for (int c = 0; c < CPL; ++c)
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float o = __shfl_xor_sync(0xffffffffu, acc[g][c][e], off);
            acc[g][c][e] = acc[g][c][e] * sa + o * sb;
          }
        m[g] = m_new;
      }
      if (sub == 0) {
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          const int ch = li + c * LPK;
          if (ch < chunks)
#pragma unroll
            for (int e = 0; e < 8; ++e) mrg_o[warp][g][ch * 8 + e] = acc[g][c][e];
        }
        if (li == 0) {
          mrg_m[warp][g] = m[g];
          mrg_l[warp][g] = l[g];
        }
      }
    }
  }
  __syncthreads();
  // merge the warps and write this split's result
  for (int i = threadIdx.x; i < ng * D; i += (WARPS + 1) * 32) {
    const int g = i / D, d = i % D;
    float mm = mrg_m[0][g];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) mm = fmaxf(mm, mrg_m[w][g]);
    float ll = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float sc = __expf(mrg_m[w][g] - mm);
      ll = fmaf(mrg_l[w][g], sc, ll);
      o = fmaf(mrg_o[w][g][d], sc, o);
    }
    const int h = kvh * G + g0 + g;
    if (a.splits == 1) {
      st_dt(a.out, a.out_dt, ((size_t)t * a.Hq + h) * D + d, ll > 0.f ? o / ll : 0.f);
    } else {
      const size_t pi = ((size_t)r * a.Hq + h) * a.splits + split;
      a.part_o[pi * D + d] = o;
      if (d == 0) {
        a.part_ml[pi * 2] = mm;
        a.part_ml[pi * 2 + 1] = ll;
      }
    }
  }
  if (a.splits > 1 && a.split_count) merge_when_last(a, r, t, kvh * G + g0, ng, D);
}

// ---------------------------------------------------------------------------------------------
// The tensor-core form, for bfloat16 caches whose head dimension is a multiple of 64.
//
// The lane-per-chunk kernel above spends a few hundred instructions per key and page, and on this
// GPU the instruction issue rate, not memory, then bounds it at about half of the memory speed.
// Here a warp takes a whole page: S = Q K^T and O += P V are m16n8k16 bf16 MMAs whose 16 rows are
// the query heads that share the kv head (rows beyond them are zero), about ninety instructions per
// page.  Pages arrive by tiled TMA copies (boxes of `page` keys x 64 elements, 128-byte swizzle) so
// that ldmatrix reads them without bank conflicts; the ring, the split over keys and the merges are
// those of the kernel above.
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

constexpr int TC_ROWS = 16;      // query heads per block (rows of the MMA)

// D: head dimension, a multiple of 64 (compile time: it sizes the fragments).
template <int D>
__global__ void __launch_bounds__((WARPS + 1) * 32, D <= 128 ? 3 : 1)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                           DecArgs a) {
  extern __shared__ __align__(1024) uint8_t dec_smem_raw[];
  constexpr int QLD = D + 8;                         // padded row of q in shared memory
  __shared__ __align__(16) bf16 q_s[TC_ROWS * QLD];
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
  __shared__ int bt_s[BT_CACHE];
  __shared__ float mrg_m[WARPS][TC_ROWS], mrg_l[WARPS][TC_ROWS];

  uint8_t* dec_smem = (uint8_t*)(((uintptr_t)dec_smem_raw + 1023) & ~(uintptr_t)1023);
  const int r = blockIdx.x;
  const int t = a.rows ? a.rows[r] : r;
  const int G = a.Hq / a.Hkv;
  const int groups = (G + TC_ROWS - 1) / TC_ROWS;
  const int kvh = blockIdx.y / groups;
  const int g0 = (blockIdx.y % groups) * TC_ROWS;
  const int ng = min(TC_ROWS, G - g0);
  const int split = blockIdx.z;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

  const int n = a.positions[t] + 1;
  const int lo = a.window > 0 ? max(0, n - a.window) : 0;
  const int p_lo = lo / a.page, p_hi = (n - 1) / a.page + 1;
  const int per = (p_hi - p_lo + a.splits - 1) / a.splits;
  const int pb = p_lo + split * per;
  const int n_pages = max(0, min(p_hi, pb + per) - pb);
  const uint32_t box_bytes = (uint32_t)a.page * 128;           // one box: `page` keys x 64 elements
  const uint32_t half_stage = box_bytes * (D / 64);            // keys of one page; values follow
  const uint32_t stage_bytes = 2 * half_stage;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_v) : "memory");
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);                   // a stage is read by one warp
    }
    mbar_fence_init();
  }
  // Launched as a programmatic dependent, the kernel may run beside the one that rotates the queries and writes
  // the newest key and value.  The block table and the positions are inputs of the whole step; every page but
  // the one that holds position n - 1 is final.  So the producer starts on the older pages at once, and the
  // queries, the newest page and all writes come after the wait.
  const int* bt = a.block_table + (size_t)a.row_entry[t] * a.max_blocks;
  for (int i = threadIdx.x; i < min(n_pages, BT_CACHE); i += (WARPS + 1) * 32) bt_s[i] = bt[pb + i];
  __syncthreads();
  if (warp < WARPS) {
    grid_dep_wait();
    grid_dep_launch();
    for (int i = threadIdx.x; i < TC_ROWS * D; i += WARPS * 32) {
      const int g = i / D, d = i % D;
      float v = 0.f;
      if (g < ng) v = ld_dt(a.qkv, a.q_dt, (size_t)t * a.q_stride + (size_t)(kvh * G + g0 + g) * D + d);
      q_s[g * QLD + d] = __float2bfloat16_rn(v);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");      // the consumer warps only
  }

  const int g = lane / 4, tq = lane % 4;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[D / 8][4];

  if (warp == WARPS) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      const int newest = (n - 1) / a.page - pb;          // this split's page that is still being written
      bool waited = false;
      int s = 0;                                   // stage of page i and the parity of its use, kept by counting
      uint32_t ph = 0;                             // (this one thread's instructions pace the ring)
      for (int i = 0; i < n_pages; ++i, s = (s + 1 == a.stages ? 0 : s + 1), ph ^= (s == 0)) {
        if (!waited && (i >= a.stages || i == newest)) {
          grid_dep_wait();
          waited = true;
        }
        mbar_wait(&empty_bar[s], ph ^ 1, a.err, 0x7111);
        const int blk = i < BT_CACHE ? bt_s[i] : bt[pb + i];
        uint8_t* st = dec_smem + (size_t)s * stage_bytes;
        if (blk < 0) {
          if (!waited) {
            grid_dep_wait();
            waited = true;
          }
          if (a.err) atomicExch(a.err, 1 + t);
          mbar_arrive(&full_bar[s]);
          continue;
        }
        const int row = (blk * a.Hkv + kvh) * a.page;          // first row of the page in the [rows, D] view
        mbar_expect_tx(&full_bar[s], stage_bytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(st + c * box_bytes, &tm_k, &full_bar[s], c * 64, row);
          tma_load_2d(st + half_stage + c * box_bytes, &tm_v, &full_bar[s], c * 64, row);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers: warp w takes pages w, w+4, ...
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    uint32_t qa[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      ldsm4(smem_u32(q_s + ((lane % 8) + 8 * ((lane / 8) % 2)) * QLD + kk * 16 + 8 * (lane / 16)), qa[kk][0], qa[kk][1],
            qa[kk][2], qa[kk][3]);
    int s = warp % a.stages;                       // stage of page i (the ring is a multiple of WARPS stages deep)
    uint32_t ph = (warp / a.stages) & 1;
    const uint32_t smem0 = smem_u32(dec_smem);
    for (int i = warp; i < n_pages; i += WARPS) {
      mbar_wait(&full_bar[s], ph, a.err, 0x7112);
      const uint32_t kbase = smem0 + (uint32_t)s * stage_bytes;
      const uint32_t vbase = kbase + half_stage;
      const int j_page = (pb + i) * a.page;
      for (int kb = 0; kb < a.page / 16; ++kb) {
        const int j0 = j_page + kb * 16;
        if (j0 >= n || j0 + 15 < lo) continue;                 // uniform: no visible key in these 16
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        {
          const int key = kb * 16 + (lane % 8) + 8 * (lane / 16);
          const uint32_t rowaddr = kbase + key * 128;
          const int half8 = (lane / 8) % 2;                    // which 8-element half of the 16-wide k block
          // fragments are fetched four k-blocks at a time before their products, so that the latency of
          // ldmatrix is paid once per batch and not once per product
#pragma unroll
          for (int k4 = 0; k4 < D / 64; ++k4) {
            uint32_t b[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int chunk = u * 2 + half8;                  // 16-byte chunk inside the 128-byte row of box k4
              ldsm4(rowaddr + k4 * box_bytes + ((chunk ^ (key & 7)) << 4), b[u][0], b[u][1], b[u][2], b[u][3]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              mma16816(s0, qa[k4 * 4 + u], b[u][0], b[u][1]);
              mma16816(s1, qa[k4 * 4 + u], b[u][2], b[u][3]);
            }
          }
        }
        // mask keys outside [lo, n): all rows of a decode step share the range
        if (j0 < lo || j0 + 15 >= n) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int ja = j0 + 2 * tq + c, jb = ja + 8;
            if (ja < lo || ja >= n) s0[c] = s0[2 + c] = -INFINITY;
            if (jb < lo || jb >= n) s1[c] = s1[2 + c] = -INFINITY;
          }
        }
        float mx_lo = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
        float mx_hi = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo * a.scale, ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi * a.scale;
        const float al_lo = exp2f(m_lo * a.scale - ms_lo), al_hi = exp2f(m_hi * a.scale - ms_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        s0[0] = exp2f(s0[0] * a.scale - ms_lo); s0[1] = exp2f(s0[1] * a.scale - ms_lo);
        s1[0] = exp2f(s1[0] * a.scale - ms_lo); s1[1] = exp2f(s1[1] * a.scale - ms_lo);
        s0[2] = exp2f(s0[2] * a.scale - ms_hi); s0[3] = exp2f(s0[3] * a.scale - ms_hi);
        s1[2] = exp2f(s1[2] * a.scale - ms_hi); s1[3] = exp2f(s1[3] * a.scale - ms_hi);
        l_lo = l_lo * al_lo + (s0[0] + s0[1] + s1[0] + s1[1]);
        l_hi = l_hi * al_hi + (s0[2] + s0[3] + s1[2] + s1[3]);
        if (al_lo != 1.f || al_hi != 1.f) {
#pragma unroll
          for (int i2 = 0; i2 < D / 8; ++i2) {
            o[i2][0] *= al_lo; o[i2][1] *= al_lo; o[i2][2] *= al_hi; o[i2][3] *= al_hi;
          }
        }
        uint32_t pa[4] = {pack_bf16(s0[0], s0[1]), pack_bf16(s0[2], s0[3]), pack_bf16(s1[0], s1[1]),
                          pack_bf16(s1[2], s1[3])};
        {
          const int key = kb * 16 + (lane % 8) + 8 * ((lane / 8) % 2);
          const uint32_t rowaddr = vbase + key * 128;
          const int half8 = lane / 16;
#pragma unroll
          for (int d4 = 0; d4 < D / 64; ++d4) {
            uint32_t b[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int chunk = u * 2 + half8;
              ldsm4_t(rowaddr + d4 * box_bytes + ((chunk ^ (key & 7)) << 4), b[u][0], b[u][1], b[u][2], b[u][3]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              mma16816(o[2 * (d4 * 4 + u)], pa, b[u][0], b[u][1]);
              mma16816(o[2 * (d4 * 4 + u) + 1], pa, b[u][2], b[u][3]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
      s += WARPS;
      if (s >= a.stages) { s -= a.stages; ph ^= 1; }
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  }
  __syncthreads();          // every page has been read: the ring's memory is free for the merge
  float* mrg_o = (float*)dec_smem;                              // [WARPS][ng][D]
  if (warp < WARPS) {
    if (tq == 0) {
      if (g < ng) { mrg_m[warp][g] = m_lo; mrg_l[warp][g] = l_lo; }
      if (g + 8 < ng) { mrg_m[warp][g + 8] = m_hi; mrg_l[warp][g + 8] = l_hi; }
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int d = i * 8 + 2 * tq;
      if (g < ng) { mrg_o[((size_t)warp * ng + g) * D + d] = o[i][0]; mrg_o[((size_t)warp * ng + g) * D + d + 1] = o[i][1]; }
      if (g + 8 < ng) {
        mrg_o[((size_t)warp * ng + g + 8) * D + d] = o[i][2];
        mrg_o[((size_t)warp * ng + g + 8) * D + d + 1] = o[i][3];
      }
    }
  }
  __syncthreads();
  // merge the warps (fixed order) and write this split's result; scores are in log2 units here
  for (int i = threadIdx.x; i < ng * D; i += (WARPS + 1) * 32) {
    const int gg = i / D, d = i % D;
    float mm = mrg_m[0][gg];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) mm = fmaxf(mm, mrg_m[w][gg]);
    const float mms = mm == -INFINITY ? 0.f : mm * a.scale;
    float ll = 0.f, ov = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float sc = exp2f(mrg_m[w][gg] * a.scale - mms);
      ll = fmaf(mrg_l[w][gg], sc, ll);
      ov = fmaf(mrg_o[((size_t)w * ng + gg) * D + d], sc, ov);
    }
    const int h = kvh * G + g0 + gg;
    if (a.splits == 1) {
      st_dt(a.out, a.out_dt, ((size_t)t * a.Hq + h) * D + d, ll > 0.f ? ov / ll : 0.f);
    } else {
      const size_t pi = ((size_t)r * a.Hq + h) * a.splits + split;
      a.part_o[pi * D + d] = ov;
      if (d == 0) {                                             // the merge kernel works in natural-log units
        a.part_ml[pi * 2] = mm == -INFINITY ? -1e30f : mms * 0.6931471805599453f;
        a.part_ml[pi * 2 + 1] = ll;
      }
    }
  }
  if (a.splits > 1 && a.split_count) merge_when_last(a, r, t, kvh * G + g0, ng, D);
}

// Combines the splits of one (row, head) in split order.
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ rows, void* __restrict__ out, int out_dt,
                                              int Hq, int D, int splits) {
  const int r = blockIdx.x, h = blockIdx.y;
  const int t = rows ? rows[r] : r;
  const size_t pi = ((size_t)r * Hq + h) * splits;
  grid_dep_wait();
  grid_dep_launch();
  float mm = -1e30f;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(pi + s) * 2]);
  float ll = 0.f;
  for (int s = 0; s < splits; ++s) ll = fmaf(part_ml[(pi + s) * 2 + 1], __expf(part_ml[(pi + s) * 2] - mm), ll);
  const float inv = ll > 0.f ? 1.f / ll : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) o = fmaf(part_o[(pi + s) * D + d], __expf(part_ml[(pi + s) * 2] - mm), o);
    st_dt(out, out_dt, ((size_t)t * Hq + h) * D + d, o * inv);
  }
}

template <typename TC, int CPL, int GB>
int launch_decode_g(const DecArgs& a, int R, int G, size_t smem, cudaStream_t s) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<TC, CPL, GB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  dim3 grid(R, a.Hkv * ((G + GB - 1) / GB), a.splits);
  NV_RETURN_IF(launch_dep(attention_decode_kernel<TC, CPL, GB>, grid, dim3((WARPS + 1) * 32), smem, s, a));
  NV_RETURN_LAST();
}

template <typename TC, int CPL>
int launch_decode(const DecArgs& a, int R, int G, size_t smem, cudaStream_t s) {
  return G == 1 ? launch_decode_g<TC, CPL, 1>(a, R, G, smem, s) : launch_decode_g<TC, CPL, 4>(a, R, G, smem, s);
}

template <int D>
int launch_decode_tc(DecArgs a, int R, const void* kc, const void* vc, int num_pages, float scale, cudaStream_t s) {
  const int G = a.Hq / a.Hkv;
  CUtensorMap tm_k, tm_v;
  const long long rows = (long long)num_pages * a.Hkv * a.page;
  int rc = nv_tensor_map_bf16(kc, rows, D, D, a.page, &tm_k);
  if (rc) return rc;
  rc = nv_tensor_map_bf16(vc, rows, D, D, a.page, &tm_v);
  if (rc) return rc;
  a.scale = scale * 1.4426950408889634f;            // the kernel works in log2 units
  const size_t ring = (size_t)a.stages * 2 * a.page * D * 2;
  const size_t merge = (size_t)WARPS * TC_ROWS * D * sizeof(float);
  const size_t smem = (ring > merge ? ring : merge) + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         160 * 1024);
    if (e != cudaSuccess) return (int)e;
    // three CTAs with a 64 KB ring each need nearly all of a multiprocessor's shared memory
    e = cudaFuncSetAttribute(attention_decode_tc_kernel<D>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  dim3 grid(R, a.Hkv * ((G + TC_ROWS - 1) / TC_ROWS), a.splits);
  NV_RETURN_IF(launch_dep(attention_decode_tc_kernel<D>, grid, dim3((WARPS + 1) * 32), smem, s, tm_k, tm_v, a));
  NV_RETURN_LAST();
}

// Stages of the page ring for a page of `page` keys of `D` elements of `esize` bytes: as many as fit in
// 64 KB (two CTAs per SM and more), at least 2 within 160 KB, else 0 (refused).
int decode_stages(int page, int D, int esize) {
  const long long stage = 2LL * page * D * esize;
  long long s = (64 * 1024) / stage;
  if (s >= 2) return (int)(s > MAX_STAGES ? MAX_STAGES : s);
  return 2 * stage <= 160 * 1024 ? 2 : 0;
}

}  // namespace

// Floats of scratch for `rows` rows: partial outputs and (max, sum) pairs of every split.
NV_API long long nv_attention_decode_scratch_floats(int rows, int Hq, int D, int splits) {
  return splits <= 1 ? 0 : (long long)rows * Hq * splits * (D + 2);
}

// Whether the kernel takes this page geometry (its ring needs two pages of keys and values in shared memory).
NV_API int nv_attention_decode_usable(int D, int page, int cache_dt) {
  if (D <= 0 || D > 256 || D % 8 || page % 16) return 0;
  return decode_stages(page, D, cache_dt == NV_DT_BF16 ? 2 : 4) > 0;
}

// Number of splits for this many rows.  Blocks are short and all alike, so what counts is how full the last
// wave of resident blocks is: the split count whose blocks fill whole waves best wins, with a small price per
// split for its start-up and the merge.  Three blocks of the kernel live on a multiprocessor.
NV_API int nv_attention_decode_splits(int rows, int Hq, int Hkv, int max_context, int num_sms) {
  const int G = Hq / Hkv;
  const long long slots = 3LL * num_sms;
  const long long blocks = (long long)rows * Hkv * ((G + 15) / 16);
  int most = (max_context + 255) / 256;          // at least 256 keys per split
  if (most > 32) most = 32;
  int best = 1;
  double best_score = -1.0;
  for (int s = 1; s <= most; ++s) {
    const long long ctas = blocks * s;
    const long long waves = (ctas + slots - 1) / slots;
    const double score = (double)ctas / ((double)waves * (double)slots) - 0.01 * s;
    if (score > best_score + 1e-9) { best_score = score; best = s; }
  }
  return best;
}

// The kernel is launched as a programmatic dependent of the kernel before it on the stream and reads the index
// arrays, the block table and every page but each row's newest one before that kernel has ended: the kernel
// directly before it may write only the query rows and the newest page of each row (the engine's rotary kernel
// over single rows does exactly that).
NV_API int nv_attention_decode(const void* qkv, int q_dt, int q_stride, const void* kc, const void* vc, int cache_dt,
                               const int* block_table, int max_blocks, const int* row_entry, const int* positions,
                               const int* rows, int R, float scale, int window, void* out, int out_dt, int Hq,
                               int Hkv, int D, int page, int num_pages, int splits, float* scratch, int* err,
                               int* split_count, int split_count_len, cudaStream_t stream) {
  if (!dt_ok(q_dt) || !dt_ok(cache_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (D <= 0 || D > 256 || D % 8 || Hkv <= 0 || Hq % Hkv || page % 16) return NV_ERR_UNSUPPORTED;
  const int esize = cache_dt == NV_DT_BF16 ? 2 : 4;
  const int stages = decode_stages(page, D, esize);
  if (stages == 0) return NV_ERR_UNSUPPORTED;          // a page of this size does not fit the ring twice
  if (((uintptr_t)kc & 15) || ((uintptr_t)vc & 15)) return NV_ERR_UNSUPPORTED;
  if (R == 0) return NV_OK;
  if (splits < 1) splits = 1;
  if (splits > 1 && !scratch) return NV_ERR_BAD_SIZE;
  DecArgs a;
  a.qkv = qkv; a.kc = kc; a.vc = vc; a.block_table = block_table; a.row_entry = row_entry; a.positions = positions;
  a.rows = rows; a.out = out; a.scale = scale; a.q_dt = q_dt; a.out_dt = out_dt; a.q_stride = q_stride;
  a.max_blocks = max_blocks; a.window = window; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.page = page; a.splits = splits;
  a.part_o = scratch;
  a.part_ml = scratch ? scratch + (size_t)R * Hq * splits * D : nullptr;
  a.err = err;
  // `split_count`: zeros (R * Hq of them are enough), kept zero from launch to launch by the kernel: the splits are
  // then added up by the block that finishes last instead of by a second kernel.  For a few rows only: with many,
  // the last blocks' sums lengthen the kernel's tail by more than the second kernel's launch costs (measured per
  // decode step: batch 1 507 -> 511 tokens/s, batch 8 2,209 -> 2,212, batch 64 6,252 -> 6,192).
  a.split_count = (split_count && (long long)R * Hq <= split_count_len && R * Hq <= 256) ? split_count : nullptr;
  a.stages = stages;
  const size_t smem = (size_t)stages * 2 * page * D * esize;
  const int G = Hq / Hkv;
  int rc;
  // The tensor-core form gives every stage of the ring to one warp (stage s to warp s % 4), so that the waits
  // of a warp on a barrier are for consecutive uses of it; that needs a ring of a multiple of four stages.
  // A ring of up to 64 KB: with pages of 16 keys of 128 elements that is eight stages, two per warp, so that a warp's
  // next page is on its way while it works on one (with one stage per warp a warp sat out the whole memory latency
  // between two pages), and three CTAs of 76 KB still share a multiprocessor.  Deeper rings lose CTAs and time.
  int tc_stages = stages / WARPS * WARPS;
  if (cache_dt == NV_DT_BF16 && D % 64 == 0 && page <= 256 && num_pages > 0 && tc_stages >= WARPS) {
    a.stages = tc_stages;
    // tensor-core form (a page of keys per warp); its blocks take up to 16 query heads of a kv head
    rc = D == 64 ? launch_decode_tc<64>(a, R, kc, vc, num_pages, scale, stream)
       : D == 128 ? launch_decode_tc<128>(a, R, kc, vc, num_pages, scale, stream)
       : D == 192 ? launch_decode_tc<192>(a, R, kc, vc, num_pages, scale, stream)
                  : launch_decode_tc<256>(a, R, kc, vc, num_pages, scale, stream);
  } else if (cache_dt == NV_DT_BF16) {
    rc = D <= 64 ? launch_decode<bf16, 1>(a, R, G, smem, stream)
                 : (D <= 128 ? launch_decode<bf16, 2>(a, R, G, smem, stream)
                             : launch_decode<bf16, 4>(a, R, G, smem, stream));
  } else {
    rc = D <= 64 ? launch_decode<float, 1>(a, R, G, smem, stream)
                 : (D <= 128 ? launch_decode<float, 2>(a, R, G, smem, stream)
                             : launch_decode<float, 4>(a, R, G, smem, stream));
  }
  if (rc) return rc;
  if (splits > 1 && !a.split_count) {
    dim3 grid(R, Hq);
    NV_RETURN_IF(launch_dep(attention_decode_merge_kernel, grid, dim3(128), 0, stream, (const float*)a.part_o,
                            (const float*)a.part_ml, rows, out, out_dt, Hq, D, splits));
  }
  NV_RETURN_LAST();
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (declared and described in no_alloc.h).
#include "no_alloc.h"

namespace {

// Partial results of the key splits.  In host code this name is only a stand-in for the symbol, not
// a device address: the address is looked up once per device below and that pointer goes to the kernel.
static __device__ __align__(256) float g_noalloc_scratch[NV_NOALLOC_SCRATCH_FLOATS];
// Set by the kernel if it gave up waiting for a page copy or met a missing page; read by
// nv_attention_decode_noalloc_status.
static __device__ int g_noalloc_err;

constexpr int MAX_DEVICES = 64;
float* g_noalloc_ptr[MAX_DEVICES] = {};   // device address of the array, per device, once looked up
int* g_noalloc_err_ptr[MAX_DEVICES] = {};

}  // namespace

NV_API int nv_attention_decode_noalloc_max_rows(int Hq, int D, int splits) {
  if (Hq <= 0 || D <= 0 || D > 256 || D % 8) return 0;
  if (splits <= 1) return 0x7fffffff;      // one split writes its result directly and needs no scratch
  return (int)((long long)NV_NOALLOC_SCRATCH_FLOATS / ((long long)Hq * splits * (D + 2)));
}

NV_API int nv_attention_decode_noalloc(const void* qkv, int q_dt, int q_stride, const void* kc, const void* vc,
                                       int cache_dt, const int* block_table, int max_blocks, const int* row_entry,
                                       const int* positions, const int* rows, int R, float scale, int window,
                                       void* out, int out_dt, int Hq, int Hkv, int D, int page, int num_pages,
                                       int splits, cudaStream_t stream) {
  if (splits < 1) splits = 1;
  // sizes that nv_attention_decode refuses are refused here first, so that the size test below sees sane numbers
  if (!dt_ok(q_dt) || !dt_ok(cache_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (R < 0 || splits > 1024) return NV_ERR_BAD_SIZE;
  if (D <= 0 || D > 256 || D % 8 || Hkv <= 0 || Hq <= 0 || Hq % Hkv || page <= 0 || page % 16) return NV_ERR_UNSUPPORTED;
  if (nv_attention_decode_scratch_floats(R, Hq, D, splits) > (long long)NV_NOALLOC_SCRATCH_FLOATS)
    return NV_ERR_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return NV_ERR_UNSUPPORTED;
  if (!g_noalloc_ptr[dev]) {               // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    int* q = nullptr;
    e = cudaGetSymbolAddress((void**)&q, g_noalloc_err);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_err_ptr[dev] = q;
    g_noalloc_ptr[dev] = p;
  }
  return nv_attention_decode(qkv, q_dt, q_stride, kc, vc, cache_dt, block_table, max_blocks, row_entry, positions,
                             rows, R, scale, window, out, out_dt, Hq, Hkv, D, page, num_pages, splits,
                             g_noalloc_ptr[dev], g_noalloc_err_ptr[dev], nullptr, 0, stream);
}

NV_API int nv_attention_decode_noalloc_status(void) {
  int dev = -1, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES || !g_noalloc_err_ptr[dev]) return 0;
  cudaError_t e = cudaMemcpy(&v, g_noalloc_err_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? v : (int)e;
}
