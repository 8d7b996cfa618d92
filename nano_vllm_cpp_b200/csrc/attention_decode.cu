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

namespace {

constexpr int WARPS = 4;                // consumer warps; one more warp produces
constexpr int MAX_STAGES = 8;
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
  int* err;
  float scale;
  int q_dt, out_dt, q_stride, max_blocks, window, Hq, Hkv, D, page, splits, stages;
};

// CPL: chunks of 8 elements per lane (D <= 64 * CPL); GB: query heads per block.
template <typename TC, int CPL, int GB>
__global__ void __launch_bounds__((WARPS + 1) * 32) attention_decode_kernel(DecArgs a) {
  extern __shared__ __align__(128) uint8_t dec_smem[];
  __shared__ float q_s[GB][256];
  __shared__ float mrg_o[WARPS][GB][256];
  __shared__ float mrg_m[WARPS][GB], mrg_l[WARPS][GB];
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];

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
  for (int i = threadIdx.x; i < ng * D; i += (WARPS + 1) * 32) {
    int g = i / D, d = i % D;
    q_s[g][d] = ld_dt(a.qkv, a.q_dt, (size_t)t * a.q_stride + (size_t)(kvh * G + g0 + g) * D + d) * a.scale;
  }
  __syncthreads();

  const int* bt = a.block_table + (size_t)a.row_entry[t] * a.max_blocks;

  if (warp == WARPS) {
    // ---------------------------------------------------------------- producer: one lane issues the copies
    if (lane == 0) {
      for (int i = 0; i < n_pages; ++i) {
        const int s = i % a.stages;
        mbar_wait(&empty_bar[s], ((i / a.stages) & 1) ^ 1, a.err, 0x7101);
        const int blk = bt[pb + i];
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
            if (ch < chunks) {
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
            const float m_new = fmaxf(m[g], sc);
            const float alpha = __expf(m[g] - m_new), p = __expf(sc - m_new);
            l[g] = l[g] * alpha + p;
            m[g] = m_new;
#pragma unroll
            for (int c = 0; c < CPL; ++c)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[g][c][e] = fmaf(p, vf[c][e], acc[g][c][e] * alpha);
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
}

// Combines the splits of one (row, head) in split order.
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ rows, void* __restrict__ out, int out_dt,
                                              int Hq, int D, int splits) {
  const int r = blockIdx.x, h = blockIdx.y;
  const int t = rows ? rows[r] : r;
  const size_t pi = ((size_t)r * Hq + h) * splits;
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
  attention_decode_kernel<TC, CPL, GB><<<grid, (WARPS + 1) * 32, smem, s>>>(a);
  NV_RETURN_LAST();
}

template <typename TC, int CPL>
int launch_decode(const DecArgs& a, int R, int G, size_t smem, cudaStream_t s) {
  return G == 1 ? launch_decode_g<TC, CPL, 1>(a, R, G, smem, s) : launch_decode_g<TC, CPL, 4>(a, R, G, smem, s);
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

// Number of splits that fills `num_sms` multiprocessors a few times over for this many rows.
NV_API int nv_attention_decode_splits(int rows, int Hq, int Hkv, int max_context, int num_sms) {
  int G = Hq / Hkv;
  int blocks = rows * Hkv * (G == 1 ? 1 : (G + 3) / 4);
  int want = (4 * num_sms + blocks - 1) / blocks;
  int most = (max_context + 255) / 256;          // at least 256 keys per split
  int s = want < most ? want : most;
  if (s > 32) s = 32;
  return s < 1 ? 1 : s;
}

NV_API int nv_attention_decode(const void* qkv, int q_dt, int q_stride, const void* kc, const void* vc, int cache_dt,
                               const int* block_table, int max_blocks, const int* row_entry, const int* positions,
                               const int* rows, int R, float scale, int window, void* out, int out_dt, int Hq,
                               int Hkv, int D, int page, int splits, float* scratch, int* err,
                               cudaStream_t stream) {
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
  a.stages = stages;
  const size_t smem = (size_t)stages * 2 * page * D * esize;
  const int G = Hq / Hkv;
  int rc;
  if (cache_dt == NV_DT_BF16) {
    rc = D <= 64 ? launch_decode<bf16, 1>(a, R, G, smem, stream)
                 : (D <= 128 ? launch_decode<bf16, 2>(a, R, G, smem, stream)
                             : launch_decode<bf16, 4>(a, R, G, smem, stream));
  } else {
    rc = D <= 64 ? launch_decode<float, 1>(a, R, G, smem, stream)
                 : (D <= 128 ? launch_decode<float, 2>(a, R, G, smem, stream)
                             : launch_decode<float, 4>(a, R, G, smem, stream));
  }
  if (rc) return rc;
  if (splits > 1) {
    dim3 grid(R, Hq);
    attention_decode_merge_kernel<<<grid, 128, 0, stream>>>(a.part_o, a.part_ml, rows, out, out_dt, Hq, D, splits);
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
  if (Hq <= 0 || D <= 0) return 0;
  if (splits <= 1) return 0x7fffffff;      // one split writes its result directly and needs no scratch
  return (int)((long long)NV_NOALLOC_SCRATCH_FLOATS / ((long long)Hq * splits * (D + 2)));
}

NV_API int nv_attention_decode_noalloc(const void* qkv, int q_dt, int q_stride, const void* kc, const void* vc,
                                       int cache_dt, const int* block_table, int max_blocks, const int* row_entry,
                                       const int* positions, const int* rows, int R, float scale, int window,
                                       void* out, int out_dt, int Hq, int Hkv, int D, int page, int splits,
                                       cudaStream_t stream) {
  if (splits < 1) splits = 1;
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
                             rows, R, scale, window, out, out_dt, Hq, Hkv, D, page, splits, g_noalloc_ptr[dev],
                             g_noalloc_err_ptr[dev], stream);
}

NV_API int nv_attention_decode_noalloc_status(void) {
  int dev = -1, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES || !g_noalloc_err_ptr[dev]) return 0;
  cudaError_t e = cudaMemcpy(&v, g_noalloc_err_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? v : (int)e;
}
