// Decode attention: one query row per request against its paged keys and values, split over the
// keys so that a few requests still fill the GPU.
//
// grid = (rows, kv heads x head groups, splits).  A block streams its share of one request's keys and
// values once, for up to GB query heads that share the kv head.  Inside a warp, groups of 8 lanes
// own one key each (4 keys per warp per pass); a lane holds 8-element chunks of the head
// dimension, so a key's row is read with 16-byte loads and the dot product needs three shuffles.
// Every (warp, lane group) keeps its own running max / sum / output (online softmax, float32) and
// the partial results are merged at the end: lane groups by shuffles, warps through shared memory,
// splits by a second small kernel.  The merge order is fixed, so a row's result does not depend
// on the batch.  Keys of row t at position p: [max(0, p + 1 - window), p].
//
// Reference twin: nv_paged_attention_plain.  (The reference's kernel: src/hip_ops.hip:473-551.)
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
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
  float scale;
  int q_dt, out_dt, q_stride, max_blocks, window, Hq, Hkv, D, page, splits;
};

// CPL: chunks of 8 elements per lane (D <= 64 * CPL); GB: query heads per block.
template <typename TC, int CPL, int GB>
__global__ void __launch_bounds__(WARPS * 32) attention_decode_kernel(DecArgs a) {
  __shared__ float q_s[GB][256];
  __shared__ float mrg_o[WARPS][GB][256];
  __shared__ float mrg_m[WARPS][GB], mrg_l[WARPS][GB];

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
  // this split's keys: a multiple of KEYS_PER_PASS per split, counted from lo
  const int per = ((n - lo + a.splits - 1) / a.splits + KEYS_PER_PASS - 1) / KEYS_PER_PASS * KEYS_PER_PASS;
  const int k_begin = lo + split * per;
  const int k_end = min(n, k_begin + per);

  for (int i = threadIdx.x; i < ng * D; i += WARPS * 32) {
    int g = i / D, d = i % D;
    q_s[g][d] = ld_dt(a.qkv, a.q_dt, (size_t)t * a.q_stride + (size_t)(kvh * G + g0 + g) * D + d) * a.scale;
  }
  __syncthreads();

  const int* bt = a.block_table + (size_t)a.row_entry[t] * a.max_blocks;
  const TC* kc = (const TC*)a.kc;
  const TC* vc = (const TC*)a.vc;

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

  for (int j0 = k_begin + warp * KEYS_PER_WARP; j0 < k_end; j0 += KEYS_PER_PASS) {
    const int j = j0 + sub;
    const bool live = j < k_end;
    size_t base = 0;
    if (live) {
      const int blk = bt[j / a.page];
      base = (((size_t)blk * a.Hkv + kvh) * a.page + j % a.page) * D;
    }
    float kf[CPL][8], vf[CPL][8];
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const int ch = li + c * LPK;
      if (live && ch < chunks) {
        Chunk<TC>::load(kc + base + ch * 8, kf[c]);
        Chunk<TC>::load(vc + base + ch * 8, vf[c]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) kf[c][e] = vf[c][e] = 0.f;
      }
    }
#pragma unroll
    for (int g = 0; g < GB; ++g) {
      if (g >= ng) break;
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = li + c * LPK;
        if (ch < chunks) {
          const float4 qa = *(const float4*)&q_s[g][ch * 8], qb = *(const float4*)&q_s[g][ch * 8 + 4];
          s = fmaf(qa.x, kf[c][0], s); s = fmaf(qa.y, kf[c][1], s); s = fmaf(qa.z, kf[c][2], s);
          s = fmaf(qa.w, kf[c][3], s); s = fmaf(qb.x, kf[c][4], s); s = fmaf(qb.y, kf[c][5], s);
          s = fmaf(qb.z, kf[c][6], s); s = fmaf(qb.w, kf[c][7], s);
        }
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (live) {
        const float m_new = fmaxf(m[g], s);
        const float alpha = __expf(m[g] - m_new), p = __expf(s - m_new);
        l[g] = l[g] * alpha + p;
        m[g] = m_new;
#pragma unroll
        for (int c = 0; c < CPL; ++c)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][c][e] = fmaf(p, vf[c][e], acc[g][c][e] * alpha);
      }
    }
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
  __syncthreads();
  // merge the warps and write this split's result
  for (int i = threadIdx.x; i < ng * D; i += WARPS * 32) {
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

template <typename TC, int CPL>
int launch_decode(const DecArgs& a, int R, int G, cudaStream_t s) {
  if (G == 1) {
    dim3 grid(R, a.Hkv, a.splits);
    attention_decode_kernel<TC, CPL, 1><<<grid, WARPS * 32, 0, s>>>(a);
  } else {
    dim3 grid(R, a.Hkv * ((G + 3) / 4), a.splits);
    attention_decode_kernel<TC, CPL, 4><<<grid, WARPS * 32, 0, s>>>(a);
  }
  NV_RETURN_LAST();
}

}  // namespace

// Floats of scratch for `rows` rows: partial outputs and (max, sum) pairs of every split.
NV_API long long nv_attention_decode_scratch_floats(int rows, int Hq, int D, int splits) {
  return splits <= 1 ? 0 : (long long)rows * Hq * splits * (D + 2);
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
                               int Hkv, int D, int page, int splits, float* scratch, cudaStream_t stream) {
  if (!dt_ok(q_dt) || !dt_ok(cache_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (D <= 0 || D > 256 || D % 8 || Hkv <= 0 || Hq % Hkv) return NV_ERR_UNSUPPORTED;
  if (R == 0) return NV_OK;
  if (splits < 1) splits = 1;
  if (splits > 1 && !scratch) return NV_ERR_BAD_SIZE;
  DecArgs a;
  a.qkv = qkv; a.kc = kc; a.vc = vc; a.block_table = block_table; a.row_entry = row_entry; a.positions = positions;
  a.rows = rows; a.out = out; a.scale = scale; a.q_dt = q_dt; a.out_dt = out_dt; a.q_stride = q_stride;
  a.max_blocks = max_blocks; a.window = window; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.page = page; a.splits = splits;
  a.part_o = scratch;
  a.part_ml = scratch ? scratch + (size_t)R * Hq * splits * D : nullptr;
  const int G = Hq / Hkv;
  int rc;
  if (cache_dt == NV_DT_BF16) {
    rc = D <= 64 ? launch_decode<bf16, 1>(a, R, G, stream)
                 : (D <= 128 ? launch_decode<bf16, 2>(a, R, G, stream) : launch_decode<bf16, 4>(a, R, G, stream));
  } else {
    rc = D <= 64 ? launch_decode<float, 1>(a, R, G, stream)
                 : (D <= 128 ? launch_decode<float, 2>(a, R, G, stream) : launch_decode<float, 4>(a, R, G, stream));
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

constexpr int MAX_DEVICES = 64;
float* g_noalloc_ptr[MAX_DEVICES] = {};   // device address of the array, per device, once looked up

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
    g_noalloc_ptr[dev] = p;
  }
  return nv_attention_decode(qkv, q_dt, q_stride, kc, vc, cache_dt, block_table, max_blocks, row_entry, positions,
                             rows, R, scale, window, out, out_dt, Hq, Hkv, D, page, splits, g_noalloc_ptr[dev],
                             stream);
}
