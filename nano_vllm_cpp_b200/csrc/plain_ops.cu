// Plain kernels: one simple, checkable implementation of every op of the model that is not a
// matrix product.  They are the float32 path's kernels, the bfloat16 path's kernels for every
// op that has no faster form yet, and the twins that the fast kernels are tested against.
// Softmax, norms, router probabilities, rotation angles and the residual sum are 32-bit (the
// router's softmax is 64-bit, as in the reference) whatever the storage type is.
#include "common.cuh"
#include "moe_route.cuh"

int g_nv_dependent_launch = 1;

namespace {

// ------------------------------------------------------------------ embedding
// out[t,:] = float(table[ids[t],:])                       (src/hip_ops.hip:553-563)
// A negative id -(r + 1) stands for "the token that the step before this one drew for its row r": it is read
// from `feed`, where that step's sampling kernel left it, so that a step can be launched before the host has
// seen the tokens of the step before.
__global__ void embedding_kernel(const int* __restrict__ ids, const void* __restrict__ table, int dt,
                                 float* __restrict__ out, int H, int V, int* __restrict__ err,
                                 const int* __restrict__ feed) {
  grid_dep_wait();
  grid_dep_launch();
  int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && feed) id = feed[-id - 1];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicExch(err, 1 + t);
    id = 0;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)t * H + i] = ld_dt(table, dt, (size_t)id * H + i);
}

// ---------------------------------------------------------- residual add + RMSNorm
// x += branch (if given); y = x * rsqrt(mean(x^2) + eps) * w     (src/hip_ops.hip:395-417)
// The branch is a float32 matrix, or a mix of rows that has not been summed yet:
//   branch[t,:] = sigmoid(gate_logit[t]) * dense[t,:] + sum_r weight[t,r] * rows[index[t,r],:]
// with the sum over r = 0..R-1 in that order and the dense term added to it afterwards, which is how
// the experts' outputs are combined (src/hip_ops.hip:873-892, 926-934; src/model.cpp:803-811).
// One block per row; a thread keeps its elements in registers between the two passes (rows wider
// than 256 * VEC * NORM_CACHE elements re-read the rest from x).  The sum of squares is taken in
// a fixed order (a thread's elements in order, a warp's shuffle tree, the warps in order), so a
// row's result does not depend on the batch.
constexpr int NORM_THREADS = 256, NORM_CACHE = 4, NORM_MAX_R = 64;

struct NormArgs {
  float* x;
  const float* branch;
  const void* w;
  void* out;
  float* out32;
  const float* rows;
  const int* index;
  const float* weight;
  const float* dense;
  const float* gate_logit;
  long long gate_ld;
  float eps;
  int w_dt, out_dt, H, R;
};

template <int VEC>
struct Chunk { float v[VEC]; };

template <int VEC>
__device__ __forceinline__ Chunk<VEC> ld_chunk(const float* p) {
  Chunk<VEC> c;
  if (VEC == 4) {
    float4 q = *reinterpret_cast<const float4*>(p);
    c.v[0] = q.x; c.v[VEC > 1 ? 1 : 0] = q.y; c.v[VEC > 2 ? 2 : 0] = q.z; c.v[VEC > 3 ? 3 : 0] = q.w;
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) c.v[j] = p[j];
  }
  return c;
}
template <int VEC>
__device__ __forceinline__ void st_chunk(float* p, const Chunk<VEC>& c) {
  if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(c.v[0], c.v[VEC > 1 ? 1 : 0], c.v[VEC > 2 ? 2 : 0], c.v[VEC > 3 ? 3 : 0]);
  else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) p[j] = c.v[j];
  }
}

template <int VEC>
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_kernel(NormArgs a) {
  __shared__ float red[NORM_THREADS / 32];
  __shared__ int s_idx[NORM_MAX_R];
  __shared__ float s_w[NORM_MAX_R];
  const int t = blockIdx.x, tid = threadIdx.x;
  const size_t base = (size_t)t * a.H;
  const int chunks = a.H / VEC;
  grid_dep_wait();
  grid_dep_launch();
  float gate = 1.f;
  if (a.R > 0) {
    if (tid < a.R) {
      s_idx[tid] = a.index[(size_t)t * a.R + tid];
      s_w[tid] = a.weight[(size_t)t * a.R + tid];
    }
    __syncthreads();
  }
  if (a.dense && a.gate_logit) gate = 1.f / (1.f + expf(-a.gate_logit[(size_t)t * a.gate_ld]));
  const bool adds = a.branch || a.R > 0 || a.dense;

  // value of the updated residual stream at chunk c (and its write-back when something was added)
  auto updated = [&](int c) {
    Chunk<VEC> v = ld_chunk<VEC>(a.x + base + (size_t)c * VEC);
    if (a.branch) {
      Chunk<VEC> b = ld_chunk<VEC>(a.branch + base + (size_t)c * VEC);
#pragma unroll
      for (int j = 0; j < VEC; ++j) v.v[j] += b.v[j];
    } else if (a.R > 0 || a.dense) {
      Chunk<VEC> r;
#pragma unroll
      for (int j = 0; j < VEC; ++j) r.v[j] = 0.f;
      // four rows' loads are in flight before the first is used; the sum keeps the order of k
      int k = 0;
      for (; k + 4 <= a.R; k += 4) {
        Chunk<VEC> y[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) y[u] = ld_chunk<VEC>(a.rows + (size_t)s_idx[k + u] * a.H + (size_t)c * VEC);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float wk = s_w[k + u];
#pragma unroll
          for (int j = 0; j < VEC; ++j) r.v[j] = fmaf(wk, y[u].v[j], r.v[j]);
        }
      }
      for (; k < a.R; ++k) {
        Chunk<VEC> y = ld_chunk<VEC>(a.rows + (size_t)s_idx[k] * a.H + (size_t)c * VEC);
        const float wk = s_w[k];
#pragma unroll
        for (int j = 0; j < VEC; ++j) r.v[j] = fmaf(wk, y.v[j], r.v[j]);
      }
      if (a.dense) {
        Chunk<VEC> d = ld_chunk<VEC>(a.dense + base + (size_t)c * VEC);
#pragma unroll
        for (int j = 0; j < VEC; ++j) r.v[j] = d.v[j] * gate + r.v[j];
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) v.v[j] += r.v[j];
    }
    if (adds) st_chunk<VEC>(a.x + base + (size_t)c * VEC, v);
    return v;
  };

  Chunk<VEC> keep[NORM_CACHE];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < NORM_CACHE; ++u) {
    const int c = tid + u * NORM_THREADS;
    if (c < chunks) {
      keep[u] = updated(c);
#pragma unroll
      for (int j = 0; j < VEC; ++j) ss = fmaf(keep[u].v[j], keep[u].v[j], ss);
    }
  }
  for (int c = tid + NORM_CACHE * NORM_THREADS; c < chunks; c += NORM_THREADS) {
    Chunk<VEC> v = updated(c);
#pragma unroll
    for (int j = 0; j < VEC; ++j) ss = fmaf(v.v[j], v.v[j], ss);
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; ++i) total += red[i];
  const float inv = rsqrtf(total / (float)a.H + a.eps);

  auto emit = [&](int c, const Chunk<VEC>& v) {
    Chunk<VEC> y;
#pragma unroll
    for (int j = 0; j < VEC; ++j) y.v[j] = v.v[j] * inv * ld_dt(a.w, a.w_dt, (size_t)c * VEC + j);
    const size_t o = base + (size_t)c * VEC;
    if (a.out_dt == NV_DT_F32) st_chunk<VEC>((float*)a.out + o, y);
    else if (VEC == 4) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(y.v[0], y.v[VEC > 1 ? 1 : 0]);
      __nv_bfloat162 hi = __floats2bfloat162_rn(y.v[VEC > 2 ? 2 : 0], y.v[VEC > 3 ? 3 : 0]);
      uint2 q;
      q.x = *reinterpret_cast<uint32_t*>(&lo);
      q.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>((bf16*)a.out + o) = q;
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) ((bf16*)a.out)[o + j] = __float2bfloat16_rn(y.v[j]);
    }
    if (a.out32) st_chunk<VEC>(a.out32 + o, y);
  };
#pragma unroll
  for (int u = 0; u < NORM_CACHE; ++u) {
    const int c = tid + u * NORM_THREADS;
    if (c < chunks) emit(c, keep[u]);
  }
  for (int c = tid + NORM_CACHE * NORM_THREADS; c < chunks; c += NORM_THREADS)
    emit(c, ld_chunk<VEC>(a.x + base + (size_t)c * VEC));
}

// ------------------------------------------------ rotary position encoding + cache write
// NeoX pairing (d, d + R/2) over the first R = rotary_dim elements of each head:
//   ang = float(pos) * inv_freq[d];  o[d] = x[d] cos - x[d+R/2] sin;  o[d+R/2] = x[d+R/2] cos + x[d] sin
// (src/hip_ops.hip:431-450).  q is rotated in place; k is rotated and written to its page; v is
// copied to its page (src/hip_ops.hip:452-466).  
// Cache layout: [page][kv head][slot in page][D].
// The position that turns pair d need not be the row's place in its sequence: rot_pos is [T][axes] (the row's
// coordinates, e.g. a place in the text and a row and a column of an image) and pair_axis[d] says which of them pair
// d is turned by (nullptr: the first).  The cache slot always comes from `positions`, the place in the sequence.
// One block per (row, group of `hpb` heads in the order q.., k.., v..): the angles are taken once per block.
__global__ void __launch_bounds__(256) rope_store_kernel(void* __restrict__ qkv, int dt, const int* __restrict__ positions,
                                  const int* __restrict__ rot_pos, int axes, const int* __restrict__ pair_axis,
                                  const float* __restrict__ inv_freq, int rotary_dim,
                                  void* __restrict__ kc, void* __restrict__ vc, int cache_dt,
                                  const int* __restrict__ block_table, int max_blocks,
                                  const int* __restrict__ row_entry, int Hq, int Hkv, int D, int page,
                                  int write_kv, int hpb, int* __restrict__ err) {
  __shared__ float cs[128], sn[128];
  grid_dep_wait();
  grid_dep_launch();
  const int t = blockIdx.x;
  const int h_begin = blockIdx.y * hpb;
  const int h_end = min(Hq + 2 * Hkv, h_begin + hpb);
  if (!write_kv && h_begin >= Hq) return;
  const int width = (Hq + 2 * Hkv) * D;
  const int pos = positions[t];
  const int half = rotary_dim / 2;
  if (h_begin < Hq + Hkv)
    for (int f = threadIdx.x; f < half; f += blockDim.x) {
      const int pf = rot_pos ? rot_pos[(size_t)t * axes + (pair_axis ? pair_axis[f] : 0)] : pos;
      float ang = (float)pf * inv_freq[f];
      cs[f] = cosf(ang);
      sn[f] = sinf(ang);
    }
  int blk = 0;
  if (h_end > Hq && write_kv) {
    blk = block_table[(size_t)row_entry[t] * max_blocks + pos / page];
    if (blk < 0) {
      if (threadIdx.x == 0) atomicExch(err, 1 + t);
      write_kv = 0;
    }
  }
  __syncthreads();
  const size_t row = (size_t)t * width;
  const size_t slot = (size_t)(pos % page);
  // rotated heads (q, and k when the cache is written): the block's (head, pair) items flattened; a thread
  // owns whole pairs (f, f + half), so rotating q in place needs no barrier
  const int rot_end = min(h_end, write_kv ? Hq + Hkv : Hq);
  const bool packed = dt == NV_DT_BF16 && cache_dt == NV_DT_BF16 && half % 2 == 0 && D % 8 == 0;
  if (packed && half % 8 == 0) {
    // bfloat16 buffers, eight pairs per thread: 16-byte loads and stores
    const int hp = half / 8;
    bf16* qb = (bf16*)qkv;
    bf16* kb = (bf16*)kc;
    for (int i = threadIdx.x; i < (rot_end - h_begin) * hp; i += blockDim.x) {
      const int h = h_begin + i / hp, f = (i % hp) * 8;
      const size_t base = row + (size_t)h * D;
      const uint4 r1 = *(const uint4*)(qb + base + f), r2 = *(const uint4*)(qb + base + f + half);
      const __nv_bfloat162* p1 = (const __nv_bfloat162*)&r1;
      const __nv_bfloat162* p2 = (const __nv_bfloat162*)&r2;
      uint4 w1, w2;
      __nv_bfloat162* o1 = (__nv_bfloat162*)&w1;
      __nv_bfloat162* o2 = (__nv_bfloat162*)&w2;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x1 = __bfloat1622float2(p1[j]), x2 = __bfloat1622float2(p2[j]);
        const float c0 = cs[f + 2 * j], c1 = cs[f + 2 * j + 1], s0 = sn[f + 2 * j], s1 = sn[f + 2 * j + 1];
        o1[j] = __floats2bfloat162_rn(x1.x * c0 - x2.x * s0, x1.y * c1 - x2.y * s1);
        o2[j] = __floats2bfloat162_rn(x2.x * c0 + x1.x * s0, x2.y * c1 + x1.y * s1);
      }
      bf16* dst = h < Hq ? qb + base : kb + (((size_t)blk * Hkv + (h - Hq)) * page + slot) * D;
      *(uint4*)(dst + f) = w1;
      *(uint4*)(dst + f + half) = w2;
    }
  } else if (packed) {
    // bfloat16 buffers: two pairs per thread, 4-byte loads and stores
    const int hp = half / 2;
    bf16* qb = (bf16*)qkv;
    bf16* kb = (bf16*)kc;
    for (int i = threadIdx.x; i < (rot_end - h_begin) * hp; i += blockDim.x) {
      const int h = h_begin + i / hp, f = (i % hp) * 2;
      const size_t base = row + (size_t)h * D;
      const float2 x1 = __bfloat1622float2(*(const __nv_bfloat162*)(qb + base + f));
      const float2 x2 = __bfloat1622float2(*(const __nv_bfloat162*)(qb + base + f + half));
      const float c0 = cs[f], c1 = cs[f + 1], s0 = sn[f], s1 = sn[f + 1];
      const __nv_bfloat162 o1 = __floats2bfloat162_rn(x1.x * c0 - x2.x * s0, x1.y * c1 - x2.y * s1);
      const __nv_bfloat162 o2 = __floats2bfloat162_rn(x2.x * c0 + x1.x * s0, x2.y * c1 + x1.y * s1);
      bf16* dst = h < Hq ? qb + base : kb + (((size_t)blk * Hkv + (h - Hq)) * page + slot) * D;
      *(__nv_bfloat162*)(dst + f) = o1;
      *(__nv_bfloat162*)(dst + f + half) = o2;
    }
  } else if (half > 0)
    for (int i = threadIdx.x; i < (rot_end - h_begin) * half; i += blockDim.x) {
      const int h = h_begin + i / half, f = i % half;
      const size_t base = row + (size_t)h * D;
      const float x1 = ld_dt(qkv, dt, base + f), x2 = ld_dt(qkv, dt, base + f + half);
      const float o1 = x1 * cs[f] - x2 * sn[f], o2 = x2 * cs[f] + x1 * sn[f];
      if (h < Hq) {
        st_dt(qkv, dt, base + f, o1);
        st_dt(qkv, dt, base + f + half, o2);
      } else {
        const size_t cbase = (((size_t)blk * Hkv + (h - Hq)) * page + slot) * D;
        st_dt(kc, cache_dt, cbase + f, o1);
        st_dt(kc, cache_dt, cbase + f + half, o2);
      }
    }
  if (!write_kv) return;
  // what is copied as it is: the part of k beyond the rotated dimensions, and v
  const int tail = D - rotary_dim;
  const int k_lo = max(h_begin, Hq), k_hi = min(h_end, Hq + Hkv);
  for (int i = threadIdx.x; i < (k_hi - k_lo) * tail; i += blockDim.x) {
    const int h = k_lo + i / tail, d = rotary_dim + i % tail;
    const size_t cbase = (((size_t)blk * Hkv + (h - Hq)) * page + slot) * D;
    st_dt(kc, cache_dt, cbase + d, ld_dt(qkv, dt, row + (size_t)h * D + d));
  }
  const int v_lo = max(h_begin, Hq + Hkv);
  if (packed) {                                    // 16-byte copies of v
    const int cpd = D / 8;
    for (int i = threadIdx.x; i < (h_end - v_lo) * cpd; i += blockDim.x) {
      const int h = v_lo + i / cpd, c = i % cpd;
      const size_t cbase = (((size_t)blk * Hkv + (h - Hq - Hkv)) * page + slot) * D;
      *((uint4*)((bf16*)vc + cbase) + c) = *((const uint4*)((const bf16*)qkv + row + (size_t)h * D) + c);
    }
    return;
  }
  for (int i = threadIdx.x; i < (h_end - v_lo) * D; i += blockDim.x) {
    const int h = v_lo + i / D, d = i % D;
    const size_t cbase = (((size_t)blk * Hkv + (h - Hq - Hkv)) * page + slot) * D;
    st_dt(vc, cache_dt, cbase + d, ld_dt(qkv, dt, row + (size_t)h * D + d));
  }
}

// --------------------------------------------------------------- paged attention (plain)
// One block per (row, query head).  Row t with position p sees keys [lo, p] where
// lo = max(0, p + 1 - window) (window 0 = all).  Keys are taken in chunks of 128 from lo
// upward with an online softmax; everything is fp32 (src/hip_ops.hip:473-551).
constexpr int ATT_THREADS = 128;
__global__ void __launch_bounds__(ATT_THREADS) paged_attention_plain_kernel(
    const void* __restrict__ qkv, int dt, int q_stride, const void* __restrict__ kc, const void* __restrict__ vc,
    int cache_dt, const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_entry,
    const int* __restrict__ positions, float scale, int window, void* __restrict__ out, int out_dt,
    int Hq, int Hkv, int D, int page) {
  __shared__ float q[256];
  __shared__ float p[ATT_THREADS];
  __shared__ int pslot[ATT_THREADS];   // element offset / D of each key of the chunk
  __shared__ float red[ATT_THREADS];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kvh = h / (Hq / Hkv);
  const int n = positions[t] + 1;
  const int lo = window > 0 ? max(0, n - window) : 0;
  const int* bt = block_table + (size_t)row_entry[t] * max_blocks;
  for (int d = tid; d < D; d += ATT_THREADS) q[d] = ld_dt(qkv, dt, (size_t)t * q_stride + (size_t)h * D + d);
  __syncthreads();
  float m = -1e30f, l = 0.f;
  float o0 = 0.f, o1 = 0.f;  // this thread's output elements d = tid and tid + 128
  for (int c0 = lo; c0 < n; c0 += ATT_THREADS) {
    const int j = c0 + tid;
    float s = -1e30f;
    if (j < n) {
      int blk = bt[j / page];
      size_t slot = ((size_t)blk * Hkv + kvh) * page + j % page;
      pslot[tid] = (int)slot;
      float acc = 0.f;
      for (int d = 0; d < D; ++d) acc = fmaf(q[d], ld_dt(kc, cache_dt, slot * D + d), acc);
      s = acc * scale;
    }
    red[tid] = s;
    __syncthreads();
    for (int st = ATT_THREADS / 2; st > 0; st >>= 1) {
      if (tid < st) red[tid] = fmaxf(red[tid], red[tid + st]);
      __syncthreads();
    }
    const float m_new = fmaxf(m, red[0]);
    __syncthreads();
    const float e = j < n ? expf(s - m_new) : 0.f;
    p[tid] = e;
    red[tid] = e;
    __syncthreads();
    for (int st = ATT_THREADS / 2; st > 0; st >>= 1) {
      if (tid < st) red[tid] += red[tid + st];
      __syncthreads();
    }
    const float alpha = expf(m - m_new);
    l = l * alpha + red[0];
    m = m_new;
    const int cnt = min(ATT_THREADS, n - c0);
    o0 *= alpha;
    o1 *= alpha;
    if (tid < D) {
      for (int i = 0; i < cnt; ++i) o0 = fmaf(p[i], ld_dt(vc, cache_dt, (size_t)pslot[i] * D + tid), o0);
    }
    if (tid + ATT_THREADS < D) {
      for (int i = 0; i < cnt; ++i)
        o1 = fmaf(p[i], ld_dt(vc, cache_dt, (size_t)pslot[i] * D + tid + ATT_THREADS), o1);
    }
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const size_t ob = (size_t)t * Hq * D + (size_t)h * D;
  if (tid < D) st_dt(out, out_dt, ob + tid, o0 * inv);
  if (tid + ATT_THREADS < D) st_dt(out, out_dt, ob + tid + ATT_THREADS, o1 * inv);
}

// ----------------------------------------------------------------------- router, expert permutation
// (the work is in moe_route.cuh)
__global__ void router_topk_kernel(const float* __restrict__ logits, long long ld, int T, int E, int K, int renorm,
                                   int* __restrict__ idx, float* __restrict__ score, int C,
                                   const float* __restrict__ gate_logit, long long gate_ld) {
  extern __shared__ double sm[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t = blockIdx.x * (blockDim.x / 32) + warp;
  if (t >= T) return;
  route_row(logits + (size_t)t * ld, E, K, renorm, sm + (size_t)warp * E, lane, idx + (size_t)t * (K + C),
            score + (size_t)t * (K + C), C, C ? gate_logit + (size_t)t * gate_ld : nullptr);
}

__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ idx, int TK, int K, int E,
                                                         int tile_m, int* __restrict__ counts,
                                                         int* __restrict__ offsets,
                                                         int* __restrict__ sorted_token, int* __restrict__ pair_pos,
                                                         int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                                         int* __restrict__ tile_rows, int* __restrict__ num_tiles,
                                                         int* __restrict__ err, int tile_m2,
                                                         int* __restrict__ t2_expert, int* __restrict__ t2_row0,
                                                         int* __restrict__ t2_rows, int* __restrict__ num_tiles2,
                                                         int n_spread, int n_static, int* __restrict__ zero,
                                                         int n_zero) {
  extern __shared__ int al_s[];
  if ((int)threadIdx.x < n_zero) zero[threadIdx.x] = 0;      // (tile counters of the products that follow)
  align_block(idx, TK, K, E, tile_m, counts, offsets, sorted_token, pair_pos, tile_expert, tile_row0, tile_rows,
              num_tiles, err, al_s, tile_m2, t2_expert, t2_row0, t2_rows, num_tiles2, n_static, n_spread);
}

// ------------------------------------------------------------------------ combine
// out[t,:] = sigmoid(gate_logit[t]) * shared[t,:] + sum_k score[t,k] * y[pair_pos[t*K+k],:]
// with the routed sum taken for k = 0..K-1 in that order, then added to the shared term
// (src/hip_ops.hip:873-892, 926-934; src/model.cpp:803-811).
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_pos,
                                   const float* __restrict__ score, const float* __restrict__ shared,
                                   const float* __restrict__ gate_logit, long long gate_ld,
                                   float* __restrict__ out, int K, int H) {
  const int t = blockIdx.x;
  float g = 1.f;
  if (gate_logit) g = 1.f / (1.f + expf(-gate_logit[(size_t)t * gate_ld]));
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
    float r = 0.f;
    for (int k = 0; k < K; ++k) {
      float w = score[(size_t)t * K + k];
      r = fmaf(w, y[(size_t)pair_pos[(size_t)t * K + k] * H + i], r);
    }
    float sh = shared ? shared[(size_t)t * H + i] * g : 0.f;
    out[(size_t)t * H + i] = sh + r;
  }
}

// ------------------------------------------------------------------------ silu_mul
// out[r,c] = silu(gu[r,c]) * gu[r,I+c]   (src/hip_ops.hip:419-429) — for callers whose product
// could not fuse it.
__global__ void silu_mul_kernel(const void* __restrict__ gu, int dt, void* __restrict__ out, int out_dt,
                                long long rows, int I) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * I) return;
  long long r = i / I;
  int c = (int)(i % I);
  st_dt(out, out_dt, i, silu_mul(ld_dt(gu, dt, r * 2 * I + c), ld_dt(gu, dt, r * 2 * I + I + c)));
}

// ------------------------------------------------------------------------ gather rows
__global__ void gather_rows_kernel(const void* __restrict__ src, int dt, const int* __restrict__ rows,
                                   void* __restrict__ dst, int H) {
  int r = rows[blockIdx.x];
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    st_dt(dst, dt, (size_t)blockIdx.x * H + i, ld_dt(src, dt, (size_t)r * H + i));
}

// ------------------------------------------------------------------------ sampling
// temperature <= 0: the first largest logit.  Otherwise p_i = exp((l_i - max) / T) in double,
// target = u * sum p, answer = first i whose running sum exceeds target, V-1 if none
// (include/nanovllm/sampler.hpp:10-34).  One block per row.  The largest logit is found with the threads striding
// through the row together (a thread meets its own candidates in ascending order and ties go to the lower index
// when threads are compared, so the first largest wins); for the running sum a thread owns a contiguous run of
// the vocabulary, so that it is taken in index order.
constexpr int SAMPLE_THREADS = 1024;
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, int V,
                                                                const float* __restrict__ temperature,
                                                                const double* __restrict__ u,
                                                                int* __restrict__ out) {
  __shared__ float fmx[SAMPLE_THREADS];
  __shared__ int fidx[SAMPLE_THREADS];
  __shared__ double part[SAMPLE_THREADS];
  __shared__ int answer;
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* l = logits + (size_t)row * V;
  const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int b = min(V, tid * per), e = min(V, b + per);
  float mx = -INFINITY;
  int mi = 0x7fffffff;
  for (int i0 = tid; i0 < V; i0 += 4 * SAMPLE_THREADS) {      // four loads in flight
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = i0 + j * SAMPLE_THREADS < V ? l[i0 + j * SAMPLE_THREADS] : -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (v[j] > mx) { mx = v[j]; mi = i0 + j * SAMPLE_THREADS; }
  }
  fmx[tid] = mx;
  fidx[tid] = mi;
  __syncthreads();
  for (int s = SAMPLE_THREADS / 2; s > 0; s >>= 1) {
    if (tid < s) {
      float o = fmx[tid + s];
      int oi = fidx[tid + s];
      if (o > fmx[tid] || (o == fmx[tid] && oi < fidx[tid])) { fmx[tid] = o; fidx[tid] = oi; }
    }
    __syncthreads();
  }
  const float T = temperature[row];
  if (T <= 0.f) {
    if (tid == 0) out[row] = fidx[0] == 0x7fffffff ? 0 : fidx[0];
    return;
  }
  const double mxd = (double)fmx[0], inv_t = 1.0 / (double)T;
  double s = 0.0;
  for (int i = b; i < e; ++i) s += exp(((double)l[i] - mxd) * inv_t);
  part[tid] = s;
  if (tid == 0) answer = V - 1;
  __syncthreads();
  // exclusive prefix over 1024 partial sums: Hillis-Steele on shared memory
  for (int off = 1; off < SAMPLE_THREADS; off <<= 1) {
    double v = tid >= off ? part[tid - off] : 0.0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  const double total = part[SAMPLE_THREADS - 1];
  const double target = u[row] * total;
  const double before = tid ? part[tid - 1] : 0.0;
  if (before <= target && part[tid] > target) {
    double cum = before;
    int a = -1;
    for (int i = b; i < e; ++i) {
      cum += exp(((double)l[i] - mxd) * inv_t);
      if (cum > target) { a = i; break; }
    }
    atomicMin(&answer, a >= 0 ? a : max(b, e - 1));
  }
  __syncthreads();
  if (tid == 0) out[row] = answer;
}

}  // namespace

// =============================================================================== launchers

NV_API const char* nv_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

NV_API int nv_embedding(const int* ids, const int* feed, const void* table, int table_dt, float* out, int T, int H, int V,
                        int* err, cudaStream_t s) {
  if (!dt_ok(table_dt)) return NV_ERR_BAD_DTYPE;
  if (T == 0) return NV_OK;
  NV_RETURN_IF(launch_dep(embedding_kernel, dim3(T), dim3(256), 0, s, ids, table, table_dt, out, H, V, err, feed));
  NV_RETURN_LAST();
}

NV_API int nv_add_rmsnorm(float* x, const float* branch, const void* w, int w_dt, float eps, void* out,
                          int out_dt, float* out32, int T, int H, const float* rows, const int* index,
                          const float* weight, int R, const float* dense, const float* gate_logit,
                          long long gate_ld, cudaStream_t s) {
  if (!dt_ok(w_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (R < 0 || R > NORM_MAX_R || (R > 0 && (!rows || !index || !weight))) return NV_ERR_BAD_SIZE;
  if (branch && (R > 0 || dense)) return NV_ERR_BAD_SIZE;   // one form of the branch at a time
  if (T == 0) return NV_OK;
  NormArgs a;
  a.x = x; a.branch = branch; a.w = w; a.out = out; a.out32 = out32; a.rows = rows; a.index = index;
  a.weight = weight; a.dense = dense; a.gate_logit = gate_logit; a.gate_ld = gate_ld; a.eps = eps;
  a.w_dt = w_dt; a.out_dt = out_dt; a.H = H; a.R = R;
  if (H % 4 == 0) NV_RETURN_IF(launch_dep(add_rmsnorm_kernel<4>, dim3(T), dim3(NORM_THREADS), 0, s, a));
  else NV_RETURN_IF(launch_dep(add_rmsnorm_kernel<1>, dim3(T), dim3(NORM_THREADS), 0, s, a));
  NV_RETURN_LAST();
}

// rot_pos [T][axes] and pair_axis [rotary_dim / 2] (entries in [0, axes)) may be nullptr: every pair is then turned
// by `positions`.
NV_API int nv_rope_store(void* qkv, int dt, const int* positions, const int* rot_pos, int axes, const int* pair_axis,
                         const float* inv_freq, int rotary_dim,
                         void* kc, void* vc, int cache_dt, const int* block_table, int max_blocks,
                         const int* row_entry, int T, int Hq, int Hkv, int D, int page, int write_kv, int* err,
                         cudaStream_t s) {
  if (!dt_ok(dt) || !dt_ok(cache_dt)) return NV_ERR_BAD_DTYPE;
  if (rotary_dim < 0 || rotary_dim > D || rotary_dim % 2) return NV_ERR_BAD_SIZE;
  if (rot_pos && axes < 1) return NV_ERR_BAD_SIZE;
  if (!rot_pos && pair_axis) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  if (D > 256 || D % 2) return NV_ERR_UNSUPPORTED;
  // few rows: many small blocks (latency); many rows: one block per row does all heads (the angles once)
  const int heads = Hq + 2 * Hkv;
  const int hpb = T >= 256 ? heads : 4;
  dim3 grid(T, (heads + hpb - 1) / hpb);
  NV_RETURN_IF(launch_dep(rope_store_kernel, grid, dim3(T >= 256 ? 256 : 128), 0, s, qkv, dt, positions, rot_pos, axes,
                          pair_axis, inv_freq, rotary_dim, kc, vc, cache_dt, block_table, max_blocks, row_entry, Hq, Hkv, D, page, write_kv,
                          hpb, err));
  NV_RETURN_LAST();
}

NV_API int nv_paged_attention_plain(const void* qkv, int dt, int q_stride, const void* kc, const void* vc,
                                    int cache_dt, const int* block_table, int max_blocks, const int* row_entry,
                                    const int* positions, float scale, int window, void* out, int out_dt, int T,
                                    int Hq, int Hkv, int D, int page, cudaStream_t s) {
  if (!dt_ok(dt) || !dt_ok(cache_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (D > 256 || D <= 0 || Hkv <= 0 || Hq % Hkv) return NV_ERR_UNSUPPORTED;
  if (T == 0) return NV_OK;
  dim3 grid(T, Hq);
  paged_attention_plain_kernel<<<grid, ATT_THREADS, 0, s>>>(qkv, dt, q_stride, kc, vc, cache_dt, block_table,
                                                            max_blocks, row_entry, positions, scale, window, out,
                                                            out_dt, Hq, Hkv, D, page);
  NV_RETURN_LAST();
}

NV_API int nv_router_topk(const float* logits, long long ld, int T, int E, int K, int renorm, int* idx,
                          float* score, int C, const float* gate_logit, long long gate_ld, cudaStream_t s) {
  if (K < 1 || K > E || K > 32 || C < 0 || C > 32 || (C > 0 && !gate_logit)) return NV_ERR_UNSUPPORTED;
  if (T == 0) return NV_OK;
  const int warps = 4;
  size_t smem = (size_t)warps * E * sizeof(double);
  if (smem > 48 * 1024) return NV_ERR_UNSUPPORTED;  // E <= 1536
  router_topk_kernel<<<(T + warps - 1) / warps, warps * 32, smem, s>>>(logits, ld, T, E, K, renorm, idx, score, C,
                                                                       gate_logit, gate_ld);
  NV_RETURN_LAST();
}

NV_API int nv_moe_align(const int* idx, int T, int K, int E, int tile_m, int* counts, int* offsets,
                        int* sorted_token, int* pair_pos, int* tile_expert, int* tile_row0, int* tile_rows,
                        int* num_tiles, int* err, int tile_m2, int* t2_expert, int* t2_row0, int* t2_rows,
                        int* num_tiles2, int n_spread, int n_static, int* zero, int n_zero, cudaStream_t s) {
  if (tile_m <= 0 || K <= 0 || E <= 0 || tile_m2 < 0 || n_spread < 0 || n_spread > E) return NV_ERR_BAD_SIZE;
  if (n_zero < 0 || n_zero > 1024 || (n_zero && !zero)) return NV_ERR_BAD_SIZE;
  if (n_static < 0 || n_static > E || (n_static && n_spread)) return NV_ERR_BAD_SIZE;
  if (E > 3000) return NV_ERR_UNSUPPORTED;   // four int arrays of E in shared memory
  moe_align_kernel<<<1, 1024, 4 * E * sizeof(int), s>>>(idx, T * K, K, E, tile_m, counts, offsets, sorted_token,
                                                        pair_pos, tile_expert, tile_row0, tile_rows, num_tiles, err,
                                                        tile_m2, t2_expert, t2_row0, t2_rows, num_tiles2, n_spread,
                                                        n_static, zero, n_zero);
  NV_RETURN_LAST();
}

NV_API int nv_moe_combine(const float* y, const int* pair_pos, const float* score, const float* shared,
                          const float* gate_logit, long long gate_ld, float* out, int T, int K, int H,
                          cudaStream_t s) {
  if (T == 0) return NV_OK;
  dim3 grid(T, (H + 1023) / 1024);
  moe_combine_kernel<<<grid, 256, 0, s>>>(y, pair_pos, score, shared, gate_logit, gate_ld, out, K, H);
  NV_RETURN_LAST();
}

NV_API int nv_silu_mul(const void* gu, int dt, void* out, int out_dt, long long rows, int I, cudaStream_t s) {
  if (!dt_ok(dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  long long n = rows * I;
  if (n == 0) return NV_OK;
  silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gu, dt, out, out_dt, rows, I);
  NV_RETURN_LAST();
}

NV_API int nv_gather_rows(const void* src, int dt, const int* rows, void* dst, int R, int H, cudaStream_t s) {
  if (!dt_ok(dt)) return NV_ERR_BAD_DTYPE;
  if (R == 0) return NV_OK;
  gather_rows_kernel<<<R, 256, 0, s>>>(src, dt, rows, dst, H);
  NV_RETURN_LAST();
}

// Zeroes the per-request state of every entry that starts its request (first position 0): a request's state must
// not begin with what the slot's previous holder, or the request itself before a preemption, left there.
// state: [slots][slot_bytes] bytes, slot_bytes a multiple of 4.  One block per entry.
__global__ void reset_fresh_state_kernel(uint32_t* __restrict__ state, long long slot_words,
                                         const int* __restrict__ entry_slot, const int* __restrict__ entry_pos0,
                                         int num_slots) {
  const int e = blockIdx.x;
  if (entry_pos0[e] != 0) return;
  const int slot = entry_slot[e];
  if (slot < 0 || slot >= num_slots) return;
  uint32_t* p = state + (size_t)slot * slot_words;
  for (long long i = threadIdx.x; i < slot_words; i += blockDim.x) p[i] = 0u;
}

NV_API int nv_reset_fresh_state(void* state, long long slot_bytes, int num_slots, const int* entry_slot,
                                const int* entry_pos0, int S, cudaStream_t s) {
  if (slot_bytes % 4 || ((uintptr_t)state & 3)) return NV_ERR_BAD_SIZE;
  if (S == 0 || slot_bytes == 0) return NV_OK;
  reset_fresh_state_kernel<<<S, 256, 0, s>>>((uint32_t*)state, slot_bytes / 4, entry_slot, entry_pos0, num_slots);
  NV_RETURN_LAST();
}

// The block tables of a step's entries, put together on the device.  tables: [slots][max_blocks], the table of
// every state slot's request as the device knows it; rows: the tables that travelled with this step (those that
// have changed since they last did); src[e]: which of them is entry e's, or -1; lens[e]: pages in entry e's table.
// Entry e's table is taken into tables[slot[e]] if it travelled, and tables[slot[e]][0 .. lens[e]) is copied to
// step[e], which the step's kernels read.  (What lies beyond lens[e] in step[e] is left as it was: no kernel reads
// beyond the pages of its rows.)  One block row per entry.  The reference builds the whole [S][max_blocks] array on
// the host for every step (src/model_runner.cpp:29-41).
__global__ void sync_block_tables_kernel(const int* __restrict__ src, const int* __restrict__ lens,
                                         const int* __restrict__ rows, const int* __restrict__ entry_slot,
                                         int* __restrict__ tables, int* __restrict__ step, int max_blocks,
                                         int num_slots) {
  const int e = blockIdx.x;
  const int slot = entry_slot[e];
  if (slot < 0 || slot >= num_slots) return;
  const int n = min(lens[e], max_blocks), s = src[e];
  int* mine = tables + (size_t)slot * max_blocks;
  int* out = step + (size_t)e * max_blocks;
  const int* sent = s >= 0 ? rows + (size_t)s * max_blocks : nullptr;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
    int v;
    if (sent) {
      v = sent[i];
      mine[i] = v;
    } else {
      v = mine[i];
    }
    out[i] = v;
  }
}

NV_API int nv_sync_block_tables(const int* src, const int* lens, const int* rows, const int* entry_slot, int* tables,
                                int* step, int S, int max_blocks, int num_slots, cudaStream_t s) {
  if (S == 0 || max_blocks <= 0) return NV_OK;
  if (S > num_slots) return NV_ERR_BAD_SIZE;       // step[] has one row per slot
  int chunks = (max_blocks + 1023) / 1024;
  if (chunks > 32) chunks = 32;
  sync_block_tables_kernel<<<dim3((unsigned)S, (unsigned)chunks), 256, 0, s>>>(src, lens, rows, entry_slot, tables, step,
                                                                              max_blocks, num_slots);
  NV_RETURN_LAST();
}

// Keeps the stream busy for about `micros` microseconds (at most 200,000) and does nothing else: a measurement queues
// it before a step, so that the host has launched the whole step by the time the GPU starts on it and the times
// between the step's kernels hold no waits for the host.
__global__ void delay_kernel(unsigned long long nanos) {
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  do {
    __nanosleep(1000);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  } while (t - t0 < nanos);
}

NV_API int nv_delay(int micros, cudaStream_t s) {
  if (micros < 0 || micros > 200000) return NV_ERR_BAD_SIZE;
  if (micros == 0) return NV_OK;
  delay_kernel<<<1, 1, 0, s>>>((unsigned long long)micros * 1000ull);
  NV_RETURN_LAST();
}

NV_API int nv_sample(const float* logits, int R, int V, const float* temperature, const double* u, int* out,
                     cudaStream_t s) {
  if (R == 0) return NV_OK;
  sample_kernel<<<R, SAMPLE_THREADS, 0, s>>>(logits, V, temperature, u, out);
  NV_RETURN_LAST();
}

// 0: every kernel is launched the ordinary way (each starts when the one before it has ended); 1 (the default):
// the kernels of a step are launched as programmatic dependents, see launch_dep.
NV_API void nv_set_dependent_launch(int on) { g_nv_dependent_launch = on ? 1 : 0; }
