// Routing of a mixture of experts: per-row top-k of the router's softmax, and the permutation of
// (row, expert) pairs into expert order that the grouped products work on.  Device functions shared
// by the stand-alone kernels (plain_ops.cu) and the fused small-batch kernel (small_ops.cu).
#pragma once

#include "common.cuh"

// One warp routes one row: p = softmax(logits) over all E in double, then K rounds of "largest
// remaining, lowest index on a tie", optional renormalisation of the K weights in double
// (src/hip_ops.hip:813-841).  `pr` is E doubles of scratch for this warp.  With C > 0 the row also
// gets C "always on" experts E .. E+C-1 with weight sigmoid(gate_logit): the chunks of a shared
// expert that is computed as C more experts (src/model.cpp:803-811 computes it separately).
// idx and score rows are K + C wide.
__device__ __forceinline__ void route_row(const float* __restrict__ r, int E, int K, int renorm, double* pr,
                                          int lane, int* __restrict__ idx_row, float* __restrict__ score_row,
                                          int C, const float* gate_logit) {
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, r[e]);
  mx = warp_max(mx);
  double s = 0.0;
  for (int e = lane; e < E; e += 32) {
    double v = exp((double)r[e] - (double)mx);
    pr[e] = v;
    s += v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __syncwarp();
  for (int e = lane; e < E; e += 32) pr[e] /= s;
  __syncwarp();
  double wsum = 0.0;
  double mine = 0.0;  // lane k keeps the k-th weight (K <= 32)
  for (int k = 0; k < K; ++k) {
    double best = -1.0;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      double v = pr[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      double ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == k) { mine = best; idx_row[k] = bi; }
    wsum += best;
    if (lane == 0) pr[bi] = -2.0;
    __syncwarp();
  }
  if (lane < K) score_row[lane] = (float)(renorm ? mine / wsum : mine);
  if (lane < C) {
    idx_row[K + lane] = E + lane;
    score_row[K + lane] = 1.f / (1.f + expf(-gate_logit[0]));
  }
}

// Re-orders a tile list of `total` entries whose last `tail` entries belong to experts that every row visits (a few
// experts with very many rows: their weights stay in L2 and their tiles are bound by arithmetic) so that those are
// spread evenly among the others (many experts with few rows each: their tiles are bound by the stream of
// weights from memory).  CTAs that walk the list together then work on both kinds at once, and the two limits
// overlap instead of following one another.  One block; every entry is read before any is written.
__device__ __forceinline__ void spread_tail_tiles(int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                                  int* __restrict__ tile_rows, int total, int tail) {
  constexpr int PER = 4;                          // entries per thread: lists longer than PER * threads stay as they are
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int head = total - tail;
  if (tail <= 0 || head <= 0 || total > PER * nthr) return;
  int e[PER], r0[PER], rw[PER];
#pragma unroll
  for (int u = 0; u < PER; ++u) {
    const int j = tid + u * nthr;
    if (j < total) {
      // of the slots before j, floor(j * tail / total) hold tail entries; slot j is one if that count steps at j + 1
      const int before = (int)((long long)j * tail / total), upto = (int)((long long)(j + 1) * tail / total);
      const int src = upto > before ? head + before : j - before;
      e[u] = tile_expert[src];
      r0[u] = tile_row0[src];
      rw[u] = tile_rows[src];
    }
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < PER; ++u) {
    const int j = tid + u * nthr;
    if (j < total) {
      tile_expert[j] = e[u];
      tile_row0[j] = r0[u];
      tile_rows[j] = rw[u];
    }
  }
}

// From idx[TK] (expert of every (row, k) pair; K pairs per row) build, for the grouped products:
// counts and offsets per expert, the pairs sorted by expert (sorted_token = source row of each sorted
// position, pair_pos = sorted position of each pair) and the list of tiles (expert, first row, rows)
// of at most tile_m rows — and a second list cut by tile_m2, for a product that prefers another tile
// (t2 == nullptr: none).  One block of 1024 threads; `al_s` is 4 * E ints of shared memory.  The
// order of pairs inside an expert's segment comes from atomics and may differ from run to run; it
// decides only where a pair's row sits, never a sum's order.
// The last `n_static` experts are ones that every row visits (a shared expert's chunks): their pairs sit in row
// order, so their part of the permutation is known before any routing is (segment of expert E - n_static + c
// starts at TK - (n_static - c) * rows), and they get no tiles here: whoever runs them has a fixed list.
// With `n_spread` instead, the tiles of the last n_spread experts are spread through the list (spread_tail_tiles).
__device__ __forceinline__ void align_block(const int* __restrict__ idx, int TK, int K, int E, int tile_m,
                                            int* __restrict__ counts, int* __restrict__ offsets,
                                            int* __restrict__ sorted_token, int* __restrict__ pair_pos,
                                            int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                            int* __restrict__ tile_rows, int* __restrict__ num_tiles,
                                            int* __restrict__ err, int* al_s, int tile_m2 = 0,
                                            int* __restrict__ t2_expert = nullptr, int* __restrict__ t2_row0 = nullptr,
                                            int* __restrict__ t2_rows = nullptr, int* __restrict__ num_tiles2 = nullptr,
                                            int n_static = 0, int n_spread = 0) {
  const int E_dyn = E - n_static;
  int* cnt = al_s;
  int* cur = al_s + E;
  int* tbase = al_s + 2 * E;
  int* tbase2 = al_s + 3 * E;
  const int tid = threadIdx.x, nthr = blockDim.x;
  for (int e = tid; e < E; e += nthr) cnt[e] = 0;
  __syncthreads();
  // eight loads in flight per thread: one load per atomic made the two passes over idx the kernel's time
  for (int i0 = tid; i0 < TK; i0 += 8 * nthr) {
    int ev[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) ev[u] = i0 + u * nthr < TK ? idx[i0 + u * nthr] : 0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * nthr;
      if (i >= TK) break;
      if (ev[u] < 0 || ev[u] >= E) { atomicExch(err, 1 + i); continue; }
      atomicAdd(&cnt[ev[u]], 1);
    }
  }
  __syncthreads();
  if (tid < 32) {                           // warp 0: exclusive prefix sums over the experts, 32 at a time
    int carry_c = 0, carry_t = 0, carry_t2 = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + tid;
      const int c = e < E ? cnt[e] : 0;
      const int tl = e < E_dyn ? (c + tile_m - 1) / tile_m : 0;
      const int tl2 = (tile_m2 && e < E_dyn) ? (c + tile_m2 - 1) / tile_m2 : 0;
      int sc = c, st = tl, st2 = tl2;       // inclusive scans
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int uc = __shfl_up_sync(0xffffffffu, sc, o), ut = __shfl_up_sync(0xffffffffu, st, o),
                  ut2 = __shfl_up_sync(0xffffffffu, st2, o);
        if (tid >= o) { sc += uc; st += ut; st2 += ut2; }
      }
      if (e < E) {
        cur[e] = carry_c + sc - c;
        tbase[e] = carry_t + st - tl;
        tbase2[e] = carry_t2 + st2 - tl2;
      }
      carry_c += __shfl_sync(0xffffffffu, sc, 31);
      carry_t += __shfl_sync(0xffffffffu, st, 31);
      carry_t2 += __shfl_sync(0xffffffffu, st2, 31);
    }
    if (tid == 0) {
      offsets[E] = carry_c;
      *num_tiles = carry_t;
      if (tile_m2) *num_tiles2 = carry_t2;
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += nthr) {
    const int c = cnt[e], off = cur[e];
    counts[e] = c;
    offsets[e] = off;
    if (e >= E_dyn) continue;
    for (int r = 0, t = tbase[e]; r < c; r += tile_m, ++t) {
      tile_expert[t] = e;
      tile_row0[t] = off + r;
      tile_rows[t] = min(tile_m, c - r);
    }
    if (tile_m2)
      for (int r = 0, t = tbase2[e]; r < c; r += tile_m2, ++t) {
        t2_expert[t] = e;
        t2_row0[t] = off + r;
        t2_rows[t] = min(tile_m2, c - r);
      }
  }
  __syncthreads();
  for (int i0 = tid; i0 < TK; i0 += 8 * nthr) {
    int ev[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) ev[u] = i0 + u * nthr < TK ? idx[i0 + u * nthr] : -1;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * nthr;
      if (i >= TK) break;
      if (ev[u] < 0 || ev[u] >= E) continue;
      const int p = ev[u] < E_dyn ? atomicAdd(&cur[ev[u]], 1) : cur[ev[u]] + i / K;
      sorted_token[p] = i / K;
      pair_pos[i] = p;
    }
  }
  if (n_spread > 0 && n_spread < E) {
    __threadfence_block();
    __syncthreads();                       // the lists are complete, and this block wrote them
    const int first = E - n_spread;        // tbase of the first spread expert = entries before the tail
    int total = 0, total2 = 0;
    {
      const int cl = cnt[E - 1];
      total = tbase[E - 1] + (cl + tile_m - 1) / tile_m;
      if (tile_m2) total2 = tbase2[E - 1] + (cl + tile_m2 - 1) / tile_m2;
    }
    spread_tail_tiles(tile_expert, tile_row0, tile_rows, total, total - tbase[first]);
    if (tile_m2) spread_tail_tiles(t2_expert, t2_row0, t2_rows, total2, total2 - tbase2[first]);
  }
}
