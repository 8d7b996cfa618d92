// bfloat16 matrix products on the 5th-generation tensor cores: tcgen05.mma with the accumulator in
// tensor memory (TMEM), operands staged in shared memory by TMA through an mbarrier ring.
//
//   out[t, n] = sum_k X[t, k] * W[n, k]        X: [tokens, K] bf16   W: [rows, K] bf16 (K contiguous)
//
// The weight matrix is the M operand of the instruction (128 rows per CTA) and the tokens are
// the N operand (16..256 per CTA), so one kernel serves decoding (a handful of tokens: the
// tile is 128 weights x 16 tokens and the kernel streams weights at memory speed) and
// prefill (128 x 256 tiles).  Options:
//   swiglu    W holds gate rows [0, N) and up rows [N, 2N); two accumulators share the token
//             operand and the epilogue writes silu(gate) * up
//   grouped   W is [E, rows, K]; token tiles come from a list (expert, first row, rows) over an
//             expert-sorted row list, as built by nv_moe_align with tile_m = the token tile
//   dual      (chosen by the launcher for many tokens) a CTA takes 256 weight rows as two tiles with two
//             accumulators over one token tile: a third fewer operand bytes per flop than one tile
//   split-K   the tile list is walked once per range of k; raw float32 partial sums go to a scratch
//             buffer and a finishing kernel adds them in split order, then bias / swiglu / cast (dense products with
//             few tiles, and grouped ones over a handful of rows, whose few tiles would leave most of the GPU idle)
//
// The kernel is persistent (one or two CTAs per SM walk the tile list) with two accumulator sets in
// TMEM, so a tile's epilogue overlaps the next tile's products.  Warp roles: warp 0 issues TMA
// loads, warp 1 allocates TMEM and issues the MMAs, warps 2-5 read the accumulator back (tcgen05.ld)
// and store.  Launched as a programmatic dependent (`early`), the kernel starts while its predecessor still runs
// and fetches its first weights meanwhile; tokens are read, and anything is written, only after that kernel
// has finished.  The caller may ask for it only if the tile lists of a grouped product were complete before
// that predecessor started.  Every wait on an mbarrier is bounded: after
// about two seconds a waiter records the fact in the error flag and goes on, so the kernel always
// ends and frees its TMEM; its output is then garbage and the host raises.
#include "tcgen05.cuh"

#include <cuda.h>
#include <stdlib.h>
#include <mutex>
#include <unordered_map>

namespace {

constexpr int TILE_W = 128;     // weight rows per CTA (M of the instruction)
constexpr int BLOCK_K = 64;     // elements of K per stage: 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int MAX_STAGES = 8;
constexpr int NUM_THREADS = 192;
constexpr int TQ_DEPTH = 4;     // tile numbers in flight between the producer and the other warps (counter mode)

struct TcArgs {
  void* out;
  float* partial;
  const void* bias;
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tiles;
  int* err;
  long long ldo;
  int out_dt, bias_dt;
  int M_tok;            // rows of X that exist
  int M_out;            // rows of the output (and of every split's partial sums): M_tok, or the sorted rows of a grouped product
  int N;                // output features (rows of W per matrix; W has 2N rows with swiglu)
  int rows_per_expert;  // rows of W per expert (grouped), N or 2N
  int k_steps_total, k_steps_per_split, splits;
  int n_tile, swiglu, dual, stages;   // swiglu and dual both mean two weight tiles per stage
  int w_per_cta;                      // output features per CTA: 128, or 256 with dual
  int n_blocks;                       // blocks of w_per_cta features
  int acc_bufs;                       // accumulator sets in TMEM: 2 when two fit, else 1
  int tmem_cols;
  int early;                          // launched as a programmatic dependent: weights are fetched before the wait
  int x_box;                          // token rows per TMA box of X: min(n_tile, 64)
  // Dense products whose tiles do not fill a last wave of CTAs: the tiles from rest_first on are cut into
  // rest_parts token parts each (numbered part by part after rest_first), so that the last wave is short.
  int rest_first, rest_parts;
  // Grouped products whose tiles' tokens are not rows row0.. of X but rows (row0 - x_sub) mod x_mod.. of it
  // (x_mod > 0): several experts that all take the same rows of a short X, outputs one segment after the other.
  int x_sub, x_mod;
  // Tiles handed out by a counter instead of by position (nullptr: CTA b takes tiles b, b + grid, ...): a CTA that
  // starts late, because another kernel still holds its multiprocessor, then takes fewer tiles, and CTAs whose tiles
  // are short take more.  The counter must be 0 at launch; the CTA that draws the last number sets it back to 0.
  int* tile_counter;
};

// ------------------------------------------------------------------ the kernel
// Persistent: the grid is as many CTAs as fit the GPU at once and every CTA walks the tile list
// tile = blockIdx.x, blockIdx.x + gridDim.x, ...  A tile is (block of output features, token tile,
// k split), features fastest so that CTAs running together share token tiles in L2.  The operand
// ring and the barriers' phases run on across tiles, and the accumulator is double-buffered in
// TMEM (when two fit), so the epilogue of one tile overlaps the products of the next.
struct Tile {
  int nb, row0, x_row0, rows_here, w_row_base, z, n_steps, k_begin;
};

__device__ __forceinline__ bool get_tile(const TcArgs& a, int tile_id, int y_tiles, Tile& t) {
  const int total = a.n_blocks * y_tiles * a.splits;
  int part = 0;
  if (a.rest_parts > 1 && tile_id >= a.rest_first) {
    const int h = tile_id - a.rest_first;
    tile_id = a.rest_first + h / a.rest_parts;
    part = h % a.rest_parts;
  }
  if (tile_id >= total) return false;
  t.nb = tile_id % a.n_blocks;
  const int rest = tile_id / a.n_blocks;
  const int y = rest % y_tiles;
  t.z = rest / y_tiles;
  if (a.tile_expert) {
    t.row0 = a.tile_row0[y];
    t.rows_here = a.tile_rows[y];
    t.w_row_base = a.tile_expert[y] * a.rows_per_expert;
    t.x_row0 = a.x_mod ? (t.row0 - a.x_sub) % a.x_mod : t.row0;
  } else {
    t.row0 = y * a.n_tile;
    t.rows_here = min(a.n_tile, a.M_tok - t.row0);
    t.w_row_base = 0;
    if (a.rest_parts > 1 && tile_id >= a.rest_first) {     // (only when every tile is whole: see the launcher)
      t.rows_here = a.n_tile / a.rest_parts;
      t.row0 += part * t.rows_here;
    }
    t.x_row0 = t.row0;
  }
  t.k_begin = t.z * a.k_steps_per_split;
  t.n_steps = max(0, min(a.k_steps_total, t.k_begin + a.k_steps_per_split) - t.k_begin);
  return true;
}


// The epilogue's work on W (16 or 32) token columns of one tile for this thread's output feature n (and, with two
// accumulator sets, the second set's: the up rows of a SwiGLU, or feature n2 of a dual tile): both sets' loads from
// tensor memory are in flight together, all values are worked out before the first store, and a whole chunk is
// stored without a test per element, so that the one warp a scheduler has for this overlaps its own latencies.
template <int W>
__device__ __forceinline__ void epilogue_chunk(const TcArgs& a, const Tile& t, int two, uint32_t taddr, int c0, int n,
                                               int n2, bool n_ok, bool n2_ok, float bias, float bias2) {
  float g[W], u[W];
  if (t.n_steps > 0) {
    if (W == 32) {
      tmem_ld32_nowait(taddr, g);
      if (two) tmem_ld32_nowait(taddr + a.n_tile, u);
    } else {
      tmem_ld16_nowait(taddr, g);
      if (two) tmem_ld16_nowait(taddr + a.n_tile, u);
    }
    tmem_ld_wait();
    tmem_ld_fence<W>(g);
    if (two) tmem_ld_fence<W>(u);
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j) g[j] = u[j] = 0.f;
  }
  if (!two) {
#pragma unroll
    for (int j = 0; j < W; ++j) u[j] = 0.f;
  }
  if (!n_ok) return;
  const size_t row = (size_t)t.row0 + c0;
  const int valid = min(W, t.rows_here - c0);
  if (a.splits > 1) {
    const int width = a.swiglu ? 2 * a.N : a.N;
    float* p = a.partial + ((size_t)t.z * a.M_out + row) * width;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (j < valid) {
        p[(size_t)j * width + n] = g[j];
        if (a.swiglu) p[(size_t)j * width + a.N + n] = u[j];
        if (n2_ok) p[(size_t)j * width + n2] = u[j];
      }
    }
    return;
  }
  if (valid < W) {
    // a ragged chunk (the few rows of an expert's tile while decoding): only the rows that exist are worked out
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (j < valid) {
        const float v = (a.swiglu ? silu_mul(g[j], u[j]) : g[j]) + bias;
        st_dt(a.out, a.out_dt, (row + j) * a.ldo + n, v);
        if (n2_ok) st_dt(a.out, a.out_dt, (row + j) * a.ldo + n2, u[j] + bias2);
      }
    }
    return;
  }
  if (a.swiglu) {
#pragma unroll
    for (int j = 0; j < W; ++j) g[j] = silu_mul(g[j], u[j]);
  }
#pragma unroll
  for (int j = 0; j < W; ++j) {
    g[j] += bias;
    u[j] += bias2;
  }
  if (a.out_dt == NV_DT_BF16) {
    bf16* o = (bf16*)a.out + row * a.ldo;
#pragma unroll
    for (int j = 0; j < W; ++j) o[(size_t)j * a.ldo + n] = __float2bfloat16_rn(g[j]);
    if (n2_ok) {
#pragma unroll
      for (int j = 0; j < W; ++j) o[(size_t)j * a.ldo + n2] = __float2bfloat16_rn(u[j]);
    }
  } else {
    float* o = (float*)a.out + row * a.ldo;
#pragma unroll
    for (int j = 0; j < W; ++j) o[(size_t)j * a.ldo + n] = g[j];
    if (n2_ok) {
#pragma unroll
      for (int j = 0; j < W; ++j) o[(size_t)j * a.ldo + n2] = u[j];
    }
  }
}

// MODE 0: the small token tiles of decoding; the epilogue takes 16 columns at a time and the kernel stays lean, so that
// the kernels launched beside it find room.  MODE 1: tiles of 32 columns or more; the epilogue works on 32 at a time
// and needs the registers for it.  MODE 2: the same with eight epilogue warps instead of four (two per quarter of the
// tensor memory's lanes, taking turns at the chunks of columns), for the big tiles of a prompt, whose CTAs have a
// multiprocessor to themselves.
constexpr int WIDE_THREADS = 320;
template <int MODE>
__global__ void __launch_bounds__(MODE == 2 ? WIDE_THREADS : NUM_THREADS, MODE == 2 ? 1 : 2)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, TcArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint64_t tq_full[TQ_DEPTH], tq_empty[TQ_DEPTH];       // the producer hands the tile numbers it drew on
  __shared__ int tq_tile[TQ_DEPTH];
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int y_tiles = a.tile_expert ? *a.num_tiles : (a.M_tok + a.n_tile - 1) / a.n_tile;

  // stage layout: [W tile 16 KB][second W tile 16 KB if swiglu or dual][X n_tile*128 B], each 1024-aligned
  const int two = (a.swiglu || a.dual) ? 1 : 0;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t a_bytes = TILE_W * 128, x_bytes = a.n_tile * 128;
  const uint32_t stage_bytes = a_bytes * (two ? 2 : 1) + x_bytes;
  const int acc_cols = a.n_tile * (two ? 2 : 1);   // TMEM columns of one accumulator set

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_x) : "memory");
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], MODE == 2 ? 8 : 4);  // one arrival per epilogue warp
    }
    for (int q = 0; q < TQ_DEPTH; ++q) {
      mbar_init(&tq_full[q], 1);
      mbar_init(&tq_empty[q], 1 + (MODE == 2 ? 8 : 4));   // the MMA thread and every epilogue warp have read it
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, a.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const bool by_counter = a.tile_counter != nullptr;
  // The n-th tile of this CTA as the MMA thread and the epilogue warps learn it: by position, or from the producer.
  // (`whole_warp`: all 32 lanes call it together, as the epilogue warps do; the MMA thread calls it alone.)
  auto nth_tile = [&](int n, bool whole_warp) -> int {
    if (!by_counter) return (int)blockIdx.x + n * (int)gridDim.x;
    const int q = n % TQ_DEPTH;
    mbar_wait(&tq_full[q], (n / TQ_DEPTH) & 1, a.err, 0x7005);
    const int tile = tq_tile[q];
    if (whole_warp) __syncwarp();                  // every lane has read the number before the slot is given back
    if (lane == 0) mbar_arrive(&tq_empty[q]);
    return tile;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // Launched early (a.early), the kernel may run beside the one before it: the weights of the first ring-full
    // of k-steps are fetched at once, the tokens (that kernel's output) only after it has finished.
    if (lane == 0) {
      const int pre = a.early ? a.stages : 0;
      const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(&full_bar[0]);
      // The n-th tile of this CTA as the producer learns it: by position, or by drawing the next number from the
      // counter, which it also hands on to the other warps.  Numbers past the last tile end the walk; the CTA that
      // draws the very last one (every CTA draws exactly one such number) sets the counter back for the next launch.
      const int total_tiles = a.n_blocks * y_tiles * a.splits;
      auto draw = [&](int n) -> int {
        if (!by_counter) return (int)blockIdx.x + n * (int)gridDim.x;
        const int tile = atomicAdd(a.tile_counter, 1);
        if (tile == total_tiles + (int)gridDim.x - 1) *a.tile_counter = 0;
        const int q = n % TQ_DEPTH;
        mbar_wait(&tq_empty[q], ((n / TQ_DEPTH) & 1) ^ 1, a.err, 0x7006);
        tq_tile[q] = tile;
        mbar_arrive(&tq_full[q]);
        return tile;
      };
      int it = 0;                                              // k-steps issued so far
      int s = 0, ph = 0;                                       // stage and phase of k-step `it`, kept by counting
      // issues k-steps [k0, k1) of a tile: weights and / or tokens
      auto issue = [&](const Tile& t, int k0, int k1, bool weights, bool tokens, int s_, int ph_) {
        // tokens come in boxes of x_box rows, as many as the tile's rows (rounded up to the 16 of the MMA) need.
        // (What a tile fixes is worked out here, once: this one thread's instructions are the pace of the ring.)
        const int n_act = min(a.n_tile, (t.rows_here + 15) & ~15);
        const int boxes = (n_act + a.x_box - 1) / a.x_box;
        const uint32_t bytes = a_bytes * (two ? 2 : 1) + (uint32_t)boxes * a.x_box * 128;
        const int wr = t.w_row_base + t.nb * a.w_per_cta;
        for (int k = k0; k < k1; ++k, s_ = (s_ + 1 == a.stages ? 0 : s_ + 1), ph_ ^= (s_ == 0)) {
          const uint32_t st = smem0 + (uint32_t)s_ * stage_bytes, bar = full0 + (uint32_t)s_ * 8;
          if (weights) {
            mbar_wait(&empty_bar[s_], ph_ ^ 1, a.err, 0x7001);
            mbar_expect_tx_a(bar, bytes);
          }
          const int kc = (t.k_begin + k) * BLOCK_K;
          if (weights) {
            tma_load_2d_a(st, &tm_w, bar, kc, wr);
            if (two)     // swiglu: the up rows of the same features; dual: the next 128 features
              tma_load_2d_a(st + a_bytes, &tm_w, bar, kc, wr + (a.swiglu ? a.N : TILE_W));
          }
          if (tokens)
            for (int b = 0; b < boxes; ++b)
              tma_load_2d_a(st + a_bytes * (two ? 2 : 1) + (uint32_t)b * a.x_box * 128, &tm_x, bar, kc,
                            t.x_row0 + b * a.x_box);
        }
      };
      auto advance = [&](int steps) {
        for (int k = 0; k < steps; ++k) {
          if (++s == a.stages) { s = 0; ph ^= 1; }
        }
        it += steps;
      };
      Tile t;
      int n = 0;
      bool have = get_tile(a, draw(n), y_tiles, t);
      if (pre) {
        // the weights of the first ring-full of k-steps before the wait, their tokens after it.  (By position the
        // ring-full may span several tiles; by counter it ends with the first tile, the second is drawn later.)
        if (!by_counter) {
          // walk the first `pre` k-steps twice
          Tile u = t;
          int n2 = 0, left = pre, s2 = 0, ph2 = 0;
          bool h2 = have;
          while (h2 && left > 0) {
            const int k1 = min(u.n_steps, left);
            issue(u, 0, k1, true, false, s2, ph2);
            for (int k = 0; k < k1; ++k) if (++s2 == a.stages) { s2 = 0; ph2 ^= 1; }
            left -= k1;
            if (k1 < u.n_steps) break;
            h2 = get_tile(a, draw(++n2), y_tiles, u);
          }
          grid_dep_wait();
          left = pre;
          while (have && left > 0) {
            const int k1 = min(t.n_steps, left);
            issue(t, 0, k1, false, true, s, ph);
            advance(k1);
            left -= k1;
            if (k1 < t.n_steps) {          // the rest of this tile follows below
              issue(t, k1, t.n_steps, true, true, s, ph);
              advance(t.n_steps - k1);
            }
            have = get_tile(a, draw(++n), y_tiles, t);
          }
        } else {
          const int k1 = have ? min(t.n_steps, pre) : 0;
          if (have) issue(t, 0, k1, true, false, s, ph);
          grid_dep_wait();
          if (have) {
            issue(t, 0, k1, false, true, s, ph);
            advance(k1);
            issue(t, k1, t.n_steps, true, true, s, ph);
            advance(t.n_steps - k1);
            have = get_tile(a, draw(++n), y_tiles, t);
          }
        }
      }
      while (have) {
        issue(t, 0, t.n_steps, true, true, s, ph);
        advance(t.n_steps);
        have = get_tile(a, draw(++n), y_tiles, t);
      }
      grid_dep_launch();          // all loads are on their way: the next kernel may take the SMs that fall idle
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int it = 0, n = 0;                           // k-steps consumed, tiles done
      int s = 0;                                   // stage of k-step `it` and the parity of its use, kept by counting:
      uint32_t ph = 0;                             // this one thread's instructions pace the tensor core
      const uint64_t desc0 = smem_desc_sw128(0);
      const uint32_t smem0 = smem_u32(smem);
      Tile t;
      for (; get_tile(a, nth_tile(n, false), y_tiles, t); ++n) {
        const int b = a.acc_bufs == 2 ? (n & 1) : 0;
        const int use = a.acc_bufs == 2 ? (n >> 1) : n;          // how often this buffer was used before
        mbar_wait(&acc_empty[b], (use & 1) ^ 1, a.err, 0x7004);  // the epilogue has drained it
        tc_fence_after();
        const uint32_t acc_addr = tmem_base + b * acc_cols;
        // the N of the instruction is what the tile's rows need, not the widest tile: a short last tile of an
        // expert costs a short product
        const uint32_t idesc = instr_desc(min(a.n_tile, (t.rows_here + 15) & ~15));
        for (int k = 0; k < t.n_steps; ++k, ++it) {
          mbar_wait(&full_bar[s], ph, a.err, 0x7002);
          tc_fence_after();
          // a descriptor is fixed bits plus the tile's address / 16 (shared memory addresses fit its 14 bits)
          const uint64_t da = desc0 + (uint64_t)((smem0 + (uint32_t)s * stage_bytes) >> 4);
          const uint64_t du = da + (uint64_t)(a_bytes >> 4);
          const uint64_t dx = da + (uint64_t)((a_bytes * (two ? 2 : 1)) >> 4);
          // (the order differs from slice-by-slice over both accumulators only in which accumulator goes first)
          umma_bf16_x4(acc_addr, da, dx, idesc, k > 0 ? 1u : 0u);
          if (two) umma_bf16_x4(acc_addr + a.n_tile, du, dx, idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);     // the stage may be refilled once these MMAs have read it
          if (++s == a.stages) { s = 0; ph ^= 1; }
        }
        umma_commit(&acc_full[b]);        // the accumulator is complete (at once if the tile had no k-steps)
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: warps 2..5
    const int q = warp % 4;                        // a warp may read TMEM lanes [32q, 32q + 32) only
    int n_done = 0;
    Tile t;
    for (; get_tile(a, nth_tile(n_done, true), y_tiles, t); ++n_done) {
      const int b = a.acc_bufs == 2 ? (n_done & 1) : 0;
      const int use = a.acc_bufs == 2 ? (n_done >> 1) : n_done;
      const int n = t.nb * a.w_per_cta + q * 32 + lane;   // this thread's output feature (dual: and n + 128)
      const int n2 = n + TILE_W;
      const bool n_ok = n < a.N, n2_ok = a.dual && n2 < a.N;
      mbar_wait(&acc_full[b], use & 1, a.err, 0x7003);
      tc_fence_after();
      float bias = 0.f, bias2 = 0.f;
      if (a.bias && a.splits == 1) {
        if (n_ok) bias = ld_dt(a.bias, a.bias_dt, n);
        if (n2_ok) bias2 = ld_dt(a.bias, a.bias_dt, n2);
      }
      const uint32_t lane_addr = tmem_base + b * acc_cols + ((uint32_t)(q * 32) << 16);
      if (MODE == 2) {
        for (int c0 = warp >= 6 ? 32 : 0; c0 < t.rows_here; c0 += 64)
          epilogue_chunk<32>(a, t, two, lane_addr + c0, c0, n, n2, n_ok, n2_ok, bias, bias2);
      } else if (MODE == 1) {
        for (int c0 = 0; c0 < t.rows_here; c0 += 32)             // uniform over the warp
          epilogue_chunk<32>(a, t, two, lane_addr + c0, c0, n, n2, n_ok, n2_ok, bias, bias2);
      } else {
        for (int c0 = 0; c0 < a.n_tile; c0 += 16) {
          if (c0 >= t.rows_here) break;                // uniform over the warp
          float g[16], u[16];
          if (t.n_steps > 0) {
            tmem_ld16(lane_addr + c0, g);
            if (two) tmem_ld16(lane_addr + a.n_tile + c0, u);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.f;
          }
          if (!n_ok) continue;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j >= t.rows_here) break;
            const size_t row = (size_t)(t.row0 + c0 + j);
            if (a.splits > 1) {
              const int width = a.swiglu ? 2 * a.N : a.N;
              float* p = a.partial + ((size_t)t.z * a.M_out + row) * width;
              p[n] = g[j];
              if (a.swiglu) p[a.N + n] = u[j];
              if (n2_ok) p[n2] = u[j];
            } else {
              float v = a.swiglu ? silu_mul(g[j], u[j]) : g[j];
              st_dt(a.out, a.out_dt, row * a.ldo + n, v + bias);
              if (n2_ok) st_dt(a.out, a.out_dt, row * a.ldo + n2, u[j] + bias2);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);   // this warp has read all it needs from the buffer
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, a.tmem_cols);
}

// Adds split-K partial sums in split order and finishes: bias, swiglu, cast.
__global__ void tc_gemm_finish_kernel(const float* __restrict__ partial, int splits, int M_tok, int N, int swiglu,
                                      const void* __restrict__ bias, int bias_dt, void* __restrict__ out, int out_dt,
                                      long long ldo) {
  grid_dep_wait();
  grid_dep_launch();
  const int width = swiglu ? 2 * N : N;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M_tok * N) return;
  const long long t = i / N;
  const int n = (int)(i % N);
  float g = 0.f, u = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* p = partial + ((size_t)s * M_tok + t) * width;
    g += p[n];
    if (swiglu) u += p[N + n];
  }
  float v = swiglu ? silu_mul(g, u) : g;
  if (bias) v += ld_dt(bias, bias_dt, n);
  st_dt(out, out_dt, t * ldo + n, v);
}

// The same for a grouped product: only the rows that the tile list covers are finished (other rows of `out` belong
// to other products).  One block per (tile, 256 features).
__global__ void tc_gemm_finish_grouped_kernel(const float* __restrict__ partial, int splits, int M_out, int N, int swiglu,
                                              const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                                              const int* __restrict__ num_tiles, void* __restrict__ out, int out_dt,
                                              long long ldo) {
  grid_dep_wait();
  grid_dep_launch();
  const int y = blockIdx.x;
  if (y >= *num_tiles) return;
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const int width = swiglu ? 2 * N : N;
  const int row0 = tile_row0[y], rows = tile_rows[y];
  for (int r = row0; r < row0 + rows; ++r) {
    float g = 0.f, u = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* p = partial + ((size_t)s * M_out + r) * width;
      g += p[n];
      if (swiglu) u += p[N + n];
    }
    st_dt(out, out_dt, (long long)r * ldo + n, swiglu ? silu_mul(g, u) : g);
  }
}

// out[r, :] = src[rows[r], :] for bf16 rows (the expert-sorted copy of the activations)
__global__ void permute_rows_bf16_kernel(const bf16* __restrict__ src, const int* __restrict__ rows,
                                         bf16* __restrict__ dst, int H) {
  grid_dep_wait();
  grid_dep_launch();
  const int r = blockIdx.x;
  const uint4* s = (const uint4*)(src + (size_t)rows[r] * H);
  uint4* d = (uint4*)(dst + (size_t)r * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) d[i] = s[i];
}

// ------------------------------------------------------------------ host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    return h * 1000003u ^ (size_t)k.box_rows;
  }
};

}  // namespace

// A row-major bf16 matrix [rows, cols] with row stride ld elements; boxes of box_rows x 64, 128-byte swizzle,
// zero fill outside.  Cached by (pointer, shape, box).  Declared in pipeline.cuh for the other kernels.
int nv_tensor_map_bf16(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return NV_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -5;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -5;
  if (cache.size() > 8192) cache.clear();
  cache[key] = m;
  *out = m;
  return NV_OK;
}

namespace {

int get_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  return nv_tensor_map_bf16(ptr, rows, cols, ld, box_rows, out);
}

int pow2_at_least(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

// Token tile the product will use for `rows` tokens (dense) or for the largest expected expert segment
// (grouped): the N of the instruction, 16..256.
NV_API int nv_tc_gemm_token_tile(int rows, int swiglu) {
  int cap = swiglu ? 128 : 256;   // SwiGLU keeps two accumulators per feature tile: a narrower token tile suits it
  int t = 16;
  while (t < rows && t < cap) t <<= 1;
  return t;
}

// Bytes of float32 scratch a call needs for its split-K partial sums (0 when it does not split).
NV_API long long nv_tc_gemm_scratch_bytes(int M_tok, int N, int swiglu, int splits) {
  if (splits <= 1) return 0;
  return (long long)splits * M_tok * (swiglu ? 2 * N : N) * 4;
}

// How many ways to split K so that a small grid still fills the GPU.  1 for large grids.
NV_API int nv_tc_gemm_splits(int M_tok, int N, int K, int n_tile, int num_sms) {
  int ctas = ((N + TILE_W - 1) / TILE_W) * ((M_tok + n_tile - 1) / n_tile);
  int k_steps = (K + BLOCK_K - 1) / BLOCK_K;
  if (ctas >= num_sms || k_steps < 8) return 1;
  // a few rows: two CTAs of these small stages live on a multiprocessor; many rows: the partial sums are big, so
  // split only what would leave more than half of the GPU idle
  int s = (M_tok <= 64 ? 2 * num_sms : num_sms) / ctas;
  if (s > k_steps / 4) s = k_steps / 4;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

NV_API int nv_tc_gemm(const void* X, long long ldx, int M_tok, const void* W, int w_rows_total, int N, int K,
                      const void* bias, int bias_dt, void* out, int out_dt, long long ldo, int swiglu, int n_tile,
                      int splits, float* scratch, const int* tile_expert, const int* tile_row0,
                      const int* tile_rows, const int* num_tiles, int max_tiles, int rows_per_expert, int* err,
                      int early, int x_sub, int x_mod, int max_ctas, int* tile_counter, int m_out,
                      cudaStream_t stream) {
  if (!dt_ok(out_dt) || (bias && !dt_ok(bias_dt))) return NV_ERR_BAD_DTYPE;
  if (K % 8 || ldx % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return NV_ERR_UNSUPPORTED;  // TMA: 16-byte rules
  if (n_tile < 16 || n_tile > 256 || (n_tile & (n_tile - 1))) return NV_ERR_BAD_SIZE;
  if (M_tok <= 0 || N <= 0) return NV_OK;
  const bool grouped = tile_expert != nullptr;
  if (grouped && splits > 1 && m_out <= 0) return NV_ERR_BAD_SIZE;     // the partial sums are [splits, m_out, width]
  if (x_mod < 0 || x_sub < 0 || (x_mod && !grouped)) return NV_ERR_BAD_SIZE;
  if (splits > 1 && !scratch) return NV_ERR_BAD_SIZE;

  CUtensorMap tm_w, tm_x;
  int rc = get_map(W, w_rows_total, K, K, TILE_W, &tm_w);
  if (rc) return rc;
  const int x_box = n_tile < 64 ? n_tile : 64;
  rc = get_map(X, M_tok, K, ldx, x_box, &tm_x);
  if (rc) return rc;

  TcArgs a;
  a.out = out; a.partial = scratch; a.bias = bias; a.tile_expert = tile_expert; a.tile_row0 = tile_row0;
  a.tile_rows = tile_rows; a.num_tiles = num_tiles; a.err = err; a.ldo = ldo; a.out_dt = out_dt; a.bias_dt = bias_dt;
  a.M_tok = M_tok; a.N = N; a.rows_per_expert = rows_per_expert;
  a.M_out = grouped && m_out > 0 ? m_out : M_tok;
  a.k_steps_total = (K + BLOCK_K - 1) / BLOCK_K;
  a.splits = splits < 1 ? 1 : splits;
  a.k_steps_per_split = (a.k_steps_total + a.splits - 1) / a.splits;
  a.n_tile = n_tile; a.swiglu = swiglu ? 1 : 0;
  a.early = early ? 1 : 0;
  a.x_box = x_box;
  a.x_sub = x_sub; a.x_mod = x_mod;
  a.tile_counter = tile_counter;
  // Many tokens per tile and enough features: two weight tiles per CTA.  The operands then cost 2*16 KB + X
  // per k-step for twice the flops, which is what the shared-memory fill rate, the limit here, rewards.
  // ... provided the halved grid still covers the GPU (measured: a half-empty GPU loses more than the tile gains)
  const bool many_tokens = tile_expert ? n_tile >= 128
                                       : (M_tok >= 256 && (long long)((N + 255) / 256) * ((M_tok + n_tile - 1) / n_tile) >= 120);
  a.dual = (!swiglu && many_tokens && N >= 2 * TILE_W && a.splits == 1) ? 1 : 0;
  a.w_per_cta = a.dual ? 2 * TILE_W : TILE_W;
  static std::once_flag once;
  static cudaError_t attr_rc = cudaSuccess;
  static int num_sms = 0;
  std::call_once(once, [] {
    attr_rc = cudaFuncSetAttribute(tc_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (attr_rc == cudaSuccess)
      attr_rc = cudaFuncSetAttribute(tc_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (attr_rc == cudaSuccess)
      attr_rc = cudaFuncSetAttribute(tc_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    int dev = 0;
    if (attr_rc == cudaSuccess) attr_rc = cudaGetDevice(&dev);
    if (attr_rc == cudaSuccess) attr_rc = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  });
  if (attr_rc != cudaSuccess) return (int)attr_rc;

  const int two = (swiglu || a.dual) ? 1 : 0;
  const int stage_bytes = TILE_W * 128 * (two ? 2 : 1) + n_tile * 128;
  a.n_blocks = (N + a.w_per_cta - 1) / a.w_per_cta;
  const int acc_cols = n_tile * (two ? 2 : 1);
  a.acc_bufs = acc_cols <= 256 ? 2 : 1;
  a.tmem_cols = pow2_at_least(acc_cols * a.acc_bufs);
  // Small stages (few tokens): keep a CTA under half of the shared memory so that two CTAs share an SM and
  // one's start-up and epilogue overlap the other's streaming.  Large stages, or more than half of the
  // TMEM columns: one CTA per SM, deep ring.
  // (with many rows, hence most experts in use and many tiles, two CTAs with three stages each stream the
  // SwiGLU product's two weight tiles a little faster than one CTA with five: measured at batch 64, not at 8 or 1)
  const int min_stages = (grouped && swiglu && M_tok >= 256) ? 3 : 4;
  const bool pair = stage_bytes * min_stages <= 104 * 1024 && a.tmem_cols <= 256;
  const int budget = pair ? 104 * 1024 : 200 * 1024;
  int stages = budget / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) return NV_ERR_UNSUPPORTED;
  a.stages = stages;
  size_t smem = (size_t)stages * stage_bytes + 1024;
  if (!pair && smem < 120 * 1024) smem = 120 * 1024;   // more than half an SM's shared memory: no second CTA

  const long long y_tiles = grouped ? max_tiles : (M_tok + n_tile - 1) / n_tile;
  const long long total = (long long)a.n_blocks * y_tiles * a.splits;     // an upper bound when grouped
  // `max_ctas` > 0 caps the grid: a product that runs beside other kernels on a second stream leaves them
  // multiprocessors (its CTAs each hold one for the whole tile list)
  long long resident = (long long)num_sms * (pair ? 2 : 1);
  if (max_ctas > 0 && max_ctas < resident) resident = max_ctas;
  dim3 grid((unsigned)(total < resident ? total : resident));
  // a last wave with tiles for less than half of the CTAs: cut those tiles into two or four token parts
  a.rest_first = 0;
  a.rest_parts = 1;
  if (!grouped && !tile_counter && a.splits == 1 && total > resident && M_tok % n_tile == 0 && n_tile >= 128) {
    const long long rest = total % resident;
    if (rest > 0 && rest * 2 <= resident) {
      a.rest_parts = (rest * 4 <= resident && n_tile >= 256) ? 4 : 2;
      a.rest_first = (int)(total - rest);
    }
  }
  const int mode = n_tile < 32 ? 0 : ((!pair && n_tile >= 128) ? 2 : 1);
  const auto kernel = mode == 0 ? tc_gemm_kernel<0> : (mode == 1 ? tc_gemm_kernel<1> : tc_gemm_kernel<2>);
  const unsigned threads = mode == 2 ? WIDE_THREADS : NUM_THREADS;
  cudaError_t e;
  if (a.early) {
    // programmatic dependent of the kernel before it in the stream (an edge of that kind when captured)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_nv_dependent_launch ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, tm_w, tm_x, a);
    if (e != cudaSuccess) return (int)e;
  } else {
    kernel<<<grid, threads, smem, stream>>>(tm_w, tm_x, a);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (a.splits > 1) {
    if (grouped) {
      NV_RETURN_IF(launch_dep(tc_gemm_finish_grouped_kernel, dim3((unsigned)max_tiles, (unsigned)((N + 255) / 256)),
                              dim3(256), 0, stream, (const float*)scratch, a.splits, a.M_out, N, a.swiglu, tile_row0,
                              tile_rows, num_tiles, out, out_dt, ldo));
    } else {
      const long long outputs = (long long)a.M_out * N;
      NV_RETURN_IF(launch_dep(tc_gemm_finish_kernel, dim3((unsigned)((outputs + 255) / 256)), dim3(256), 0, stream,
                              (const float*)scratch, a.splits, a.M_out, N, a.swiglu, bias, bias_dt, out, out_dt, ldo));
    }
  }
  NV_RETURN_LAST();
}

NV_API int nv_permute_rows_bf16(const void* src, const int* rows, void* dst, int R, int H, cudaStream_t stream) {
  if (H % 8 || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) return NV_ERR_UNSUPPORTED;
  if (R == 0) return NV_OK;
  NV_RETURN_IF(launch_dep(permute_rows_bf16_kernel, dim3(R), dim3(128), 0, stream, (const bf16*)src, rows, (bf16*)dst, H));
  NV_RETURN_LAST();
}

