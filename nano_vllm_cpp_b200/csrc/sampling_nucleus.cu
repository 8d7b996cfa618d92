// Nucleus (top-p) sampling with a windowed repetition penalty: the rule of the reference's second sampler
// (include/nanovllm/sampler.hpp:46-88), one block per row, without sorting the vocabulary.
//
//   temperature <= 0: the first largest logit (never penalised).
//   s_i = float(exp(double(l_i - max) / T))
//   every id seen among the row's recent tokens (each id once): s_id /= float(penalty)       (penalty 1 = off)
//   tokens in descending order of s (equal scores: lower id first); running mass acc; the nucleus ends at the first
//     position i > 0 with acc >= top_p * sum (so it holds at least two tokens); if none, at the last token
//   r = u * acc(nucleus); the answer is the first token of the nucleus whose running mass reaches r
//
// Instead of a sort, a position in the descending order is found by its running mass: three passes of a radix
// histogram over the bits of s (11 + 11 + 10), each bin holding a count and a mass, walk down from the largest
// scores to the bin in which the running mass reaches the target; equal scores are then taken in index order.
// Masses are 64-bit integers, s * 2^40 rounded: integer sums do not depend on the order of the atomic adds, so
// a row's token is the same in every run.  (A token whose s is below 2^-41 of the largest carries no mass.)
#include "common.cuh"

namespace {

constexpr int NUC_THREADS = 1024;
constexpr int NUC_BINS = 2048;
constexpr float MASS_SCALE = 1099511627776.f;      // 2^40

__device__ __forceinline__ unsigned long long mass_of(float s) { return __float2ull_rn(s * MASS_SCALE); }

struct Found {
  unsigned int key;                 // bits of the score at the position
  unsigned long long cum;           // mass of all scores above `key`
  unsigned int cnt;                 // their number
  unsigned int ties, take;          // scores equal to `key`, and how many of them (index order) reach the position
  unsigned long long tie_mass;      // mass of one of them
  int found;                        // 0: no position fulfils the target (it lies beyond the whole vocabulary)
};

// The first position p >= min_pos of the descending order whose running mass is >= target.
__device__ void descend(const float* __restrict__ s, int V, unsigned long long target, unsigned int min_pos,
                        unsigned long long* hm, unsigned int* hc, Found* res) {
  const int tid = threadIdx.x;
  __shared__ unsigned int prefix_s;
  __shared__ unsigned long long cum_s;
  __shared__ unsigned int cnt_s;
  __shared__ int ok_s;
  if (tid == 0) { prefix_s = 0; cum_s = 0; cnt_s = 0; ok_s = 1; }
  __syncthreads();
  for (int level = 0; level < 3; ++level) {
    const int shift = level == 0 ? 21 : (level == 1 ? 10 : 0);
    const int bins = level == 2 ? 1024 : 2048;
    for (int b = tid; b < NUC_BINS; b += NUC_THREADS) { hm[b] = 0; hc[b] = 0; }
    __syncthreads();
    const unsigned int prefix = prefix_s;           // bits above this level's, already fixed
    for (int i = tid; i < V; i += NUC_THREADS) {
      const float v = s[i];
      const unsigned int key = __float_as_uint(v);
      const bool in = level == 0 || (level == 1 ? (key >> 21) == prefix : (key >> 10) == prefix);
      if (in) {
        const unsigned int b = (key >> shift) & (bins - 1);
        atomicAdd(&hm[b], mass_of(v));
        atomicAdd(&hc[b], 1u);
      }
    }
    __syncthreads();
    if (tid == 0 && ok_s) {
      unsigned long long cum = cum_s;
      unsigned int cnt = cnt_s;
      int pick = -1;
      for (int b = bins - 1; b >= 0; --b) {
        if (hc[b] == 0) continue;
        if (cum + hm[b] >= target && cnt + hc[b] >= min_pos) { pick = b; break; }
        cum += hm[b];
        cnt += hc[b];
      }
      if (pick < 0) {
        ok_s = 0;
      } else {
        cum_s = cum;
        cnt_s = cnt;
        prefix_s = level == 2 ? ((prefix << 10) | (unsigned int)pick) : ((prefix << 11) | (unsigned int)pick);
        if (level == 2) {
          res->key = prefix_s;
          res->cum = cum;
          res->cnt = cnt;
          res->ties = hc[pick];
          res->tie_mass = hm[pick] / hc[pick];
          unsigned long long need = 0;
          if (target > cum) need = res->tie_mass ? (target - cum + res->tie_mass - 1) / res->tie_mass : 1;
          unsigned int take = need > (unsigned long long)res->ties ? res->ties : (unsigned int)need;
          if (cnt + take < min_pos) take = min_pos - cnt;
          if (take < 1) take = 1;
          if (take > res->ties) take = res->ties;
          res->take = take;
        }
      }
    }
    __syncthreads();
  }
  if (tid == 0) res->found = ok_s;
  __syncthreads();
}

// params[row] = (temperature, top_p, penalty, u) as doubles; recent[recent_off[row] .. recent_off[row + 1]) are the ids
// whose scores are divided by the penalty; work is [R, V] floats of scratch (the scores).
__global__ void __launch_bounds__(NUC_THREADS) sample_nucleus_kernel(const float* __restrict__ logits, float* __restrict__ work,
                                                                     int V, const double* __restrict__ params,
                                                                     const int* __restrict__ recent,
                                                                     const int* __restrict__ recent_off,
                                                                     int* __restrict__ out) {
  __shared__ unsigned long long hm[NUC_BINS];
  __shared__ unsigned int hc[NUC_BINS];
  __shared__ Found f1, f2;
  __shared__ unsigned long long total_s;
  __shared__ int answer;
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* l = logits + (size_t)row * V;
  float* s = work + (size_t)row * V;
  const double T = params[row * 4 + 0], top_p = params[row * 4 + 1], pen = params[row * 4 + 2], u = params[row * 4 + 3];

  // the first largest logit: threads own contiguous runs, then a tree over (value, index)
  float* fmx = (float*)hm;
  int* fidx = (int*)hc;
  const int per = (V + NUC_THREADS - 1) / NUC_THREADS;
  const int b0 = min(V, tid * per), e0 = min(V, b0 + per);
  float mx = -INFINITY;
  int mi = 0x7fffffff;
  for (int i = b0; i < e0; ++i)
    if (l[i] > mx) { mx = l[i]; mi = i; }
  fmx[tid] = mx;
  fidx[tid] = mi;
  __syncthreads();
  for (int h = NUC_THREADS / 2; h > 0; h >>= 1) {
    if (tid < h) {
      const float o = fmx[tid + h];
      const int oi = fidx[tid + h];
      if (o > fmx[tid] || (o == fmx[tid] && oi < fidx[tid])) { fmx[tid] = o; fidx[tid] = oi; }
    }
    __syncthreads();
  }
  const float top = fmx[0];
  const int top_i = fidx[0] == 0x7fffffff ? 0 : fidx[0];
  __syncthreads();                                   // hm and hc are histograms from here on
  if (T <= 0.0 || V == 1) {
    if (tid == 0) out[row] = top_i;
    return;
  }
  for (int i = tid; i < V; i += NUC_THREADS) s[i] = (float)exp((double)(l[i] - top) / T);
  if (tid == 0) { total_s = 0; answer = V - 1; }
  __syncthreads();
  const int r0 = recent_off[row], rn = recent_off[row + 1] - r0;
  if (pen != 1.0 && pen > 0.0 && rn > 0) {
    const float fp = (float)pen;
    for (int k = tid; k < rn; k += NUC_THREADS) {
      const int id = recent[r0 + k];
      if (id < 0 || id >= V) continue;
      bool first = true;                             // an id is penalised once, by the thread of its first place
      for (int j = 0; j < k; ++j)
        if (recent[r0 + j] == id) { first = false; break; }
      if (first) s[id] = s[id] / fp;
    }
    __syncthreads();
  }
  unsigned long long part = 0;
  for (int i = tid; i < V; i += NUC_THREADS) part += mass_of(s[i]);
  atomicAdd(&total_s, part);
  __syncthreads();
  const unsigned long long total = total_s;

  // the nucleus: first position i > 0 (1-based: >= 2) whose running mass is >= top_p * total
  unsigned long long t1 = 0;
  if (top_p > 0.0) {
    const double want = ceil(top_p * (double)total);
    t1 = want >= 1.8e19 ? 0xffffffffffffffffull : (unsigned long long)want;
  }
  descend(s, V, t1, 2u, hm, hc, &f1);
  const unsigned long long nucleus = f1.found ? f1.cum + (unsigned long long)f1.take * f1.tie_mass : total;

  // the draw: first position whose running mass is >= u * nucleus
  unsigned long long t2 = (unsigned long long)ceil(u * (double)nucleus);
  if (t2 > nucleus) t2 = nucleus;
  descend(s, V, t2, 1u, hm, hc, &f2);
  if (!f2.found) {                                   // (cannot happen: t2 <= nucleus <= total)
    if (tid == 0) out[row] = top_i;
    return;
  }
  // the `take`-th score equal to `key`, in index order
  const unsigned int key = f2.key, take = f2.take;
  unsigned int* cnts = hc;                           // per-thread counts over contiguous runs of the vocabulary
  unsigned int mine = 0;
  for (int i = b0; i < e0; ++i) mine += __float_as_uint(s[i]) == key;
  __syncthreads();
  cnts[tid] = mine;
  __syncthreads();
  if (tid == 0) {                                    // exclusive prefix, serial: a thousand adds
    unsigned int run = 0;
    for (int t = 0; t < NUC_THREADS; ++t) {
      const unsigned int c = cnts[t];
      cnts[t] = run;
      run += c;
    }
  }
  __syncthreads();
  const unsigned int before = cnts[tid];
  if (mine > 0 && before < take && take <= before + mine) {
    unsigned int seen = before;
    for (int i = b0; i < e0; ++i)
      if (__float_as_uint(s[i]) == key && ++seen == take) { answer = i; break; }
  }
  __syncthreads();
  if (tid == 0) out[row] = answer;
}

}  // namespace

// One token per row by the rule above.  `work` holds R * V floats of scratch; `params` R * 4 doubles
// (temperature, top_p, penalty, u); `recent_off` R + 1 offsets into `recent`.
NV_API int nv_sample_nucleus(const float* logits, float* work, int R, int V, const double* params, const int* recent,
                             const int* recent_off, int* out, cudaStream_t s) {
  if (R == 0) return NV_OK;
  if (V < 1) return NV_ERR_BAD_SIZE;
  sample_nucleus_kernel<<<R, NUC_THREADS, 0, s>>>(logits, work, V, params, recent, recent_off, out);
  NV_RETURN_LAST();
}
