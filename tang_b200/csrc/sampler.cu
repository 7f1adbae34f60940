// Sampler::sample of tang-infer on the device (crates/tang-infer/src/sampling.rs:86-158): repetition penalty,
// temperature, softmax numerators, top-k threshold (ties kept), normalisation, top-p (nucleus) filter,
// categorical draw with the reference's 64-bit LCG (sampling.rs:72-79).  One CTA per sequence.
//
// The vocabulary-wide passes (penalty, max, exp, k-th largest by radix selection on the f64 bit patterns)
// are parallel and order-free.  What depends on the ORDER of f64 additions in the reference (the two
// normalising sums, the nucleus' running sum in descending-probability order, the draw's running sum in index
// order) is done in the reference's order by one thread whenever at most kCompact probabilities are still
// non-zero after the top-k filter, which is the usual case (top_k = 40): zeros add exactly nothing, so summing
// the survivors in index order IS the reference's sum.  With more survivors (top_k disabled) the sums are block
// reductions and the nucleus threshold a weighted radix selection: same result unless a running sum lands within
// rounding of a threshold.
#include <cuda_runtime.h>

#include <cmath>

#include "internal.h"

namespace tq {

constexpr int kSamplerThreads = 1024;
constexpr int kCompact = 1024;

struct SamplerParams {
  const float* logits;   // [slices][rows][cols]
  int slices, rows, cols;
  double temperature, top_p, penalty;
  unsigned long long top_k;
  unsigned long long* rng;   // [rows] LCG states, advanced by one step per non-greedy draw
  const int* past;           // [rows][past_ld] or null
  const int* past_lens;      // [rows] or null
  int past_ld;
  double* probs;             // [rows][V] workspace
  int* counts;               // [rows][V] workspace (occurrences in past), only with a penalty
  int* out;                  // [rows]
};

__device__ __forceinline__ double block_max(double v, double* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = red[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); ++i) v = fmax(v, red[i]);
  return v;
}

// fixed-shape tree: the same bits on every run
__device__ __forceinline__ double block_sum(double v, double* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  double s = 0.0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
  return s;
}

__device__ __forceinline__ int block_sum_int(int v, int* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int s = 0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
  return s;
}

// first maximum (strict '>' scan from index 0) of p[0..V)
__device__ int block_argmax_first(const double* p, int V, double* redv, int* redi) {
  double best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x)
    if (p[i] > best) {
      best = p[i];
      bi = i;
    }
  for (int o = 16; o > 0; o >>= 1) {
    const double ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) {
    redv[warp] = best;
    redi[warp] = bi;
  }
  __syncthreads();
  best = redv[0];
  bi = redi[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); ++i)
    if (redv[i] > best || (redv[i] == best && redi[i] < bi)) {
      best = redv[i];
      bi = redi[i];
    }
  return bi == 0x7fffffff ? 0 : bi;
}

__global__ void __launch_bounds__(kSamplerThreads) sampler_kernel(const SamplerParams p) {
  __shared__ double red[32];
  __shared__ int redi[32];
  __shared__ unsigned int hist[256];
  __shared__ double mass[256];
  __shared__ double cp[kCompact];       // surviving probabilities, index order
  __shared__ int ci[kCompact];          // their token ids
  __shared__ int order[kCompact];       // positions of cp[] in descending-probability order
  __shared__ unsigned long long sel_prefix;
  __shared__ unsigned long long sel_k;
  __shared__ double sh_d[2];
  __shared__ int sh_i[2];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int V = p.slices * p.cols;
  double* pr = p.probs + (size_t)row * V;

  // ---- logits as f64, repetition penalty once per occurrence (sampling.rs:91-104)
  int* cnt = nullptr;
  if (p.penalty != 1.0 && p.past && p.past_lens) {
    cnt = p.counts + (size_t)row * V;
    for (int i = tid; i < V; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    const int n_past = p.past_lens[row];
    for (int j = tid; j < n_past; j += blockDim.x) {
      const int t = p.past[(size_t)row * p.past_ld + j];
      if (t >= 0 && t < V) atomicAdd(&cnt[t], 1);
    }
    __syncthreads();
  }
  const bool greedy = p.temperature == 0.0;
  const double inv_t = greedy ? 1.0 : 1.0 / p.temperature;
  double mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) {
    const int sl = i / p.cols, c = i - sl * p.cols;
    double v = (double)p.logits[((size_t)sl * p.rows + row) * p.cols + c];
    if (cnt)
      for (int r = cnt[i]; r > 0; --r) v = v > 0.0 ? v / p.penalty : v * p.penalty;
    if (!greedy && p.temperature != 1.0) v *= inv_t;
    pr[i] = v;
    mx = fmax(mx, v);
  }
  __syncthreads();
  if (greedy) {   // sampling.rs:107-110
    const int best = block_argmax_first(pr, V, red, redi);
    if (tid == 0) p.out[row] = best;
    return;
  }
  mx = block_max(mx, red);
  for (int i = tid; i < V; i += blockDim.x) pr[i] = exp(pr[i] - mx);   // sampling.rs:119-123
  __syncthreads();

  // ---- top-k: everything below the k-th largest value goes to zero (sampling.rs:125-133); radix selection
  // over the bit patterns of the non-negative doubles, most significant byte first
  if (p.top_k > 0 && p.top_k < (unsigned long long)V) {
    if (tid == 0) {
      sel_prefix = 0ull;
      sel_k = p.top_k;
    }
    for (int shift = 56; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0u;
      __syncthreads();
      const unsigned long long prefix = sel_prefix, himask = shift == 56 ? 0ull : (~0ull << (shift + 8));
      for (int i = tid; i < V; i += blockDim.x) {
        const unsigned long long b = (unsigned long long)__double_as_longlong(pr[i]);
        if ((b & himask) == prefix) atomicAdd(&hist[(b >> shift) & 0xFF], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long k = sel_k;
        int d = 255;
        for (; d > 0; --d) {
          if (hist[d] >= k) break;
          k -= hist[d];
        }
        sel_k = k;
        sel_prefix = prefix | ((unsigned long long)d << shift);
      }
      __syncthreads();
    }
    const double thr = __longlong_as_double((long long)sel_prefix);
    for (int i = tid; i < V; i += blockDim.x)
      if (pr[i] < thr) pr[i] = 0.0;
    __syncthreads();
  }

  // ---- how many survive?
  int nz_local = 0;
  const int chunk = (V + blockDim.x - 1) / blockDim.x;            // contiguous index range per thread
  const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
  for (int i = lo; i < hi; ++i) nz_local += pr[i] > 0.0;
  const int nz = block_sum_int(nz_local, redi);

  if (nz <= kCompact) {
    // ---- compact path: the survivors in index order, every order-dependent sum in the reference's order
    // exclusive scan of the per-thread counts (warp scan + warp totals)
    int incl = nz_local;
    const int lane = tid & 31, warp = tid >> 5;
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) redi[warp] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += redi[w];
    int pos = base + incl - nz_local;
    for (int i = lo; i < hi; ++i)
      if (pr[i] > 0.0) {
        cp[pos] = pr[i];
        ci[pos] = i;
        ++pos;
      }
    __syncthreads();
    if (tid == 0) {   // sampling.rs:135-142
      double sum = 0.0;
      for (int j = 0; j < nz; ++j) sum += cp[j];
      sh_d[0] = sum;
    }
    __syncthreads();
    const double sum = sh_d[0];
    if (sum <= 0.0) {   // cannot happen after exp (the maximum maps to 1), kept for the reference's branch
      const int best = block_argmax_first(pr, V, red, redi);
      if (tid == 0) p.out[row] = best;
      return;
    }
    for (int j = tid; j < nz; j += blockDim.x) cp[j] /= sum;
    __syncthreads();
    if (p.top_p < 1.0) {   // sampling.rs:144-153, 196-218
      // descending probability, ascending index among equals (a stable sort): rank by counting
      for (int j = tid; j < nz; j += blockDim.x) {
        int rank = 0;
        const double v = cp[j];
        for (int q = 0; q < nz; ++q) rank += (cp[q] > v) || (cp[q] == v && q < j);
        order[rank] = j;
      }
      __syncthreads();
      if (tid == 0) {
        double cum = 0.0;
        int cutoff = nz;
        for (int r = 0; r < nz; ++r) {
          cum += cp[order[r]];
          if (cum >= p.top_p) {
            cutoff = r + 1;
            break;
          }
        }
        sh_i[0] = cutoff;
      }
      __syncthreads();
      const int cutoff = sh_i[0];
      for (int r = cutoff + tid; r < nz; r += blockDim.x) cp[order[r]] = 0.0;
      __syncthreads();
      if (tid == 0) {
        double s2 = 0.0;
        for (int j = 0; j < nz; ++j) s2 += cp[j];
        sh_d[1] = s2;
      }
      __syncthreads();
      const double s2 = sh_d[1];
      if (s2 > 0.0)
        for (int j = tid; j < nz; j += blockDim.x) cp[j] /= s2;
      __syncthreads();
    }
    if (tid == 0) {   // sampling.rs:161-174 with rand_f64 (:72-79)
      unsigned long long st = p.rng[row] * 6364136223846793005ULL + 1442695040888963407ULL;
      p.rng[row] = st;
      const double r = (double)(st >> 11) / 9007199254740992.0;
      double cum = 0.0;
      int tok = V - 1;
      for (int j = 0; j < nz; ++j) {
        cum += cp[j];
        if (r < cum) {
          tok = ci[j];
          break;
        }
      }
      p.out[row] = tok;
    }
    return;
  }

  // ---- wide path (more than kCompact survivors): block reductions and a weighted radix selection
  {
    double part = 0.0;
    for (int i = lo; i < hi; ++i) part += pr[i];
    const double sum = block_sum(part, red);
    if (sum <= 0.0) {
      const int best = block_argmax_first(pr, V, red, redi);
      if (tid == 0) p.out[row] = best;
      return;
    }
    for (int i = tid; i < V; i += blockDim.x) pr[i] /= sum;
    __syncthreads();
  }
  if (p.top_p < 1.0) {
    // the key K* with mass{key > K*} < top_p <= mass{key >= K*}; ties at K* are admitted in index order until the
    // running sum reaches top_p
    if (tid == 0) {
      sel_prefix = 0ull;
      sh_d[0] = 0.0;   // mass above the current prefix range
    }
    for (int shift = 56; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += blockDim.x) {
        hist[i] = 0u;
        mass[i] = 0.0;
      }
      __syncthreads();
      const unsigned long long prefix = sel_prefix, himask = shift == 56 ? 0ull : (~0ull << (shift + 8));
      for (int i = tid; i < V; i += blockDim.x) {
        const unsigned long long b = (unsigned long long)__double_as_longlong(pr[i]);
        if ((b & himask) == prefix && pr[i] > 0.0) {
          atomicAdd(&hist[(b >> shift) & 0xFF], 1u);
          atomicAdd(&mass[(b >> shift) & 0xFF], pr[i]);
        }
      }
      __syncthreads();
      if (tid == 0) {
        double above = sh_d[0];
        int d = 255;
        for (; d > 0; --d) {
          if (hist[d] && above + mass[d] >= p.top_p) break;
          above += mass[d];
        }
        sh_d[0] = above;
        sel_prefix = prefix | ((unsigned long long)d << shift);
      }
      __syncthreads();
    }
    const double kstar = __longlong_as_double((long long)sel_prefix), above = sh_d[0];
    // ties at K*: admit them in index order while the running sum is still below top_p
    int ties_local = 0;
    for (int i = lo; i < hi; ++i) ties_local += pr[i] == kstar;
    int incl = ties_local;
    const int lane = tid & 31, warp = tid >> 5;
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) redi[warp] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += redi[w];
    if (tid == 0) {
      int total = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += redi[w];
      double cum = above;
      int admit = 0;
      while (admit < total) {
        cum += kstar;
        ++admit;
        if (cum >= p.top_p) break;
      }
      sh_i[0] = kstar > 0.0 ? admit : total;
    }
    __syncthreads();
    const int admit = sh_i[0];
    int tie_rank = base + incl - ties_local;
    double part = 0.0;
    for (int i = lo; i < hi; ++i) {
      double v = pr[i];
      if (v < kstar) v = 0.0;
      else if (v == kstar && tie_rank++ >= admit) v = 0.0;
      pr[i] = v;
      part += v;
    }
    const double s2 = block_sum(part, red);
    if (s2 > 0.0)
      for (int i = lo; i < hi; ++i) pr[i] /= s2;
    __syncthreads();
  }
  // ---- draw: first index whose running sum (index order) exceeds r
  if (tid == 0) {
    unsigned long long st = p.rng[row] * 6364136223846793005ULL + 1442695040888963407ULL;
    p.rng[row] = st;
    sh_d[0] = (double)(st >> 11) / 9007199254740992.0;
  }
  double part = 0.0;
  for (int i = lo; i < hi; ++i) part += pr[i];
  // exclusive scan of the per-thread sums (f64): warp scan, then warp totals in order
  double incl = part;
  {
    const int lane = tid & 31, warp = tid >> 5;
    for (int o = 1; o < 32; o <<= 1) {
      const double t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) red[warp] = incl;
    __syncthreads();
    double base = 0.0;
    for (int w = 0; w < warp; ++w) base += red[w];
    incl += base;
  }
  const double r = sh_d[0];
  int found = 0x7fffffff;
  {
    double cum = incl - part;
    for (int i = lo; i < hi; ++i) {
      cum += pr[i];
      if (r < cum) {
        found = i;
        break;
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) found = min(found, __shfl_xor_sync(0xffffffffu, found, o));
  __syncthreads();
  if ((tid & 31) == 0) redi[tid >> 5] = found;
  __syncthreads();
  if (tid == 0) {
    int best = 0x7fffffff;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) best = min(best, redi[w]);
    p.out[row] = best == 0x7fffffff ? V - 1 : best;
  }
}

}  // namespace tq

using namespace tq;

extern "C" {

int tq_sample(tq_ctx* ctx, const float* logits_dev, size_t slices, size_t rows, size_t cols, const tq_sampler_config* cfg,
              unsigned long long* rng_states_dev, const int* past_tokens_dev, const int* past_lens_dev, size_t past_ld,
              int* tokens_out_dev) {
  if (int st = bind(ctx)) return st;
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(ctx, logits_dev && cfg && tokens_out_dev && slices > 0 && cols > 0, "tq_sample: null pointer or empty vocabulary");
  TQ_REQUIRE(ctx, slices * cols < (1ull << 31), "tq_sample: vocabulary too large");
  TQ_REQUIRE(ctx, cfg->temperature >= 0.0 && cfg->repetition_penalty > 0.0, "tq_sample: temperature >= 0 and penalty > 0 required");
  TQ_REQUIRE(ctx, cfg->temperature == 0.0 || rng_states_dev != nullptr, "tq_sample: sampling needs the LCG states");
  const size_t V = slices * cols;
  const bool penal = cfg->repetition_penalty != 1.0 && past_tokens_dev && past_lens_dev;
  const size_t bytes = rows * V * sizeof(double) + (penal ? rows * V * sizeof(int) : 0);
  if (int st = ensure_scratch(ctx, bytes)) return st;
  SamplerParams p;
  p.logits = logits_dev;
  p.slices = (int)slices;
  p.rows = (int)rows;
  p.cols = (int)cols;
  p.temperature = cfg->temperature;
  p.top_p = cfg->top_p;
  p.penalty = cfg->repetition_penalty;
  p.top_k = cfg->top_k;
  p.rng = rng_states_dev;
  p.past = past_tokens_dev;
  p.past_lens = past_lens_dev;
  p.past_ld = (int)past_ld;
  p.probs = static_cast<double*>(ctx->scratch);
  p.counts = penal ? reinterpret_cast<int*>(static_cast<char*>(ctx->scratch) + rows * V * sizeof(double)) : nullptr;
  p.out = tokens_out_dev;
  sampler_kernel<<<(unsigned)rows, kSamplerThreads, 0, ctx->stream>>>(p);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

}  // extern "C"
