// Mixture-of-experts FFN layer (include/tangq.h, tq_moe_*).  The reference has no MoE; the layer is
// composed in the reference's idiom from its primitives: the quantised matvec
// (crates/tang-infer/src/quantize.rs:256-289) per expert, SwiGLU (crates/tang-compute/src/device.rs:
// 727-736), a max-subtracted softmax (crates/tang-infer/src/sampling.rs:119-123) and an exactly-k
// selection whose tie rule (larger logit first, lower index among equals) completes what
// sampling.rs:126-133,176-181 leaves open.
//
// Pipeline for T tokens:  router (f64 logits, top-k, softmax weights)  ->  count / offset / slot
// assignment per expert  ->  gather token rows into expert order  ->  grouped gate|up GEMM  ->
// SwiGLU  ->  grouped down GEMM  ->  weighted scatter-add per token (+ shared experts, dense).
#include <cuda_bf16.h>

#include <new>
#include <vector>

#include "common.cuh"
#include "internal.h"

struct tq_comm;
extern "C" int tq_all_reduce_f32(tq_ctx*, tq_comm*, float*, size_t);

namespace tq {

int launch_qgemm_grouped(tq_ctx* ctx, const tq_qweight* w, int n_groups, const void* x_bf16, size_t ldx, int mx,
                         const int* counts, const int* offsets, int max_rows, long long x_stride, long long y_stride,
                         void* y, int y_dtype, size_t ldy, const int* active = nullptr,
                         int max_active = 0, size_t total_rows = 0);

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 16;

int all_to_all_v(tq_ctx* ctx, tq_comm* comm, const void* send_dev, const size_t* send_off, const size_t* send_bytes, void* recv_dev,
                 const size_t* recv_off, const size_t* recv_bytes);
int launch_qgemm_umma_grouped(tq_ctx* ctx, const tq_qweight* w, int n_groups, const void* x_bf16, size_t ldx, size_t m_total,
                              const int* counts, const int* offsets, const int* active, int max_active, int max_rows,
                              int expected_rows, void* y, int y_dtype, size_t ldy);
bool umma_grouped_supported(const tq_qweight* w, int n_groups);

// One CTA of eight warps per token; warp w computes the logits of experts w, w + 8, ...
// The reference order is one f64 addition per k, ascending, of products that are exact in f64 (bf16 x
// bf16).  A warp-parallel sum gives the SAME BITS whenever no addition can round, whatever the order:
// every product is a multiple of q = 2^qexp and the sum of |products| stays below 2^53 q, so every
// partial sum of every subset is an integer below 2^53 times q: exactly representable.  The warp certifies this from the exponents
// (qexp = min over non-zero products of the operands' unit-in-the-last-place exponents, sum |p| with
// a factor two of slack); an expert that fails the test is redone by one lane in the reference order.
__device__ __forceinline__ int bf16_ulp_exp(unsigned short bits) {   // value is a multiple of 2^this
  const int e = (bits >> 7) & 0xFF;
  return (e ? e : 1) - 127 - 7;
}

// 16-bit halves: the unit-in-the-last-place exponent (biased by 134) of each bf16 of a pair, or 0x2000 for a zero
// (a product with a zero operand is zero and does not enter the minimum).
__device__ __forceinline__ unsigned bf16x2_ulp_code(unsigned pair) {
  const unsigned e = (pair >> 7) & 0x00FF00FFu;
  unsigned lo = e & 0xFFFFu, hi = e >> 16;
  lo = (pair & 0x7FFFu) == 0u ? 0x2000u : (lo ? lo : 1u);
  hi = (pair & 0x7FFF0000u) == 0u ? 0x2000u : (hi ? hi : 1u);
  return lo | (hi << 16);
}

// A gate row times a token in the reference order (one f64 addition per k, ascending), for rows whose additions may
// round; called by a whole warp, every lane returns the sum.
__device__ __noinline__ double router_ordered_sum(const unsigned short* hrow_s, const unsigned short* wrow, int d, int lane) {
  // The reference order, without adding 2048 numbers one after the other.  Lane c takes the c-th run of
  // consecutive k: its sum from zero in order, the sum of the magnitudes and the smallest ulp code.  Then the runs
  // are joined in order: while the running sum s is a multiple of 2^qs, a run whose partial sums s + prefix all
  // stay below 2^53 units of 2^min(qs, its own) adds without any rounding, so its sum is added in one step; a run
  // that fails this is added term by term (by every lane alike), after which s is only known to be a multiple
  // of its own last place.  Typically one run holds the offending tiny product.
  const int CH = ((d + 255) >> 8) << 3;                   // terms per run, a multiple of eight
  auto products = [&](int k0, double (&pr)[8], unsigned& code) {
    const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k0), hv = *reinterpret_cast<const uint4*>(hrow_s + k0);
    const unsigned ww[4] = {wv.x, wv.y, wv.z, wv.w}, hh[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pr[2 * j] = (double)__uint_as_float(hh[j] << 16) * (double)__uint_as_float(ww[j] << 16);
      pr[2 * j + 1] = (double)__uint_as_float(hh[j] & 0xFFFF0000u) * (double)__uint_as_float(ww[j] & 0xFFFF0000u);
      code = __viaddmin_u16x2(bf16x2_ulp_code(hh[j]), bf16x2_ulp_code(ww[j]), code);
    }
  };
  double cs = 0.0, ca = 0.0;
  unsigned cq2 = 0xFFFFFFFFu;
  for (int k0 = lane * CH; k0 < min(d, (lane + 1) * CH); k0 += 8) {
    double pr[8];
    products(k0, pr, cq2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      cs += pr[j];
      ca += fabs(pr[j]);
    }
  }
  const unsigned cq = min(cq2 & 0xFFFFu, cq2 >> 16);
  constexpr int kAny = 1 << 20;                           // "a multiple of anything": s is zero
  double sr = 0.0;
  int qs = kAny;
  for (int c = 0; c < 32; ++c) {
    const double cs_c = __shfl_sync(0xffffffffu, cs, c), ca_c = __shfl_sync(0xffffffffu, ca, c);
    const unsigned cq_c = __shfl_sync(0xffffffffu, cq, c);
    if (c * CH >= d || cq_c >= 0x2000u) continue;         // nothing there, or zeros only: s + 0 = s
    const int qq = min(qs, (int)cq_c - 268);
    // integer multiples of 2^qq up to 2^53 of them are representable; the left side is an upper bound up to
    // the rounding of its own additions, which the factor covers (false for NaN and infinity)
    if ((fabs(sr) + ca_c) * (1.0 + 0x1p-30) < ldexp(1.0, 53 + qq)) {
      sr += cs_c;
      qs = sr == 0.0 ? kAny : qq;
    } else {
      for (int k0 = c * CH; k0 < min(d, (c + 1) * CH); k0 += 8) {
        double pr[8];
        unsigned unused = 0xFFFFFFFFu;
        products(k0, pr, unused);
#pragma unroll
        for (int j = 0; j < 8; ++j) sr += pr[j];
      }
      qs = sr == 0.0 ? kAny : (sr == sr && fabs(sr) < 1.7e308 ? ilogb(sr) - 52 : -(1 << 20));
    }
  }
  return sr;
}

// TT tokens per CTA share every load of a gate row (many tokens: the rows then come from L2 once per TT tokens).
template <int TT>
__global__ void __launch_bounds__(256, 4) router_kernel(const __nv_bfloat16* h, const __nv_bfloat16* wg, int T, int d, int E,
                                                     int top_k, int renorm, int* idx_out, float* w_out, double* logits_out, int* counters) {
  extern __shared__ __align__(16) unsigned short hs[];   // [TT][d] activations (bf16 bits), then [TT][d] their ulp codes
  __shared__ double lg[TT][kMaxExperts];
  unsigned short* he = hs + (size_t)TT * d;
  const int t0 = blockIdx.x * TT, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = 2 * threadIdx.x; i < TT * d; i += 2 * blockDim.x) {
    const int tt = i / d, t = t0 + tt;
    const unsigned pair = t < T ? *reinterpret_cast<const unsigned*>(reinterpret_cast<const unsigned short*>(h) + (size_t)t0 * d + i) : 0u;
    *reinterpret_cast<unsigned*>(hs + i) = pair;
    *reinterpret_cast<unsigned*>(he + i) = bf16x2_ulp_code(pair);
  }
  __syncthreads();
  // gridDim.y CTAs share a token's experts (few tokens would otherwise occupy few SMs); the CTA that
  // finishes last (counter) reads all logits back and makes the selection
  for (int e = blockIdx.y * 8 + warp; e < E; e += 8 * gridDim.y) {
    const unsigned short* wrow = reinterpret_cast<const unsigned short*>(wg) + (size_t)e * d;
    double acc[TT];
    float sabs[TT];
    unsigned qm[TT];           // per 16-bit half: the smallest sum of ulp codes over the non-zero products so far
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      acc[tt] = 0.0;
      sabs[tt] = 0.f;
      qm[tt] = 0xFFFFFFFFu;
    }
    // eight consecutive k per lane and load (d is a multiple of 8: checked by the host)
#pragma unroll 2
    for (int k0 = 8 * lane; k0 < d; k0 += 256) {
      const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k0);
      const unsigned ww[4] = {wv.x, wv.y, wv.z, wv.w};
      float wl[4], wh[4];
      unsigned wc[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        wl[j] = __uint_as_float(ww[j] << 16);
        wh[j] = __uint_as_float(ww[j] & 0xFFFF0000u);
        wc[j] = bf16x2_ulp_code(ww[j]);
      }
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) {
        const uint4 hv = *reinterpret_cast<const uint4*>(hs + (size_t)tt * d + k0);
        const uint4 cv = *reinterpret_cast<const uint4*>(he + (size_t)tt * d + k0);
        const unsigned hh[4] = {hv.x, hv.y, hv.z, hv.w}, hc[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = __uint_as_float(hh[j] << 16) * wl[j];          // 16 significant bits: exact
          const float p1 = __uint_as_float(hh[j] & 0xFFFF0000u) * wh[j];
          acc[tt] += (double)p0;
          acc[tt] += (double)p1;
          sabs[tt] += fabsf(p0) + fabsf(p1);   // a bound only (rounded f32 sum; the test below leaves a factor of two)
          qm[tt] = __viaddmin_u16x2(hc[j], wc[j], qm[tt]);
        }
      }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      unsigned q = min(qm[tt] & 0xFFFFu, qm[tt] >> 16);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], o);
        sabs[tt] += __shfl_xor_sync(0xffffffffu, sabs[tt], o);
        q = min(q, __shfl_xor_sync(0xffffffffu, q, o));
      }
      // every non-zero product is a multiple of 2^(q - 268); none at all: the sum is zero.  NaN or infinity anywhere,
      // or a product that underflowed in f32, fails the comparison and takes the reference order as well
      // (q < 140: some product lies below the normal range of f32, where p0 / p1 above are no longer exact)
      const bool exact = q >= 0x2000u || (q >= 140u && (double)sabs[tt] < ldexp(1.0, 52 + (int)q - 268));
      if (!exact) acc[tt] = router_ordered_sum(hs + (size_t)tt * d, wrow, d, lane);
      if (lane == 0 && t0 + tt < T) {
        lg[tt][e] = acc[tt];
        if (logits_out) logits_out[(size_t)(t0 + tt) * E + e] = acc[tt];
      }
    }
  }
  if (gridDim.y > 1) {
    __shared__ int last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      last = atomicAdd(&counters[blockIdx.x], 1) == (int)gridDim.y - 1;
      if (last) counters[blockIdx.x] = 0;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int i = threadIdx.x; i < TT * E; i += blockDim.x)
      if (t0 + i / E < T) lg[i / E][i % E] = __ldcg(logits_out + (size_t)t0 * E + i);
  }
  __syncthreads();
  for (int tt = 0; tt < TT && t0 + tt < T; ++tt) {
  const int t = t0 + tt;
  const double* lgt = lg[tt];
  // softmax terms in parallel (one f64 exp per thread), their sum in index order by one thread; the maximum and
  // the top-k selection by the first warp (lane l owns experts l, l + 32, ...): the rule is "highest logit first,
  // lowest index on ties, exactly top_k", which a (value, index) tournament reproduces for ordered values.  A NaN
  // logit has no order; then one thread runs the comparison loop as written.
  __shared__ double ex[kMaxExperts];
  __shared__ double mx_s;
  __shared__ int pick[kMaxTopK];
  if (warp == 0) {
    double mx = lgt[0];
    bool any_nan = false;
    for (int i = lane; i < E; i += 32) {
      mx = fmax(mx, lgt[i]);
      any_nan |= lgt[i] != lgt[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    any_nan = __any_sync(0xffffffffu, any_nan);
    if (lane == 0) mx_s = mx;
    if (!any_nan) {
      unsigned taken = 0;                                  // bit j: expert lane + 32 j is chosen
      for (int s = 0; s < top_k; ++s) {
        double bv = 0.0;
        int bi = -1;
        for (int j = 0, i = lane; i < E; ++j, i += 32)
          if (!((taken >> j) & 1u) && (bi < 0 || lgt[i] > bv)) {   // ascending i: '>' keeps the lower index
            bv = lgt[i];
            bi = i;
          }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const double ov = __shfl_xor_sync(0xffffffffu, bv, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) {
            bv = ov;
            bi = oi;
          }
        }
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (lane == 0) pick[s] = bi;
      }
    } else if (lane == 0) {
      unsigned long long taken[kMaxExperts / 64] = {0, 0, 0, 0};
      for (int s = 0; s < top_k; ++s) {
        int best = -1;
        for (int i = 0; i < E; ++i) {
          if ((taken[i >> 6] >> (i & 63)) & 1ull) continue;
          if (best < 0 || lgt[i] > lgt[best]) best = i;   // strict '>' keeps the lower index on ties
        }
        taken[best >> 6] |= 1ull << (best & 63);
        pick[s] = best;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) ex[i] = exp(lgt[i] - mx_s);
  __syncthreads();
  if (threadIdx.x == 0) {
    double sum = 0.0;
    for (int i = 0; i < E; ++i) sum += ex[i];
    double chosen = 0.0;
    double pw[kMaxTopK];
    for (int s = 0; s < top_k; ++s) {
      pw[s] = ex[pick[s]] / sum;
      chosen += pw[s];
    }
    for (int s = 0; s < top_k; ++s) {
      idx_out[(size_t)t * top_k + s] = pick[s];
      w_out[(size_t)t * top_k + s] = (float)(renorm ? pw[s] / chosen : pw[s]);
    }
  }
  __syncthreads();   // (the selection arrays are reused by the next token)
  }
}

// counts[e] = rows routed to expert e (a single CTA; T*top_k entries).
__global__ void moe_count_kernel(const int* idx, int n, int E, int* counts, int* offsets, int* cursor, int* active,
                                 int n_listed) {
  __shared__ int c[kMaxExperts];
  for (int i = threadIdx.x; i < E; i += blockDim.x) c[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&c[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      counts[e] = c[e];
      offsets[e] = run;
      cursor[e] = run;
      run += c[e];
    }
    int j = 0;                                   // ids of the first n_listed groups that received rows, then -1s
    for (int e = 0; e < n_listed; ++e)
      if (c[e] > 0) active[j++] = e;
    for (; j < n_listed; ++j) active[j] = -1;
  }
}

// slot[i] = row of (token, choice) i in expert order; rows of one expert keep no particular order
// (they are independent), results are scattered back through slot[].
__global__ void moe_slot_kernel(const int* idx, int n, int* cursor, int* slot) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) slot[i] = atomicAdd(&cursor[idx[i]], 1);
}

__global__ void moe_gather_kernel(const __nv_bfloat16* h, const int* slot, int n, int top_k, int d, __nv_bfloat16* xs) {
  const int i = blockIdx.x;   // (token, choice)
  const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(i / top_k) * d);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)slot[i] * d);
  for (int v = threadIdx.x; v < d / 8; v += blockDim.x) dst[v] = src[v];
}

// out[t, :] = sum_s w[t,s] * yo[slot[t,s], :] (+ shared[t, :])
__global__ void moe_combine_kernel(const float* yo, const int* slot, const float* w, const float* shared, int top_k, int d,
                                   float* out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < top_k; ++s) acc += w[(size_t)t * top_k + s] * yo[(size_t)slot[(size_t)t * top_k + s] * d + c];
    if (shared) acc += shared[(size_t)t * d + c];
    out[(size_t)t * d + c] = acc;
  }
}

// ---- expert parallelism with token dispatch (tokens sharded over ranks) ----------------------------
// Every (token, choice) pair of this rank gets a place in the block of the send buffer that goes to the
// expert's owner: place = owner * cap + (running count for that owner).  meta[] carries the owner's local
// expert id, -1 marks padding.  Which pair gets which place within a block is not fixed (atomic counter),
// but every row is processed on its own and its result comes back to the same place, so outputs do not
// depend on it.
__global__ void moe_dispatch_plan_kernel(const int* idx, int n, int n_local, int world, int cap, int* place, int* send_meta,
                                         int* send_cnt) {
  __shared__ int cnt[64];
  for (int i = threadIdx.x; i < world; i += blockDim.x) cnt[i] = 0;
  for (int i = threadIdx.x; i < world * cap; i += blockDim.x) send_meta[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int owner = idx[i] / n_local;
    const int pos = atomicAdd(&cnt[owner], 1);
    place[i] = owner * cap + pos;
    send_meta[owner * cap + pos] = idx[i] - owner * n_local;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < world; i += blockDim.x) send_cnt[i] = cnt[i];   // rows for every owner
}

__global__ void moe_dispatch_rows_kernel(const __nv_bfloat16* h, const int* place, int top_k, int d, __nv_bfloat16* send_x) {
  const int i = blockIdx.x;   // (token, choice)
  const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(i / top_k) * d);
  uint4* dst = reinterpret_cast<uint4*>(send_x + (size_t)place[i] * d);
  for (int v = threadIdx.x; v < d / 8; v += blockDim.x) dst[v] = src[v];
}

// received meta (-1 = padding) -> bucket ids for the count/slot kernels (padding goes to bucket n_local)
__global__ void moe_recv_bucket_kernel(const int* meta, int n, int n_local, int* bucket) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) bucket[i] = meta[i] < 0 ? n_local : meta[i];
}

__global__ void moe_gather_recv_kernel(const __nv_bfloat16* recv_x, const int* bucket, const int* slot, int n_local, int d,
                                       __nv_bfloat16* xs) {
  const int i = blockIdx.x;
  if (bucket[i] >= n_local) return;
  const uint4* src = reinterpret_cast<const uint4*>(recv_x + (size_t)i * d);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)slot[i] * d);
  for (int v = threadIdx.x; v < d / 8; v += blockDim.x) dst[v] = src[v];
}

// expert-order results -> the order the rows arrived in (padding rows are left untouched: nobody reads them)
__global__ void moe_scatter_back_kernel(const float* yo, const int* bucket, const int* slot, int n_local, int d, float* back) {
  const int i = blockIdx.x;
  if (bucket[i] >= n_local) return;
  const float4* src = reinterpret_cast<const float4*>(yo + (size_t)slot[i] * d);
  float4* dst = reinterpret_cast<float4*>(back + (size_t)i * d);
  for (int v = threadIdx.x; v < d / 4; v += blockDim.x) dst[v] = src[v];
}

}  // namespace tq

struct tq_moe {
  tq_ctx* ctx = nullptr;
  tq_moe_config cfg{};
  const void* wg = nullptr;                 // bf16 [n_experts, d_model]
  const tq_qweight* w_gate_up = nullptr;    // stacked [n_local * 2*ffn, d_model]
  const tq_qweight* w_down = nullptr;       // stacked [n_local * d_model, ffn]
  std::vector<const tq_qweight*> sh_gate_up, sh_down;
  int expert_lo = 0, n_local = 0;           // experts held by this rank
  int* host_counts = nullptr;               // pinned [2][64]: rows per peer, sent and received (counts-first dispatch)
};

using namespace tq;

extern "C" {

// logits_ws: [n_tokens][n_experts] f64 that the kernel may use to share logits between the CTAs of a token
// (null: one CTA per token).
static int launch_router(tq_ctx* ctx, const void* h_bf16_dev, const void* wg_bf16_dev, size_t n_tokens, size_t d_model,
                         size_t n_experts, size_t top_k, int renormalize, int* idx_out_dev, float* weight_out_dev,
                         double* logits_ws) {
  TQ_REQUIRE(ctx, n_experts > 0 && n_experts <= kMaxExperts && top_k > 0 && top_k <= kMaxTopK && top_k <= n_experts,
             "tq_moe_router: need 1 <= top_k <= n_experts <= %d and top_k <= %d", kMaxExperts, kMaxTopK);
  if (n_tokens == 0) return TQ_OK;
  TQ_REQUIRE(ctx, h_bf16_dev && wg_bf16_dev && idx_out_dev && weight_out_dev, "tq_moe_router: null pointer");
  TQ_REQUIRE(ctx, d_model <= 24576 && d_model % 8 == 0 && ((uintptr_t)h_bf16_dev & 15) == 0 && ((uintptr_t)wg_bf16_dev & 15) == 0,
             "tq_moe_router: d_model must be a multiple of 8 and at most 24576, arrays 16-byte aligned");
  unsigned gy = 1;
  if (logits_ws && n_tokens <= 64 && n_tokens <= (size_t)kTileCounters) gy = (unsigned)((n_experts + 7) / 8);
  // four tokens per CTA once there are several waves of CTAs anyway (their activations and ulp codes: 16 d bytes;
  // measured alone at 1000 / 2048 tokens: 154 / 209 us against 119 / 206 us with one token per CTA)
  const bool four = n_tokens >= 2048 && 16 * d_model <= 64 * 1024;
  const size_t smem = (four ? 4 : 1) * d_model * 2 * sizeof(unsigned short);
  auto kern = four ? router_kernel<4> : router_kernel<1>;
  if (smem > 48 * 1024) TQ_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3((unsigned)((n_tokens + (four ? 3 : 0)) / (four ? 4 : 1)), gy), 256, smem, ctx->stream>>>(
      static_cast<const __nv_bfloat16*>(h_bf16_dev), static_cast<const __nv_bfloat16*>(wg_bf16_dev), (int)n_tokens,
      (int)d_model, (int)n_experts, (int)top_k, renormalize, idx_out_dev, weight_out_dev, logits_ws, ctx->dev_err + 1);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

int tq_moe_router(tq_ctx* ctx, const void* h_bf16_dev, const void* wg_bf16_dev, size_t n_tokens, size_t d_model,
                  size_t n_experts, size_t top_k, int renormalize, int* idx_out_dev, float* weight_out_dev,
                  double* logits_out_dev) {
  if (int st = bind(ctx)) return st;
  return launch_router(ctx, h_bf16_dev, wg_bf16_dev, n_tokens, d_model, n_experts, top_k, renormalize, idx_out_dev,
                       weight_out_dev, logits_out_dev);
}

int tq_moe_create(tq_ctx* ctx, const tq_moe_config* cfg, const void* wg_bf16_dev, const tq_qweight* w_gate_up_stacked,
                  const tq_qweight* w_down_stacked, const tq_qweight* const* shared_gate_up,
                  const tq_qweight* const* shared_down, tq_moe** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, cfg && out && wg_bf16_dev && w_gate_up_stacked && w_down_stacked, "tq_moe_create: null argument");
  *out = nullptr;
  TQ_REQUIRE(ctx, cfg->n_experts > 0 && cfg->n_experts <= (uint32_t)kMaxExperts && cfg->top_k > 0 && cfg->top_k <= (uint32_t)kMaxTopK,
             "tq_moe_create: bad expert / top_k count");
  TQ_REQUIRE(ctx, cfg->ep_size >= 1 && cfg->n_experts % cfg->ep_size == 0 && cfg->ep_rank < cfg->ep_size,
             "tq_moe_create: experts must divide by the expert-parallel size");
  const uint32_t n_local = cfg->n_experts / cfg->ep_size;
  TQ_REQUIRE(ctx, cfg->d_model % 128 == 0 && cfg->ffn % 128 == 0, "tq_moe_create: d_model and ffn must be multiples of 128");
  TQ_REQUIRE(ctx, w_gate_up_stacked->rows == (size_t)n_local * 2 * cfg->ffn && w_gate_up_stacked->cols == cfg->d_model,
             "tq_moe_create: stacked gate|up must be [%u * 2*%u, %u]", n_local, cfg->ffn, cfg->d_model);
  TQ_REQUIRE(ctx, w_down_stacked->rows == (size_t)n_local * cfg->d_model && w_down_stacked->cols == cfg->ffn,
             "tq_moe_create: stacked down must be [%u * %u, %u]", n_local, cfg->d_model, cfg->ffn);
  tq_moe* m = new (std::nothrow) tq_moe();
  if (!m) return fail(ctx, TQ_ENOMEM, "out of host memory");
  m->ctx = ctx;
  m->cfg = *cfg;
  m->wg = wg_bf16_dev;
  m->w_gate_up = w_gate_up_stacked;
  m->w_down = w_down_stacked;
  m->n_local = (int)n_local;
  m->expert_lo = (int)(cfg->ep_rank * n_local);
  for (uint32_t i = 0; i < cfg->n_shared; ++i) {
    if (!shared_gate_up || !shared_down || !shared_gate_up[i] || !shared_down[i]) {
      delete m;
      return fail(ctx, TQ_EINVAL, "tq_moe_create: missing shared expert %u", i);
    }
    m->sh_gate_up.push_back(shared_gate_up[i]);
    m->sh_down.push_back(shared_down[i]);
  }
  *out = m;
  return TQ_OK;
}

// Maps global expert ids to this rank's local ids; experts held elsewhere go to the dump group n_local.
__global__ void moe_localize_kernel(const int* idx, int n, int lo, int n_local, int* idx_local) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int e = idx[i] - lo;
    idx_local[i] = (e >= 0 && e < n_local) ? e : n_local;
  }
}

__global__ void moe_combine_local_kernel(const float* yo, const int* slot, const int* idx_local, const float* w,
                                         const float* shared, int n_shared, size_t shared_stride, int shared_lo, int shared_hi,
                                         int top_k, int d, int n_local, float* out) {
  // the token's few (row, weight) pairs first, then wide independent loads over the model dimension
  __shared__ int rows[kMaxTopK];
  __shared__ float wts[kMaxTopK];
  const int t = blockIdx.x;
  if (threadIdx.x < top_k) {
    const size_t i = (size_t)t * top_k + threadIdx.x;
    const bool local = idx_local[i] < n_local;
    rows[threadIdx.x] = local ? slot[i] : -1;
    wts[threadIdx.x] = local ? w[i] : 0.f;
  }
  __syncthreads();
  const bool add_shared = shared && t >= shared_lo && t < shared_hi;
  for (int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x); c < d; c += 4 * gridDim.y * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < top_k; ++s) {
      if (rows[s] < 0) continue;
      const float4 v = *reinterpret_cast<const float4*>(yo + (size_t)rows[s] * d + c);
      acc.x += wts[s] * v.x;
      acc.y += wts[s] * v.y;
      acc.z += wts[s] * v.z;
      acc.w += wts[s] * v.w;
    }
    if (add_shared) {
      // the shared experts' outputs, one buffer each (so that each down projection may run on the tensor-core
      // path, which takes no residual input), summed first in expert order
      float4 v = *reinterpret_cast<const float4*>(shared + (size_t)(t - shared_lo) * d + c);
      for (int e = 1; e < n_shared; ++e) {
        const float4 u = *reinterpret_cast<const float4*>(shared + e * shared_stride + (size_t)(t - shared_lo) * d + c);
        v.x = u.x + v.x;
        v.y = u.y + v.y;
        v.z = u.z + v.z;
        v.w = u.w + v.w;
      }
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)t * d + c) = acc;
  }
}

int tq_moe_ffn(tq_moe* m, const void* h_bf16_dev, size_t n_tokens, float* out_dev, tq_comm* comm, int* idx_out_dev,
               float* weight_out_dev) {
  if (!m) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  if (int st = bind(ctx)) return st;
  if (n_tokens == 0) return TQ_OK;
  TQ_REQUIRE(ctx, h_bf16_dev && out_dev, "tq_moe_ffn: null pointer");
  TQ_REQUIRE(ctx, ((uintptr_t)h_bf16_dev & 15) == 0, "tq_moe_ffn: activations must be 16-byte aligned");
  const tq_moe_config& c = m->cfg;
  const size_t T = n_tokens, k = c.top_k, d = c.d_model, f = c.ffn, n = T * k;
  const int nl = m->n_local;
  // shared experts: this rank serves a contiguous slice of the tokens
  const size_t sh_lo = c.n_shared ? T * c.ep_rank / c.ep_size : 0, sh_hi = c.n_shared ? T * (c.ep_rank + 1) / c.ep_size : 0;
  const size_t Ts = sh_hi - sh_lo;
  auto up = [](size_t b) { return (b + 255) / 256 * 256; };
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += up(bytes);
    return o;
  };
  const size_t o_idx = take(n * 4), o_idl = take(n * 4), o_w = take(n * 4), o_slot = take(n * 4), o_cnt = take((nl + 1) * 4),
               o_off = take((nl + 1) * 4), o_cur = take((nl + 1) * 4), o_act_list = take((nl + 1) * 4), o_lg = take(T * c.n_experts * 8), o_xs = take(n * d * 2), o_gu = take(n * 2 * f * 4),
               o_act = take(n * f * 2), o_yo = take(n * d * 4), o_sh = take((size_t)(c.n_shared ? c.n_shared : 1) * Ts * d * 4), o_shgu = take(Ts * 2 * f * 4),
               o_shact = take(Ts * f * 2);
  if (int st = ensure_scratch(ctx, off)) return st;
  uint8_t* s = static_cast<uint8_t*>(ctx->scratch);
  int* idx = reinterpret_cast<int*>(s + o_idx);
  int* idl = reinterpret_cast<int*>(s + o_idl);
  float* w = reinterpret_cast<float*>(s + o_w);
  int* slot = reinterpret_cast<int*>(s + o_slot);
  int *cnt = reinterpret_cast<int*>(s + o_cnt), *offs = reinterpret_cast<int*>(s + o_off), *cur = reinterpret_cast<int*>(s + o_cur);
  int* active = reinterpret_cast<int*>(s + o_act_list);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(s + o_xs);
  float* gu = reinterpret_cast<float*>(s + o_gu);
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(s + o_act);
  float* yo = reinterpret_cast<float*>(s + o_yo);
  float* sh = reinterpret_cast<float*>(s + o_sh);
  float* shgu = reinterpret_cast<float*>(s + o_shgu);
  __nv_bfloat16* shact = reinterpret_cast<__nv_bfloat16*>(s + o_shact);
  const __nv_bfloat16* h = static_cast<const __nv_bfloat16*>(h_bf16_dev);
  int st;
#define TQ_STEP(expr) \
  if ((st = (expr)) != TQ_OK) return st;
#define TQ_LAUNCHED()   \
  ctx->launches++;      \
  TQ_CUDA(ctx, cudaGetLastError());

  TQ_STEP(launch_router(ctx, h, m->wg, T, d, c.n_experts, k, c.renormalize, idx, w, reinterpret_cast<double*>(s + o_lg)));
  moe_localize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(idx, (int)n, m->expert_lo, nl, idl);
  TQ_LAUNCHED();
  moe_count_kernel<<<1, 1024, 0, ctx->stream>>>(idl, (int)n, nl + 1, cnt, offs, cur, active, nl);
  TQ_LAUNCHED();
  moe_slot_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(idl, (int)n, cur, slot);
  TQ_LAUNCHED();
  moe_gather_kernel<<<(unsigned)n, 128, 0, ctx->stream>>>(h, slot, (int)n, (int)k, (int)d, xs);
  TQ_LAUNCHED();
  // a token picks an expert at most once (counts[e] <= T); the chunk of rows one CTA takes follows the
  // expected rows per expert (T k / E), so that small batches do not pay for 64-row tiles
  size_t want = 2 * n / (size_t)c.n_experts + 1;
  int cap = 8;
  while (cap < 64 && (size_t)cap < want) cap <<= 1;
  if ((size_t)cap > T) cap = (int)T;
  const int max_active = (int)(n < (size_t)nl ? n : (size_t)nl);   // at most one expert per (token, choice)
  // from about 24 rows per expert on, the expert GEMMs run on the tcgen05 kernel (one launch over all experts)
  const size_t expected = n / (size_t)c.n_experts;
  const bool tensor_path = expected >= 24 && umma_grouped_supported(m->w_gate_up, nl) && umma_grouped_supported(m->w_down, nl);
  if (tensor_path) {
    TQ_STEP(launch_qgemm_umma_grouped(ctx, m->w_gate_up, nl, xs, d, n, cnt, offs, active, max_active, (int)T, (int)(expected * 3 / 2),
                                      gu, TQ_F32, 2 * f));
  } else {
    TQ_STEP(launch_qgemm_grouped(ctx, m->w_gate_up, nl, xs, d, cap, cnt, offs, (int)T, 0, 0, gu, TQ_F32, 2 * f, active, max_active, n));
  }
  TQ_STEP(tq_swiglu(ctx, gu, gu + f, TQ_F32, 2 * f, n, f, act, TQ_BF16));
  if (tensor_path) {
    TQ_STEP(launch_qgemm_umma_grouped(ctx, m->w_down, nl, act, f, n, cnt, offs, active, max_active, (int)T, (int)(expected * 3 / 2), yo,
                                      TQ_F32, d));
  } else {
    TQ_STEP(launch_qgemm_grouped(ctx, m->w_down, nl, act, f, cap, cnt, offs, (int)T, 0, 0, yo, TQ_F32, d, active, max_active, n));
  }
  for (size_t i = 0; i < m->sh_gate_up.size() && Ts > 0; ++i) {
    TQ_STEP(tq_qlinear(ctx, m->sh_gate_up[i], h + sh_lo * d, TQ_BF16, d, Ts, shgu, TQ_F32, 2 * f, nullptr));
    TQ_STEP(tq_swiglu(ctx, shgu, shgu + f, TQ_F32, 2 * f, Ts, f, shact, TQ_BF16));
    TQ_STEP(tq_qlinear(ctx, m->sh_down[i], shact, TQ_BF16, f, Ts, sh + i * Ts * d, TQ_F32, d, nullptr));
  }
  moe_combine_local_kernel<<<dim3((unsigned)T, (unsigned)((d + 1023) / 1024)), 256, 0, ctx->stream>>>(yo, slot, idl, w, (c.n_shared && Ts) ? sh : nullptr, (int)c.n_shared,
                                                                 Ts * d, (int)sh_lo, (int)sh_hi, (int)k, (int)d, nl, out_dev);
  TQ_LAUNCHED();
  if (comm) TQ_STEP(tq_all_reduce_f32(ctx, comm, out_dev, T * d));
  if (idx_out_dev) TQ_CUDA(ctx, cudaMemcpyAsync(idx_out_dev, idx, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  if (weight_out_dev) TQ_CUDA(ctx, cudaMemcpyAsync(weight_out_dev, w, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
#undef TQ_STEP
#undef TQ_LAUNCHED
  return TQ_OK;
}

int tq_moe_ffn_dispatch(tq_moe* m, const void* h_bf16_dev, size_t n_tokens, float* out_dev, tq_comm* comm, int* idx_out_dev,
                        float* weight_out_dev) {
  if (!m) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  if (int st = bind(ctx)) return st;
  const tq_moe_config& c = m->cfg;
  const int W = comm ? tq_comm_world(comm) : 1;
  TQ_REQUIRE(ctx, (uint32_t)W == c.ep_size && (!comm || (uint32_t)tq_comm_rank(comm) == c.ep_rank),
             "tq_moe_ffn_dispatch: the communicator must match the layer's expert-parallel rank and size");
  TQ_REQUIRE(ctx, W <= 64, "tq_moe_ffn_dispatch: at most 64 ranks");
  TQ_REQUIRE(ctx, n_tokens > 0 && h_bf16_dev && out_dev, "tq_moe_ffn_dispatch: every rank needs at least one token");
  TQ_REQUIRE(ctx, ((uintptr_t)h_bf16_dev & 15) == 0, "tq_moe_ffn_dispatch: activations must be 16-byte aligned");
  const size_t T = n_tokens, k = c.top_k, d = c.d_model, f = c.ffn, n = T * k;
  const int nl = m->n_local;
  const size_t cap = n;                      // places per peer: the worst case (every pair to one owner)
  const size_t R = (size_t)W * cap;          // rows this rank may receive
  auto up = [](size_t b) { return (b + 255) / 256 * 256; };
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += up(bytes);
    return o;
  };
  const size_t o_scnt = take(64 * 4), o_rcnt = take(64 * 4);
  const size_t o_idx = take(n * 4), o_w = take(n * 4), o_place = take(n * 4), o_zero = take(n * 4), o_lg = take(T * c.n_experts * 8),
               o_smeta = take(R * 4), o_rmeta = take(R * 4), o_sx = take(R * d * 2), o_rx = take(R * d * 2), o_bucket = take(R * 4),
               o_slot = take(R * 4), o_cnt = take((nl + 2) * 4), o_off = take((nl + 2) * 4), o_cur = take((nl + 2) * 4),
               o_active = take((nl + 2) * 4), o_xs = take(R * d * 2), o_gu = take(R * 2 * f * 4), o_act = take(R * f * 2),
               o_yo = take(R * d * 4), o_back = take(R * d * 4), o_ret = take(R * d * 4), o_sh = take((size_t)(c.n_shared ? c.n_shared : 1) * T * d * 4),
               o_shgu = take(T * 2 * f * 4), o_shact = take(T * f * 2);
  if (int st = ensure_scratch(ctx, off)) return st;
  uint8_t* s = static_cast<uint8_t*>(ctx->scratch);
  int *idx = reinterpret_cast<int*>(s + o_idx), *place = reinterpret_cast<int*>(s + o_place), *zero = reinterpret_cast<int*>(s + o_zero);
  float* w = reinterpret_cast<float*>(s + o_w);
  int *smeta = reinterpret_cast<int*>(s + o_smeta), *rmeta = reinterpret_cast<int*>(s + o_rmeta);
  __nv_bfloat16 *sx = reinterpret_cast<__nv_bfloat16*>(s + o_sx), *rx = reinterpret_cast<__nv_bfloat16*>(s + o_rx);
  int *bucket = reinterpret_cast<int*>(s + o_bucket), *slot = reinterpret_cast<int*>(s + o_slot);
  int *cnt = reinterpret_cast<int*>(s + o_cnt), *offs = reinterpret_cast<int*>(s + o_off), *cur = reinterpret_cast<int*>(s + o_cur);
  int* active = reinterpret_cast<int*>(s + o_active);
  __nv_bfloat16 *xs = reinterpret_cast<__nv_bfloat16*>(s + o_xs), *act = reinterpret_cast<__nv_bfloat16*>(s + o_act);
  float *gu = reinterpret_cast<float*>(s + o_gu), *yo = reinterpret_cast<float*>(s + o_yo), *back = reinterpret_cast<float*>(s + o_back),
        *ret = reinterpret_cast<float*>(s + o_ret), *sh = reinterpret_cast<float*>(s + o_sh), *shgu = reinterpret_cast<float*>(s + o_shgu);
  __nv_bfloat16* shact = reinterpret_cast<__nv_bfloat16*>(s + o_shact);
  const __nv_bfloat16* h = static_cast<const __nv_bfloat16*>(h_bf16_dev);
  int st;
#define TQ_STEP(expr) \
  if ((st = (expr)) != TQ_OK) return st;
#define TQ_LAUNCHED()   \
  ctx->launches++;      \
  TQ_CUDA(ctx, cudaGetLastError());

  // route this rank's tokens, plan the places, fill the send buffers
  TQ_STEP(launch_router(ctx, h, m->wg, T, d, c.n_experts, k, c.renormalize, idx, w, reinterpret_cast<double*>(s + o_lg)));
  int *scnt = reinterpret_cast<int*>(s + o_scnt), *rcnt = reinterpret_cast<int*>(s + o_rcnt);
  moe_dispatch_plan_kernel<<<1, 1024, 0, ctx->stream>>>(idx, (int)n, nl, W, (int)cap, place, smeta, scnt);
  TQ_LAUNCHED();
  moe_dispatch_rows_kernel<<<(unsigned)n, 128, 0, ctx->stream>>>(h, place, (int)k, (int)d, sx);
  TQ_LAUNCHED();
  // Counts first, for batches large enough to pay for a host round trip (and outside a graph capture, which cannot
  // wait for the host): the ranks tell one another how many rows follow, the host reads the counts, and rows, ids
  // and results travel with their true sizes into one contiguous block per owner.  Otherwise every peer block has
  // the worst-case `cap` rows (padding marked -1) and the exchange has a fixed size.
  const bool exact = comm && W > 1 && !ctx->capturing && n >= 256;
  size_t Rr = R;                             // rows on the owner's side
  size_t s_off[64], s_len[64], r_off[64], r_len[64];
  if (exact) {
    if (!m->host_counts) TQ_CUDA(ctx, cudaHostAlloc(&m->host_counts, 2 * 64 * sizeof(int), cudaHostAllocDefault));
    TQ_STEP(tq_all_to_all(ctx, comm, scnt, rcnt, 4));
    TQ_CUDA(ctx, cudaMemcpyAsync(m->host_counts, scnt, W * 4, cudaMemcpyDeviceToHost, ctx->stream));
    TQ_CUDA(ctx, cudaMemcpyAsync(m->host_counts + 64, rcnt, W * 4, cudaMemcpyDeviceToHost, ctx->stream));
    TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    Rr = 0;
    for (int p = 0; p < W; ++p) {
      TQ_REQUIRE(ctx, m->host_counts[p] >= 0 && (size_t)m->host_counts[p] <= cap && m->host_counts[64 + p] >= 0 &&
                          (size_t)m->host_counts[64 + p] <= cap, "tq_moe_ffn_dispatch: a peer announced an impossible row count");
      s_off[p] = (size_t)p * cap;            // rows: the send side keeps the place layout the combine reads
      s_len[p] = (size_t)m->host_counts[p];
      r_off[p] = Rr;
      r_len[p] = (size_t)m->host_counts[64 + p];
      Rr += r_len[p];
    }
    auto scaled = [&](const size_t* v, size_t mul, size_t* out) {
      for (int p = 0; p < W; ++p) out[p] = v[p] * mul;
    };
    size_t so[64], sl[64], ro[64], rl[64];
    scaled(s_off, d * 2, so); scaled(s_len, d * 2, sl); scaled(r_off, d * 2, ro); scaled(r_len, d * 2, rl);
    TQ_STEP(all_to_all_v(ctx, comm, sx, so, sl, rx, ro, rl));
    scaled(s_off, 4, so); scaled(s_len, 4, sl); scaled(r_off, 4, ro); scaled(r_len, 4, rl);
    TQ_STEP(all_to_all_v(ctx, comm, smeta, so, sl, rmeta, ro, rl));
  } else {
    // dispatch: rows and their expert ids to the owners
    TQ_STEP(tq_all_to_all(ctx, comm, sx, rx, cap * d * 2));
    TQ_STEP(tq_all_to_all(ctx, comm, smeta, rmeta, cap * 4));
  }
  // the owner's side: bucket by local expert, run the experts on what arrived
  if (Rr > 0) {
  moe_recv_bucket_kernel<<<(unsigned)((Rr + 255) / 256), 256, 0, ctx->stream>>>(rmeta, (int)Rr, nl, bucket);
  TQ_LAUNCHED();
  moe_count_kernel<<<1, 1024, 0, ctx->stream>>>(bucket, (int)Rr, nl + 1, cnt, offs, cur, active, nl);
  TQ_LAUNCHED();
  moe_slot_kernel<<<(unsigned)((Rr + 255) / 256), 256, 0, ctx->stream>>>(bucket, (int)Rr, cur, slot);
  TQ_LAUNCHED();
  moe_gather_recv_kernel<<<(unsigned)Rr, 128, 0, ctx->stream>>>(rx, bucket, slot, nl, (int)d, xs);
  TQ_LAUNCHED();
  size_t want = 2 * R / (size_t)(nl > 0 ? nl : 1) / (size_t)W + 1;   // expected rows per local expert, with slack
  int chunk = 8;
  while (chunk < 64 && (size_t)chunk < want) chunk <<= 1;
  const int max_rows = (int)((size_t)W * T < R ? (size_t)W * T : R);   // an expert gets a token at most once
  const int max_active = (int)(R < (size_t)nl ? R : (size_t)nl);
  const size_t expected = (size_t)W * n / (size_t)c.n_experts;      // rows per local expert when routing is even
  const bool tensor_path = expected >= 24 && umma_grouped_supported(m->w_gate_up, nl) && umma_grouped_supported(m->w_down, nl);
  if (tensor_path) {
    TQ_STEP(launch_qgemm_umma_grouped(ctx, m->w_gate_up, nl, xs, d, Rr, cnt, offs, active, max_active, max_rows, (int)(expected * 3 / 2),
                                      gu, TQ_F32, 2 * f));
  } else {
    TQ_STEP(launch_qgemm_grouped(ctx, m->w_gate_up, nl, xs, d, chunk, cnt, offs, max_rows, 0, 0, gu, TQ_F32, 2 * f, active, max_active, Rr));
  }
  TQ_STEP(tq_swiglu(ctx, gu, gu + f, TQ_F32, 2 * f, Rr, f, act, TQ_BF16));
  if (tensor_path) {
    TQ_STEP(launch_qgemm_umma_grouped(ctx, m->w_down, nl, act, f, Rr, cnt, offs, active, max_active, max_rows, (int)(expected * 3 / 2), yo,
                                      TQ_F32, d));
  } else {
    TQ_STEP(launch_qgemm_grouped(ctx, m->w_down, nl, act, f, chunk, cnt, offs, max_rows, 0, 0, yo, TQ_F32, d, active, max_active, Rr));
  }
  moe_scatter_back_kernel<<<(unsigned)Rr, 128, 0, ctx->stream>>>(yo, bucket, slot, nl, (int)d, back);
  TQ_LAUNCHED();
  }
  // combine: results back to the places they came from
  if (exact) {
    size_t so[64], sl[64], ro[64], rl[64];
    for (int p = 0; p < W; ++p) {
      so[p] = r_off[p] * d * 4;              // what arrived from p goes back to p ...
      sl[p] = r_len[p] * d * 4;
      ro[p] = s_off[p] * d * 4;              // ... and what was sent to p comes back into p's block of places
      rl[p] = s_len[p] * d * 4;
    }
    TQ_STEP(all_to_all_v(ctx, comm, back, so, sl, ret, ro, rl));
  } else {
    TQ_STEP(tq_all_to_all(ctx, comm, back, ret, cap * d * 4));
  }
  // shared experts run where the token lives
  for (size_t i = 0; i < m->sh_gate_up.size(); ++i) {
    TQ_STEP(tq_qlinear(ctx, m->sh_gate_up[i], h, TQ_BF16, d, T, shgu, TQ_F32, 2 * f, nullptr));
    TQ_STEP(tq_swiglu(ctx, shgu, shgu + f, TQ_F32, 2 * f, T, f, shact, TQ_BF16));
    TQ_STEP(tq_qlinear(ctx, m->sh_down[i], shact, TQ_BF16, f, T, sh + i * T * d, TQ_F32, d, nullptr));
  }
  TQ_CUDA(ctx, cudaMemsetAsync(zero, 0, n * 4, ctx->stream));
  moe_combine_local_kernel<<<dim3((unsigned)T, (unsigned)((d + 1023) / 1024)), 256, 0, ctx->stream>>>(
      ret, place, zero, w, c.n_shared ? sh : nullptr, (int)c.n_shared, T * d, 0, (int)T, (int)k, (int)d, 1, out_dev);
  TQ_LAUNCHED();
  if (idx_out_dev) TQ_CUDA(ctx, cudaMemcpyAsync(idx_out_dev, idx, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  if (weight_out_dev) TQ_CUDA(ctx, cudaMemcpyAsync(weight_out_dev, w, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
#undef TQ_STEP
#undef TQ_LAUNCHED
  return TQ_OK;
}

int tq_moe_destroy(tq_moe* m) {
  if (m && m->host_counts) cudaFreeHost(m->host_counts);
  delete m;
  return TQ_OK;
}

}  // extern "C"
