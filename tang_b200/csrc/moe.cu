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
                         void* y, int y_dtype, size_t ldy);

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 16;

// One CTA per token, one thread per expert.  Logits are accumulated in f64 in ascending k, one
// product at a time — the same sequence of additions as the CPU restatement, and bf16 x bf16
// products are exact in f64, so the logits (hence the selection) are bit-identical to it.
__global__ void router_kernel(const __nv_bfloat16* h, const __nv_bfloat16* wg, int T, int d, int E, int top_k,
                              int renorm, int* idx_out, float* w_out, double* logits_out) {
  extern __shared__ double sh[];          // [128] h chunk | [E][129] gate chunk
  double* hs = sh;
  double* ws = sh + 128;
  __shared__ double lg[kMaxExperts];
  const int t = blockIdx.x, e = threadIdx.x;
  double acc = 0.0;
  for (int k0 = 0; k0 < d; k0 += 128) {
    const int kn = min(128, d - k0);
    for (int i = threadIdx.x; i < kn; i += blockDim.x) hs[i] = (double)__bfloat162float(h[(size_t)t * d + k0 + i]);
    for (int i = threadIdx.x; i < E * kn; i += blockDim.x) {
      const int ee = i / kn, kk = i % kn;
      ws[ee * 129 + kk] = (double)__bfloat162float(wg[(size_t)ee * d + k0 + kk]);
    }
    __syncthreads();
    if (e < E)
      for (int kk = 0; kk < kn; ++kk) acc += hs[kk] * ws[e * 129 + kk];
    __syncthreads();
  }
  if (e < E) {
    lg[e] = acc;
    if (logits_out) logits_out[(size_t)t * E + e] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double mx = lg[0];
    for (int i = 1; i < E; ++i) mx = fmax(mx, lg[i]);
    double sum = 0.0;
    for (int i = 0; i < E; ++i) sum += exp(lg[i] - mx);
    unsigned long long taken[kMaxExperts / 64] = {0, 0, 0, 0};
    double chosen = 0.0;
    double pw[kMaxTopK];
    int pi[kMaxTopK];
    for (int s = 0; s < top_k; ++s) {
      int best = -1;
      for (int i = 0; i < E; ++i) {
        if ((taken[i >> 6] >> (i & 63)) & 1ull) continue;
        if (best < 0 || lg[i] > lg[best]) best = i;   // strict '>' keeps the lower index on ties
      }
      taken[best >> 6] |= 1ull << (best & 63);
      pi[s] = best;
      pw[s] = exp(lg[best] - mx) / sum;
      chosen += pw[s];
    }
    for (int s = 0; s < top_k; ++s) {
      idx_out[(size_t)t * top_k + s] = pi[s];
      w_out[(size_t)t * top_k + s] = (float)(renorm ? pw[s] / chosen : pw[s]);
    }
  }
}

// counts[e] = rows routed to expert e (a single CTA; T*top_k entries).
__global__ void moe_count_kernel(const int* idx, int n, int E, int* counts, int* offsets, int* cursor) {
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

}  // namespace tq

struct tq_moe {
  tq_ctx* ctx = nullptr;
  tq_moe_config cfg{};
  const void* wg = nullptr;                 // bf16 [n_experts, d_model]
  const tq_qweight* w_gate_up = nullptr;    // stacked [n_local * 2*ffn, d_model]
  const tq_qweight* w_down = nullptr;       // stacked [n_local * d_model, ffn]
  std::vector<const tq_qweight*> sh_gate_up, sh_down;
  int expert_lo = 0, n_local = 0;           // experts held by this rank
};

using namespace tq;

extern "C" {

int tq_moe_router(tq_ctx* ctx, const void* h_bf16_dev, const void* wg_bf16_dev, size_t n_tokens, size_t d_model,
                  size_t n_experts, size_t top_k, int renormalize, int* idx_out_dev, float* weight_out_dev,
                  double* logits_out_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, n_experts > 0 && n_experts <= kMaxExperts && top_k > 0 && top_k <= kMaxTopK && top_k <= n_experts,
             "tq_moe_router: need 1 <= top_k <= n_experts <= %d and top_k <= %d", kMaxExperts, kMaxTopK);
  if (n_tokens == 0) return TQ_OK;
  TQ_REQUIRE(ctx, h_bf16_dev && wg_bf16_dev && idx_out_dev && weight_out_dev, "tq_moe_router: null pointer");
  const int threads = (int)((n_experts + 31) / 32 * 32);
  const size_t smem = (128 + n_experts * 129) * sizeof(double);
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    TQ_CUDA(ctx, cudaFuncSetAttribute(router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    smem_set = smem;
  }
  router_kernel<<<(unsigned)n_tokens, threads, smem, ctx->stream>>>(
      static_cast<const __nv_bfloat16*>(h_bf16_dev), static_cast<const __nv_bfloat16*>(wg_bf16_dev), (int)n_tokens,
      (int)d_model, (int)n_experts, (int)top_k, renormalize, idx_out_dev, weight_out_dev, logits_out_dev);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
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
                                         const float* shared, int shared_lo, int shared_hi, int top_k, int d, int n_local,
                                         float* out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < top_k; ++s) {
      const size_t i = (size_t)t * top_k + s;
      if (idx_local[i] < n_local) acc += w[i] * yo[(size_t)slot[i] * d + c];
    }
    if (shared && t >= shared_lo && t < shared_hi) acc += shared[(size_t)(t - shared_lo) * d + c];
    out[(size_t)t * d + c] = acc;
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
               o_off = take((nl + 1) * 4), o_cur = take((nl + 1) * 4), o_xs = take(n * d * 2), o_gu = take(n * 2 * f * 4),
               o_act = take(n * f * 2), o_yo = take(n * d * 4), o_sh = take(Ts * d * 4), o_shgu = take(Ts * 2 * f * 4),
               o_shact = take(Ts * f * 2);
  if (int st = ensure_scratch(ctx, off)) return st;
  uint8_t* s = static_cast<uint8_t*>(ctx->scratch);
  int* idx = reinterpret_cast<int*>(s + o_idx);
  int* idl = reinterpret_cast<int*>(s + o_idl);
  float* w = reinterpret_cast<float*>(s + o_w);
  int* slot = reinterpret_cast<int*>(s + o_slot);
  int *cnt = reinterpret_cast<int*>(s + o_cnt), *offs = reinterpret_cast<int*>(s + o_off), *cur = reinterpret_cast<int*>(s + o_cur);
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

  TQ_STEP(tq_moe_router(ctx, h, m->wg, T, d, c.n_experts, k, c.renormalize, idx, w, nullptr));
  moe_localize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(idx, (int)n, m->expert_lo, nl, idl);
  TQ_LAUNCHED();
  moe_count_kernel<<<1, 1024, 0, ctx->stream>>>(idl, (int)n, nl + 1, cnt, offs, cur);
  TQ_LAUNCHED();
  moe_slot_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(idl, (int)n, cur, slot);
  TQ_LAUNCHED();
  moe_gather_kernel<<<(unsigned)n, 128, 0, ctx->stream>>>(h, slot, (int)n, (int)k, (int)d, xs);
  TQ_LAUNCHED();
  const int cap = (int)(T < 64 ? T : 64);   // a token picks an expert at most once: counts[e] <= T
  TQ_STEP(launch_qgemm_grouped(ctx, m->w_gate_up, nl, xs, d, cap, cnt, offs, (int)T, 0, 0, gu, TQ_F32, 2 * f));
  TQ_STEP(tq_swiglu(ctx, gu, gu + f, TQ_F32, 2 * f, n, f, act, TQ_BF16));
  TQ_STEP(launch_qgemm_grouped(ctx, m->w_down, nl, act, f, cap, cnt, offs, (int)T, 0, 0, yo, TQ_F32, d));
  for (size_t i = 0; i < m->sh_gate_up.size() && Ts > 0; ++i) {
    TQ_STEP(tq_qlinear(ctx, m->sh_gate_up[i], h + sh_lo * d, TQ_BF16, d, Ts, shgu, TQ_F32, 2 * f, nullptr));
    TQ_STEP(tq_swiglu(ctx, shgu, shgu + f, TQ_F32, 2 * f, Ts, f, shact, TQ_BF16));
    TQ_STEP(tq_qlinear(ctx, m->sh_down[i], shact, TQ_BF16, f, Ts, sh, TQ_F32, d, i ? sh : nullptr));
  }
  moe_combine_local_kernel<<<(unsigned)T, 256, 0, ctx->stream>>>(yo, slot, idl, w, (c.n_shared && Ts) ? sh : nullptr, (int)sh_lo,
                                                                 (int)sh_hi, (int)k, (int)d, nl, out_dev);
  TQ_LAUNCHED();
  if (comm) TQ_STEP(tq_all_reduce_f32(ctx, comm, out_dev, T * d));
  if (idx_out_dev) TQ_CUDA(ctx, cudaMemcpyAsync(idx_out_dev, idx, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  if (weight_out_dev) TQ_CUDA(ctx, cudaMemcpyAsync(weight_out_dev, w, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
#undef TQ_STEP
#undef TQ_LAUNCHED
  return TQ_OK;
}

int tq_moe_destroy(tq_moe* m) {
  delete m;
  return TQ_OK;
}

}  // extern "C"
