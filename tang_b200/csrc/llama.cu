// Llama-shaped decode step on the device (include/tangq.h, tq_llama_*).
//
// Follows the reference's one decode loop, crates/tang-train/examples/smollm.rs:215-296, op for op:
// pre-norm -> q/k/v -> RoPE -> cache append -> GQA attention -> o_proj -> residual -> pre-norm ->
// SwiGLU -> down -> residual; final norm; LM head.  Differences are scheduling only:
//   * q/k/v and gate/up are single fused quantised GEMVs (weights concatenated along rows);
//   * the residual add is folded into the next RMSNorm (the reference's own fused operator,
//     rms_norm_residual, crates/tang-compute/src/device.rs:546-575), so under tensor parallelism
//     the row-parallel o_proj / down partial sums are all-reduced in place and consumed directly;
//   * the KV cache lives in HBM as bf16 [sequence][position][kv_dim] and is appended in place.
// Sharding (crates/tang-mesh/src/placement.rs:12-31 names Split{axis}; nothing executes it there):
// q/k/v, gate/up and the LM head are split by output rows, o_proj and down by input columns;
// attention heads follow their KV head.
#include <cuda_bf16.h>

#include <new>
#include <utility>
#include <vector>

#include "internal.h"
#include "qlayout.cuh"

struct tq_comm;
extern "C" int tq_all_reduce_f32(tq_ctx*, tq_comm*, float*, size_t);
extern "C" int tq_all_gather(tq_ctx*, tq_comm*, const void*, void*, size_t);
extern "C" int tq_comm_world(const tq_comm*);
extern "C" int tq_comm_rank(const tq_comm*);
extern "C" int tq_comm_enable_peer(tq_ctx*, tq_comm*, size_t);

namespace tq {
int launch_qkv_post(tq_ctx* ctx, const float* qkv, const float* cos_t, const float* sin_t, const int* positions,
                    const int* rope_positions, int B, int n_heads, int n_kv, int hd, int max_seq, void* q_out, void* k_cache,
                    void* v_cache, size_t seq_stride, int q_len);
int launch_gqa_decode(tq_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, const int* lens, int B,
                      int n_heads, int n_kv, int head_dim, size_t seq_stride, int max_len, void* out, int out_dtype);

// Attention length of each sequence: its new token's position + 1, kept inside the cache whatever the position
// says (a position outside 0 .. max_seq-1 is reported through the status word by the kernel that appends K/V).
__global__ void lens_kernel(const int* positions, int* lens, int n, int max_seq) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) lens[i] = min(max(positions[i] + 1, 0), max_seq);
}

// KVCache::trim_to (crates/tang-infer/src/kv_cache.rs:138-149) for one layer's K and V caches: a sequence that
// holds more than `keep` positions drops its OLDEST ones, i.e. rows [len - keep, len) move to [0, keep).  The move
// is in place: each thread owns one 16-byte column of a sequence's rows and walks it front to back, eight rows at
// a time (read eight, then write eight), so a row is always read before the same column's writes reach it.
__global__ void kv_trim_kernel(__nv_bfloat16* k_cache, __nv_bfloat16* v_cache, const int* lens, int keep, int max_seq,
                               size_t row_elems, size_t seq_stride) {
  const int b = blockIdx.y;
  __nv_bfloat16* base = (blockIdx.z ? v_cache : k_cache) + (size_t)b * seq_stride;
  const int len = min(max(lens[b], 0), max_seq);
  const int drop = len - keep;
  if (drop <= 0) return;
  const size_t vecs = row_elems / 8;                       // 16-byte columns per row
  const size_t col = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= vecs) return;
  uint4* p = reinterpret_cast<uint4*>(base) + col;
  for (int r = 0; r < keep; r += 8) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (r + i < keep) v[i] = p[(size_t)(r + i + drop) * vecs];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (r + i < keep) p[(size_t)(r + i) * vecs] = v[i];
  }
}

__global__ void kv_trim_lens_kernel(int* lens, int n, int keep, int max_seq) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) lens[i] = min(min(max(lens[i], 0), max_seq), keep);
}
}  // namespace tq

struct LlamaLayerW {
  const tq_qweight *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wdown = nullptr;
  const void *attn_norm = nullptr, *ffn_norm = nullptr;  // bf16 [d_model]
  __nv_bfloat16 *k_cache = nullptr, *v_cache = nullptr;  // [max_batch][max_seq][kv_dim_local]
};

struct tq_llama {
  tq_ctx* ctx = nullptr;
  tq_llama_config cfg{};
  int tp = 1, rank = 0;
  int heads_l = 0, kv_l = 0, ffn_l = 0, vocab_l = 0;  // per-rank shard sizes
  std::vector<LlamaLayerW> layers;
  const void* embed = nullptr;       // bf16 [vocab, d_model] (replicated)
  const void* final_norm = nullptr;  // bf16 [d_model]
  const tq_qweight* lm_head = nullptr;
  tq_comm* comm = nullptr;
  float *cos_t = nullptr, *sin_t = nullptr;
  // activations
  float *h = nullptr, *h2 = nullptr, *delta = nullptr, *qkv = nullptr, *gu = nullptr, *logits_l = nullptr;
  float* h_last = nullptr;   // which of h / h2 holds the residual stream after the last decode step
  float* ss = nullptr;       // [8][d_model / 16]: row sums of squares handed from a projection to the next pre-norm
  __nv_bfloat16 *xn = nullptr, *qb = nullptr, *attn = nullptr, *act = nullptr;
  int* lens = nullptr;
  // prefill workspaces (rows = sequences x chunk length), grown on demand by tq_llama_prefill
  size_t pre_rows = 0;
  float *p_h = nullptr, *p_delta = nullptr, *p_qkv = nullptr, *p_gu = nullptr;
  __nv_bfloat16 *p_xn = nullptr, *p_qb = nullptr, *p_attn = nullptr, *p_act = nullptr, *p_last = nullptr;
  std::vector<void*> owned;
};

using namespace tq;

static int dev_alloc(tq_llama* m, void** p, size_t bytes) {
  TQ_CUDA(m->ctx, cudaMalloc(p, bytes ? bytes : 16));
  m->owned.push_back(*p);
  return TQ_OK;
}

extern "C" {

int tq_qweight_concat_rows(tq_ctx* ctx, const tq_qweight* const* parts, size_t n_parts, tq_qweight** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, parts && n_parts > 0 && out, "tq_qweight_concat_rows: null argument");
  *out = nullptr;
  size_t rows = 0;
  for (size_t i = 0; i < n_parts; ++i) {
    TQ_REQUIRE(ctx, parts[i] != nullptr, "tq_qweight_concat_rows: null part");
    TQ_REQUIRE(ctx, parts[i]->kind == parts[0]->kind && parts[i]->cols == parts[0]->cols,
               "tq_qweight_concat_rows: parts must share kind and column count");
    TQ_REQUIRE(ctx, i + 1 == n_parts || parts[i]->rows % kTileRows == 0,
               "tq_qweight_concat_rows: every part but the last needs a row count that is a multiple of 16");
    rows += parts[i]->rows;
  }
  tq_qweight* w = new (std::nothrow) tq_qweight();
  if (!w) return fail(ctx, TQ_ENOMEM, "out of host memory");
  *w = *parts[0];
  w->rows = rows;
  w->n_rb = (int)((rows + kTileRows - 1) / kTileRows);
  w->tile_bytes = (size_t)w->n_rb * w->n_kc * qk_tile_bytes(w->kind);
  w->tiles = nullptr;
  w->row_scales = nullptr;
  cudaError_t e = cudaMalloc(&w->tiles, w->tile_bytes);
  if (e == cudaSuccess && w->kind == TQ_I8_ROW) e = cudaMalloc(&w->row_scales, rows * sizeof(float));
  size_t off = 0, roff = 0;
  for (size_t i = 0; i < n_parts && e == cudaSuccess; ++i) {
    e = cudaMemcpyAsync(w->tiles + off, parts[i]->tiles, parts[i]->tile_bytes, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e == cudaSuccess && w->kind == TQ_I8_ROW)
      e = cudaMemcpyAsync(w->row_scales + roff, parts[i]->row_scales, parts[i]->rows * sizeof(float),
                          cudaMemcpyDeviceToDevice, ctx->stream);
    off += parts[i]->tile_bytes;
    roff += parts[i]->rows;
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) {
    if (w->tiles) cudaFree(w->tiles);
    if (w->row_scales) cudaFree(w->row_scales);
    delete w;
    cudaGetLastError();
    return fail(ctx, TQ_ECUDA, "tq_qweight_concat_rows: %s", cudaGetErrorString(e));
  }
  *out = w;
  return TQ_OK;
}

int tq_llama_create(tq_ctx* ctx, const tq_llama_config* cfg, tq_comm* comm, tq_llama** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, cfg && out, "tq_llama_create: null argument");
  *out = nullptr;
  const int tp = comm ? tq_comm_world(comm) : 1;
  TQ_REQUIRE(ctx, cfg->n_layers > 0 && cfg->d_model > 0 && cfg->head_dim == 128, "tq_llama_create: head_dim must be 128");
  TQ_REQUIRE(ctx, cfg->n_kv_heads > 0 && cfg->n_heads % cfg->n_kv_heads == 0 && cfg->n_heads / cfg->n_kv_heads <= 8,
             "tq_llama_create: n_heads / n_kv_heads must be 1..8");
  TQ_REQUIRE(ctx, cfg->n_kv_heads % tp == 0 && cfg->ffn % (32 * tp) == 0 && cfg->vocab % tp == 0,
             "tq_llama_create: kv heads, ffn/32 and vocab must divide by the tensor-parallel size %d", tp);
  TQ_REQUIRE(ctx, cfg->max_batch > 0 && cfg->max_batch <= 64 && cfg->max_seq > 0, "tq_llama_create: max_batch must be 1..64");
  tq_llama* m = new (std::nothrow) tq_llama();
  if (!m) return fail(ctx, TQ_ENOMEM, "out of host memory");
  m->ctx = ctx;
  m->cfg = *cfg;
  m->comm = comm;
  m->tp = tp;
  m->rank = comm ? tq_comm_rank(comm) : 0;
  m->heads_l = cfg->n_heads / tp;
  m->kv_l = cfg->n_kv_heads / tp;
  m->ffn_l = cfg->ffn / tp;
  m->vocab_l = cfg->vocab / tp;
  m->layers.resize(cfg->n_layers);
  const size_t B = cfg->max_batch, d = cfg->d_model, hd = cfg->head_dim;
  const size_t kv_dim = (size_t)m->kv_l * hd, q_dim = (size_t)m->heads_l * hd;
  int st = TQ_OK;
  auto A = [&](void** p, size_t bytes) {
    if (st == TQ_OK) st = dev_alloc(m, p, bytes);
  };
  A((void**)&m->cos_t, (size_t)cfg->max_seq * (hd / 2) * 4);
  A((void**)&m->sin_t, (size_t)cfg->max_seq * (hd / 2) * 4);
  A((void**)&m->h, B * d * 4);
  A((void**)&m->h2, B * d * 4);
  A((void**)&m->delta, B * d * 4);
  A((void**)&m->ss, 8 * ((d + 15) / 16) * 4);
  A((void**)&m->qkv, B * (q_dim + 2 * kv_dim) * 4);
  A((void**)&m->gu, B * 2 * m->ffn_l * 4);
  A((void**)&m->logits_l, B * m->vocab_l * 4);
  A((void**)&m->xn, B * d * 2);
  A((void**)&m->qb, B * q_dim * 2);
  A((void**)&m->attn, B * q_dim * 2);
  A((void**)&m->act, B * m->ffn_l * 2);
  A((void**)&m->lens, B * 4);
  for (auto& L : m->layers) {
    A((void**)&L.k_cache, B * cfg->max_seq * kv_dim * 2);
    A((void**)&L.v_cache, B * cfg->max_seq * kv_dim * 2);
  }
  if (st == TQ_OK) st = tq_rope_tables(ctx, hd, cfg->max_seq, cfg->rope_base, m->cos_t, m->sin_t);
  if (st != TQ_OK) {
    for (void* p : m->owned) cudaFree(p);
    delete m;
    cudaGetLastError();
    return st;
  }
  *out = m;
  return TQ_OK;
}

int tq_llama_destroy(tq_llama* m) {
  if (!m) return TQ_OK;
  bind(m->ctx);
  cudaStreamSynchronize(m->ctx->stream);
  for (void* p : m->owned) cudaFree(p);
  delete m;
  return TQ_OK;
}

int tq_llama_set_layer(tq_llama* m, size_t layer, const tq_qweight* wqkv, const tq_qweight* wo, const tq_qweight* wgate_up,
                       const tq_qweight* wdown, const void* attn_norm_bf16_dev, const void* ffn_norm_bf16_dev) {
  if (!m) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  TQ_REQUIRE(ctx, layer < m->layers.size(), "tq_llama_set_layer: layer %zu out of range", layer);
  TQ_REQUIRE(ctx, wqkv && wo && wgate_up && wdown && attn_norm_bf16_dev && ffn_norm_bf16_dev, "tq_llama_set_layer: null weight");
  const size_t d = m->cfg.d_model, hd = m->cfg.head_dim;
  const size_t q_dim = (size_t)m->heads_l * hd, kv_dim = (size_t)m->kv_l * hd;
  TQ_REQUIRE(ctx, wqkv->rows == q_dim + 2 * kv_dim && wqkv->cols == d, "tq_llama_set_layer: wqkv must be [%zu, %zu]", q_dim + 2 * kv_dim, d);
  TQ_REQUIRE(ctx, wo->rows == d && wo->cols == q_dim, "tq_llama_set_layer: wo must be [%zu, %zu]", d, q_dim);
  TQ_REQUIRE(ctx, wgate_up->rows == 2 * (size_t)m->ffn_l && wgate_up->cols == d, "tq_llama_set_layer: wgate_up must be [%zu, %zu]", 2 * (size_t)m->ffn_l, d);
  TQ_REQUIRE(ctx, wdown->rows == d && wdown->cols == (size_t)m->ffn_l, "tq_llama_set_layer: wdown must be [%zu, %zu]", d, (size_t)m->ffn_l);
  LlamaLayerW& L = m->layers[layer];
  L.wqkv = wqkv;
  L.wo = wo;
  L.wgu = wgate_up;
  L.wdown = wdown;
  L.attn_norm = attn_norm_bf16_dev;
  L.ffn_norm = ffn_norm_bf16_dev;
  return TQ_OK;
}

int tq_llama_set_head(tq_llama* m, const void* embed_bf16_dev, const void* final_norm_bf16_dev, const tq_qweight* lm_head) {
  if (!m) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  TQ_REQUIRE(ctx, embed_bf16_dev && final_norm_bf16_dev && lm_head, "tq_llama_set_head: null argument");
  TQ_REQUIRE(ctx, lm_head->rows == (size_t)m->vocab_l && lm_head->cols == m->cfg.d_model, "tq_llama_set_head: lm_head must be [%d, %u]",
             m->vocab_l, m->cfg.d_model);
  m->embed = embed_bf16_dev;
  m->final_norm = final_norm_bf16_dev;
  m->lm_head = lm_head;
  return TQ_OK;
}

int tq_llama_kv_cache(tq_llama* m, size_t layer, void** k_cache_dev, void** v_cache_dev, size_t* seq_stride_elems) {
  if (!m || layer >= m->layers.size()) return TQ_EINVAL;
  if (k_cache_dev) *k_cache_dev = m->layers[layer].k_cache;
  if (v_cache_dev) *v_cache_dev = m->layers[layer].v_cache;
  if (seq_stride_elems) *seq_stride_elems = (size_t)m->cfg.max_seq * m->kv_l * m->cfg.head_dim;
  return TQ_OK;
}

int tq_llama_kv_trim(tq_llama* m, int* seq_lens_io_dev, size_t batch, size_t keep) {
  if (!m) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  if (int st = bind(ctx)) return st;
  const tq_llama_config& c = m->cfg;
  TQ_REQUIRE(ctx, seq_lens_io_dev != nullptr, "tq_llama_kv_trim: null lengths");
  TQ_REQUIRE(ctx, batch > 0 && batch <= c.max_batch, "tq_llama_kv_trim: batch must be 1..%u", c.max_batch);
  if (keep >= c.max_seq) return TQ_OK;   // no sequence can hold more than max_seq positions: nothing to drop
  const size_t row_elems = (size_t)m->kv_l * c.head_dim, seq_stride = (size_t)c.max_seq * row_elems;
  TQ_REQUIRE(ctx, row_elems % 8 == 0, "tq_llama_kv_trim: cache rows must be a multiple of 16 bytes");
  if (keep > 0) {
    const unsigned gx = (unsigned)((row_elems / 8 + 127) / 128);
    for (auto& L : m->layers) {
      kv_trim_kernel<<<dim3(gx, (unsigned)batch, 2), 128, 0, ctx->stream>>>(L.k_cache, L.v_cache, seq_lens_io_dev, (int)keep,
                                                                          (int)c.max_seq, row_elems, seq_stride);
      ctx->launches++;
    }
    TQ_CUDA(ctx, cudaGetLastError());
  }
  kv_trim_lens_kernel<<<(unsigned)((batch + 63) / 64), 64, 0, ctx->stream>>>(seq_lens_io_dev, (int)batch, (int)keep, (int)c.max_seq);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

int tq_llama_hidden(tq_llama* m, float** hidden_dev) {
  if (!m || !hidden_dev) return TQ_EINVAL;
  *hidden_dev = m->h_last ? m->h_last : m->h;
  return TQ_OK;
}

int tq_llama_decode(tq_llama* m, const int* token_ids_dev, const int* positions_dev, size_t batch, size_t max_len,
                    float* logits_dev) {
  return tq_llama_decode_at(m, token_ids_dev, positions_dev, nullptr, batch, max_len, logits_dev);
}

int tq_llama_decode_at(tq_llama* m, const int* token_ids_dev, const int* positions_dev, const int* rope_positions_dev,
                       size_t batch, size_t max_len, float* logits_dev) {
  if (!m) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  if (int st = bind(ctx)) return st;
  const tq_llama_config& c = m->cfg;
  TQ_REQUIRE(ctx, batch > 0 && batch <= c.max_batch, "tq_llama_decode: batch must be 1..%u", c.max_batch);
  TQ_REQUIRE(ctx, token_ids_dev && positions_dev && logits_dev, "tq_llama_decode: null pointer");
  TQ_REQUIRE(ctx, max_len > 0 && max_len <= c.max_seq, "tq_llama_decode: max_len must be 1..max_seq");
  TQ_REQUIRE(ctx, m->lm_head != nullptr, "tq_llama_decode: head weights not set");
  for (auto& L : m->layers) TQ_REQUIRE(ctx, L.wqkv != nullptr, "tq_llama_decode: a layer has no weights");
  const int B = (int)batch;
  const size_t d = c.d_model, hd = c.head_dim;
  const size_t q_dim = (size_t)m->heads_l * hd, kv_dim = (size_t)m->kv_l * hd;
  const size_t seq_stride = (size_t)c.max_seq * kv_dim;
  int st;
#define TQ_STEP(expr) \
  if ((st = (expr)) != TQ_OK) return st;

  TQ_CUDA(ctx, launch_k(ctx, lens_kernel, dim3((B + 63) / 64), dim3(64), 0, positions_dev, m->lens, B, (int)c.max_seq));
  TQ_STEP(tq_embedding(ctx, m->embed, TQ_BF16, token_ids_dev, B, d, c.vocab, m->h, TQ_F32));

  // The residual stream alternates between two buffers, and every pre-norm is fused into the projection that follows
  // it; with a gate/up weight in the interleaved row order the SwiGLU is that projection's epilogue.  Per layer: qkv
  // (+norm), RoPE/append, attention, merge, o, gate/up (+norm, +SwiGLU), down.  Batches above eight rows take the
  // same path through the separate operators.
  //   * One GPU, up to eight rows: o and down add the residual themselves (y = h_next, residual = h) and, from four
  //     rows on, leave the rows' sums of squares per 16-row block, so that the pre-norm that follows reads only its
  //     slab of the stream.
  //   * Tensor parallel, or more than eight rows: o and down write this rank's partial sums to `delta`, which is all-reduced; each CTA of the
  //     next projection forms rms_norm(h + delta) itself and its first CTA writes h + delta to the OTHER buffer while
  //     its siblings still read the old one.
  float *h_cur = m->h, *h_nxt = m->h2;
  const bool fold = m->comm == nullptr && B <= 8;   // (the tensor-memory GEMM of the larger batches takes no residual)
  // (measured per decode step against the plain prologue: -1.3 % at four rows, -5.3 % at eight, nothing below)
  const int ss_min = 4;
  const int n_ss = (int)((d + 15) / 16);
  struct SsGuard {   // (no request outlives this call, whichever way it returns)
    tq_ctx* c;
    ~SsGuard() { c->ss_req = nullptr; }
  } ss_guard{ctx};
  bool have_delta = false;  // true once `delta` holds a projection output not yet added to h
  bool have_ss = false;     // true while `ss` describes h_cur
  // y = h_nxt = h_cur + W x (one GPU), or delta = W x, all-reduced
  auto project_back = [&](const tq_qweight* w, const void* x, size_t cols) -> int {
    if (!fold) {
      if (int e = tq_qlinear(ctx, w, x, TQ_BF16, cols, B, m->delta, TQ_F32, d, nullptr)) return e;
      have_delta = true;
      return tq_all_reduce_f32(ctx, m->comm, m->delta, (size_t)B * d);
    }
    ctx->ss_req = B >= ss_min ? m->ss : nullptr;
    ctx->ss_written = false;
    const int e = tq_qlinear(ctx, w, x, TQ_BF16, cols, B, h_nxt, TQ_F32, d, h_cur);
    ctx->ss_req = nullptr;
    have_ss = e == TQ_OK && ctx->ss_written;
    std::swap(h_cur, h_nxt);
    return e;
  };
  auto pre_norm = [&](const void* gain) {
    QlinearNorm n;
    n.h = h_cur;
    n.delta = have_delta ? m->delta : nullptr;
    n.gain_bf16 = gain;
    n.h_out = fold ? nullptr : h_nxt;
    n.eps = c.eps;
    n.xn_tmp = m->xn;
    n.sumsq = have_ss ? m->ss : nullptr;
    n.n_sumsq = have_ss ? n_ss : 0;
    return n;
  };
  for (size_t l = 0; l < m->layers.size(); ++l) {
    const LlamaLayerW& L = m->layers[l];
    const QlinearNorm n1 = pre_norm(L.attn_norm);
    TQ_STEP(qlinear_fused(ctx, L.wqkv, nullptr, &n1, B, m->qkv, TQ_F32, q_dim + 2 * kv_dim, false, nullptr));
    if (!fold) std::swap(h_cur, h_nxt);
    TQ_STEP(launch_qkv_post(ctx, m->qkv, m->cos_t, m->sin_t, positions_dev, rope_positions_dev, B, m->heads_l, m->kv_l, (int)hd, (int)c.max_seq,
                            m->qb, L.k_cache, L.v_cache, seq_stride, 1));
    TQ_STEP(launch_gqa_decode(ctx, m->qb, L.k_cache, L.v_cache, m->lens, B, m->heads_l, m->kv_l, (int)hd, seq_stride,
                              (int)max_len, m->attn, TQ_BF16));
    TQ_STEP(project_back(L.wo, m->attn, q_dim));
    // h += attention output; pre-norm of the MLP; gate/up; SwiGLU
    const QlinearNorm n2 = pre_norm(L.ffn_norm);
    if (L.wgu->gate_up_interleaved) {
      TQ_STEP(qlinear_fused(ctx, L.wgu, nullptr, &n2, B, m->act, TQ_BF16, m->ffn_l, true, m->gu));
    } else {
      TQ_STEP(qlinear_fused(ctx, L.wgu, nullptr, &n2, B, m->gu, TQ_F32, 2 * (size_t)m->ffn_l, false, nullptr));
      TQ_STEP(tq_swiglu(ctx, m->gu, m->gu + m->ffn_l, TQ_F32, 2 * (size_t)m->ffn_l, B, m->ffn_l, m->act, TQ_BF16));
    }
    if (!fold) std::swap(h_cur, h_nxt);
    TQ_STEP(project_back(L.wdown, m->act, m->ffn_l));
  }
  // final norm (under tensor parallelism it adds the last MLP output) fused into the LM head, which sees every row
  // (each is a sequence's last token)
  const QlinearNorm nf = pre_norm(m->final_norm);
  m->h_last = fold ? h_cur : h_nxt;   // (tensor parallel: the head kernel writes h + the last MLP output there)
  if (m->tp == 1) {
    TQ_STEP(qlinear_fused(ctx, m->lm_head, nullptr, &nf, B, logits_dev, TQ_F32, c.vocab, false, nullptr));
  } else {
    // column-parallel head: this rank's vocabulary slice, gathered rank-major: logits_dev is
    // [tp][B][vocab/tp]
    TQ_STEP(qlinear_fused(ctx, m->lm_head, nullptr, &nf, B, m->logits_l, TQ_F32, m->vocab_l, false, nullptr));
    TQ_STEP(tq_all_gather(ctx, m->comm, m->logits_l, logits_dev, (size_t)B * m->vocab_l * sizeof(float)));
  }
#undef TQ_STEP
  return TQ_OK;
}

int tq_llama_prefill(tq_llama* m, const int* token_ids_dev, const int* cache_start_dev, size_t batch, size_t q_len,
                     float* logits_dev) {
  if (!m) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  if (int st = bind(ctx)) return st;
  const tq_llama_config& c = m->cfg;
  TQ_REQUIRE(ctx, batch > 0 && batch <= c.max_batch, "tq_llama_prefill: batch must be 1..%u", c.max_batch);
  TQ_REQUIRE(ctx, q_len > 0 && q_len <= c.max_seq, "tq_llama_prefill: chunk length must be 1..max_seq");
  TQ_REQUIRE(ctx, token_ids_dev && cache_start_dev && logits_dev, "tq_llama_prefill: null pointer");
  TQ_REQUIRE(ctx, m->lm_head != nullptr, "tq_llama_prefill: head weights not set");
  for (auto& L : m->layers) TQ_REQUIRE(ctx, L.wqkv != nullptr, "tq_llama_prefill: a layer has no weights");
  const size_t R = batch * q_len, d = c.d_model, hd = c.head_dim;
  const size_t q_dim = (size_t)m->heads_l * hd, kv_dim = (size_t)m->kv_l * hd;
  const size_t seq_stride = (size_t)c.max_seq * kv_dim;
  if (R > m->pre_rows) {   // (re)size the chunk's workspaces
    TQ_REQUIRE(ctx, !ctx->capturing, "tq_llama_prefill: workspaces must be sized before graph capture (run once eagerly)");
    TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->ws_generation++;   // graphs recorded over the old chunk buffers must not be replayed
    void** slots[] = {(void**)&m->p_h, (void**)&m->p_delta, (void**)&m->p_qkv, (void**)&m->p_gu, (void**)&m->p_xn,
                      (void**)&m->p_qb, (void**)&m->p_attn, (void**)&m->p_act, (void**)&m->p_last};
    const size_t bytes[] = {R * d * 4, R * d * 4, R * (q_dim + 2 * kv_dim) * 4, R * 2 * m->ffn_l * 4, R * d * 2,
                            R * q_dim * 2, R * q_dim * 2, R * (size_t)m->ffn_l * 2, (size_t)c.max_batch * d * 2};
    for (int i = 0; i < 9; ++i) {
      if (*slots[i]) {
        for (auto& o : m->owned)
          if (o == *slots[i]) o = nullptr;
        cudaFree(*slots[i]);
        *slots[i] = nullptr;
      }
      if (int st = dev_alloc(m, slots[i], bytes[i])) return st;
    }
    m->pre_rows = R;
  }
  int st;
#define TQ_STEP(expr) \
  if ((st = (expr)) != TQ_OK) return st;
  const int Ri = (int)R, B = (int)batch;
  TQ_STEP(tq_embedding(ctx, m->embed, TQ_BF16, token_ids_dev, R, d, c.vocab, m->p_h, TQ_F32));
  bool have_delta = false;
  for (size_t l = 0; l < m->layers.size(); ++l) {
    const LlamaLayerW& L = m->layers[l];
    TQ_STEP(tq_rms_norm(ctx, have_delta ? (const void*)m->p_delta : (const void*)m->p_h, TQ_F32, have_delta ? m->p_h : nullptr,
                        L.attn_norm, TQ_BF16, R, d, c.eps, m->p_xn, TQ_BF16, have_delta ? m->p_h : nullptr));
    TQ_STEP(tq_qlinear(ctx, L.wqkv, m->p_xn, TQ_BF16, d, R, m->p_qkv, TQ_F32, q_dim + 2 * kv_dim, nullptr));
    TQ_STEP(launch_qkv_post(ctx, m->p_qkv, m->cos_t, m->sin_t, cache_start_dev, nullptr, Ri, m->heads_l, m->kv_l, (int)hd, (int)c.max_seq,
                            m->p_qb, L.k_cache, L.v_cache, seq_stride, (int)q_len));
    TQ_STEP(tq_gqa_prefill(ctx, m->p_qb, L.k_cache, L.v_cache, cache_start_dev, batch, q_len, m->heads_l, m->kv_l, hd, seq_stride,
                           m->p_attn, TQ_BF16));
    TQ_STEP(tq_qlinear(ctx, L.wo, m->p_attn, TQ_BF16, q_dim, R, m->p_delta, TQ_F32, d, nullptr));
    TQ_STEP(tq_all_reduce_f32(ctx, m->comm, m->p_delta, R * d));
    TQ_STEP(tq_rms_norm(ctx, m->p_delta, TQ_F32, m->p_h, L.ffn_norm, TQ_BF16, R, d, c.eps, m->p_xn, TQ_BF16, m->p_h));
    if (L.wgu->gate_up_interleaved) {
      TQ_STEP(qlinear_fused(ctx, L.wgu, m->p_xn, nullptr, R, m->p_act, TQ_BF16, m->ffn_l, true, m->p_gu));
    } else {
      TQ_STEP(tq_qlinear(ctx, L.wgu, m->p_xn, TQ_BF16, d, R, m->p_gu, TQ_F32, 2 * (size_t)m->ffn_l, nullptr));
      TQ_STEP(tq_swiglu(ctx, m->p_gu, m->p_gu + m->ffn_l, TQ_F32, 2 * (size_t)m->ffn_l, R, m->ffn_l, m->p_act, TQ_BF16));
    }
    TQ_STEP(tq_qlinear(ctx, L.wdown, m->p_act, TQ_BF16, m->ffn_l, R, m->p_delta, TQ_F32, d, nullptr));
    TQ_STEP(tq_all_reduce_f32(ctx, m->comm, m->p_delta, R * d));
    have_delta = true;
  }
  TQ_STEP(tq_rms_norm(ctx, m->p_delta, TQ_F32, m->p_h, m->final_norm, TQ_BF16, R, d, c.eps, m->p_xn, TQ_BF16, m->p_h));
  // the LM head only sees each sequence's last row
  TQ_CUDA(ctx, cudaMemcpy2DAsync(m->p_last, d * 2, m->p_xn + (q_len - 1) * d, q_len * d * 2, d * 2, batch, cudaMemcpyDeviceToDevice,
                                 ctx->stream));
  if (m->tp == 1) {
    TQ_STEP(tq_qlinear(ctx, m->lm_head, m->p_last, TQ_BF16, d, B, logits_dev, TQ_F32, c.vocab, nullptr));
  } else {
    TQ_STEP(tq_qlinear(ctx, m->lm_head, m->p_last, TQ_BF16, d, B, m->logits_l, TQ_F32, m->vocab_l, nullptr));
    TQ_STEP(tq_all_gather(ctx, m->comm, m->logits_l, logits_dev, (size_t)B * m->vocab_l * sizeof(float)));
  }
#undef TQ_STEP
  return TQ_OK;
}

}  // extern "C"
