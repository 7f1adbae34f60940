// tang_oracle_models — CPU restatement of the layer compositions built on the quantised matvec.
//
// TEST INFRASTRUCTURE ONLY (see tang_oracle.cpp).  The Llama block follows the reference's one
// decode loop, crates/tang-train/examples/smollm.rs, step for step in f64, with the dense
// `matmul_weight` calls replaced by the quantised matvec of crates/tang-infer/src/quantize.rs.
// The MoE and MLA layers have no counterpart in the reference ("parity unpinned"); they are
// composed from the same primitives and their algebra is written out beside each function.
//
// Activation dtype contract.  The benchmark configurations fix activations and the KV cache to
// bf16.  Wherever the device path stores a bf16 tensor, this file rounds the f64 value to bf16
// (round-to-nearest-even, crates/tang-compute/src/cuda.rs:22-27) at the same point, so the two
// sides see identical inputs to every matvec; everything between two rounding points is f64.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#define ORC_API extern "C" __attribute__((visibility("default")))

extern "C" {
uint16_t orc_f32_to_bf16(float v);
float orc_bf16_to_f32(uint16_t bits);
void orc_qmatmul(int kind, const void* scales, const void* payload, size_t rows, size_t cols, const double* x,
                 size_t m, double* y, int threads);
void orc_rms_norm_f64(const double* x, const double* w, double* out, size_t n, double eps);
void orc_rope_heads_f64(const double* x, double* out, size_t n_heads, size_t head_dim, size_t pos, double base);
void orc_attention_decode_f64(const double* q, const double* k_cache, const double* v_cache, double* out,
                              size_t total_seq, size_t n_heads, size_t n_kv_heads, size_t head_dim, int threads);
void orc_swiglu_f64(const double* gate, const double* up, double* out, size_t n);
void orc_topk_indices_f64(const double* v, size_t n, size_t k, int32_t* idx_out);
}

namespace {

inline double round_bf16(double v) { return (double)orc_bf16_to_f32(orc_f32_to_bf16((float)v)); }

inline void round_bf16_inplace(std::vector<double>& v) {
  for (double& e : v) e = round_bf16(e);
}

}  // namespace

// One quantised weight matrix [rows, cols]: `kind` as in orc_qmatmul.
struct OrcQWeight {
  int32_t kind;
  int32_t _pad;
  const void* scales;
  const void* payload;
  uint64_t rows;
  uint64_t cols;
};

// Weights of one Llama block, in the reference's order [wq, wk, wv, wo, gate, up, down]
// (crates/tang-mesh/src/inference.rs:1306-1413 uses the same order), plus the two norm gains
// as bf16 bit patterns.
struct OrcLlamaLayer {
  OrcQWeight wq, wk, wv, wo, gate, up, down;
  const uint16_t* attn_norm_bf16;
  const uint16_t* ffn_norm_bf16;
};

struct OrcLlamaDims {
  uint64_t d_model, n_heads, n_kv_heads, head_dim, ffn;
  double rope_base;
  double eps;
};

// smollm.rs:215-231 (LlamaBlock::forward) with :72-159 (attention) and :181-191 (MLP), for ONE
// new token at position `pos` of ONE sequence.  `hidden` [d_model] is updated in place.
// k_cache / v_cache are this layer's bf16 caches, [max_seq, n_kv_heads*head_dim] row-major
// (crates/tang-infer/src/kv_cache.rs:12-24); row `pos` is written (append, kv_cache.rs:76-107)
// and rows 0..=pos are attended.
// After KVCache::trim_to (kv_cache.rs:138-149) the row a token is appended at (the cache's seq_len, `pos` here)
// and the position its rotation uses (the caller's running count, `rope_pos`) are no longer the same number.
ORC_API void orc_llama_layer_at_f64(const OrcLlamaDims* dims, const OrcLlamaLayer* L, double* hidden,
                                    uint16_t* k_cache, uint16_t* v_cache, uint64_t pos, uint64_t rope_pos, int threads);
ORC_API void orc_llama_layer_f64(const OrcLlamaDims* dims, const OrcLlamaLayer* L, double* hidden,
                                 uint16_t* k_cache, uint16_t* v_cache, uint64_t pos, int threads) {
  orc_llama_layer_at_f64(dims, L, hidden, k_cache, v_cache, pos, pos, threads);
}
ORC_API void orc_llama_layer_at_f64(const OrcLlamaDims* dims, const OrcLlamaLayer* L, double* hidden,
                                    uint16_t* k_cache, uint16_t* v_cache, uint64_t pos, uint64_t rope_pos, int threads) {
  const size_t d = dims->d_model, nh = dims->n_heads, nkv = dims->n_kv_heads, hd = dims->head_dim;
  const size_t kv_dim = nkv * hd, q_dim = nh * hd, ffn = dims->ffn;

  std::vector<double> w(d), normed(d);
  for (size_t i = 0; i < d; ++i) w[i] = (double)orc_bf16_to_f32(L->attn_norm_bf16[i]);
  orc_rms_norm_f64(hidden, w.data(), normed.data(), d, dims->eps);
  round_bf16_inplace(normed);  // bf16 activation entering q/k/v

  std::vector<double> q(q_dim), k(kv_dim), v(kv_dim), qr(q_dim), kr(kv_dim);
  orc_qmatmul(L->wq.kind, L->wq.scales, L->wq.payload, q_dim, d, normed.data(), 1, q.data(), threads);
  orc_qmatmul(L->wk.kind, L->wk.scales, L->wk.payload, kv_dim, d, normed.data(), 1, k.data(), threads);
  orc_qmatmul(L->wv.kind, L->wv.scales, L->wv.payload, kv_dim, d, normed.data(), 1, v.data(), threads);
  orc_rope_heads_f64(q.data(), qr.data(), nh, hd, rope_pos, dims->rope_base);
  orc_rope_heads_f64(k.data(), kr.data(), nkv, hd, rope_pos, dims->rope_base);
  round_bf16_inplace(qr);  // bf16 query entering attention

  for (size_t i = 0; i < kv_dim; ++i) {  // cache.append: bf16 storage
    k_cache[pos * kv_dim + i] = orc_f32_to_bf16((float)kr[i]);
    v_cache[pos * kv_dim + i] = orc_f32_to_bf16((float)v[i]);
  }
  size_t total = pos + 1;
  std::vector<double> kc(total * kv_dim), vc(total * kv_dim);
  for (size_t i = 0; i < total * kv_dim; ++i) {
    kc[i] = (double)orc_bf16_to_f32(k_cache[i]);
    vc[i] = (double)orc_bf16_to_f32(v_cache[i]);
  }
  std::vector<double> attn(q_dim);
  orc_attention_decode_f64(qr.data(), kc.data(), vc.data(), attn.data(), total, nh, nkv, hd, threads);
  round_bf16_inplace(attn);  // bf16 activation entering o_proj

  std::vector<double> o(d);
  orc_qmatmul(L->wo.kind, L->wo.scales, L->wo.payload, d, q_dim, attn.data(), 1, o.data(), threads);
  for (size_t i = 0; i < d; ++i) hidden[i] += o[i];

  for (size_t i = 0; i < d; ++i) w[i] = (double)orc_bf16_to_f32(L->ffn_norm_bf16[i]);
  orc_rms_norm_f64(hidden, w.data(), normed.data(), d, dims->eps);
  round_bf16_inplace(normed);  // bf16 activation entering gate/up

  std::vector<double> g(ffn), u(ffn), act(ffn), dn(d);
  orc_qmatmul(L->gate.kind, L->gate.scales, L->gate.payload, ffn, d, normed.data(), 1, g.data(), threads);
  orc_qmatmul(L->up.kind, L->up.scales, L->up.payload, ffn, d, normed.data(), 1, u.data(), threads);
  orc_swiglu_f64(g.data(), u.data(), act.data(), ffn);
  round_bf16_inplace(act);  // bf16 activation entering down
  orc_qmatmul(L->down.kind, L->down.scales, L->down.payload, d, ffn, act.data(), 1, dn.data(), threads);
  for (size_t i = 0; i < d; ++i) hidden[i] += dn[i];
}

// KVCache::trim_to (crates/tang-infer/src/kv_cache.rs:138-149) on one layer's cache rows [seq_len, kv_dim] (any 16-bit
// element): the first seq_len - keep rows are drained, the rest move to the front.  Returns the new seq_len.
ORC_API uint64_t orc_kv_trim_to(uint16_t* rows, uint64_t seq_len, uint64_t kv_dim, uint64_t keep) {
  if (seq_len <= keep) return seq_len;
  const uint64_t drop_elems = (seq_len - keep) * kv_dim;
  std::memmove(rows, rows + drop_elems, keep * kv_dim * sizeof(uint16_t));
  return keep;
}

// smollm.rs:255-296 tail: final RMSNorm, then the LM head on the (single) last row.
ORC_API void orc_llama_head_f64(const OrcLlamaDims* dims, const uint16_t* final_norm_bf16, const OrcQWeight* lm_head,
                                const double* hidden, double* logits, int threads) {
  const size_t d = dims->d_model;
  std::vector<double> w(d), normed(d);
  for (size_t i = 0; i < d; ++i) w[i] = (double)orc_bf16_to_f32(final_norm_bf16[i]);
  orc_rms_norm_f64(hidden, w.data(), normed.data(), d, dims->eps);
  round_bf16_inplace(normed);
  orc_qmatmul(lm_head->kind, lm_head->scales, lm_head->payload, lm_head->rows, d, normed.data(), 1, logits, threads);
}

// ---------------------------------------------------------------------------------------------
// Mixture-of-experts FFN (no reference counterpart; parity unpinned)
//
//   logits_e = sum_k h_k * Wg[e,k]                (f64, k ascending)
//   chosen   = top-k of logits by (value desc, index asc)      -> orc_topk_indices_f64
//   p_e      = exp(logits_e - max) / sum_all exp(logits - max) (softmax over ALL routed experts;
//              optionally renormalised over the chosen ones)
//   expert(h)= down( bf16( silu(gate h) * (up h) ) )           (SwiGLU as smollm.rs:181-191)
//   out      = sum_{e in chosen} p_e * expert_e(h) + sum_{s in shared} expert_s(h)
// Selecting on logits instead of on exp(logits - max) picks the same experts (exp is monotone)
// without depending on a libm.
// ---------------------------------------------------------------------------------------------

ORC_API void orc_router_f64(const double* h, const double* wg, size_t n_experts, size_t d, size_t top_k,
                            int renormalize, int32_t* idx_out, double* weight_out, double* logits_out) {
  std::vector<double> logits(n_experts);
  for (size_t e = 0; e < n_experts; ++e) {
    double s = 0.0;
    for (size_t k = 0; k < d; ++k) s += h[k] * wg[e * d + k];
    logits[e] = s;
  }
  if (logits_out) std::memcpy(logits_out, logits.data(), n_experts * sizeof(double));
  orc_topk_indices_f64(logits.data(), n_experts, top_k, idx_out);
  double mx = -std::numeric_limits<double>::infinity();
  for (size_t e = 0; e < n_experts; ++e) mx = std::fmax(mx, logits[e]);
  double sum = 0.0;
  for (size_t e = 0; e < n_experts; ++e) sum += std::exp(logits[e] - mx);
  double chosen_sum = 0.0;
  for (size_t i = 0; i < top_k; ++i) {
    weight_out[i] = std::exp(logits[idx_out[i]] - mx) / sum;
    chosen_sum += weight_out[i];
  }
  if (renormalize)
    for (size_t i = 0; i < top_k; ++i) weight_out[i] /= chosen_sum;
}

// One SwiGLU expert applied to one token: out[d] = down(bf16(silu(gate x) * (up x))).
ORC_API void orc_expert_ffn_f64(const OrcQWeight* gate, const OrcQWeight* up, const OrcQWeight* down,
                                const double* x, double* out, int threads) {
  size_t ffn = gate->rows, d = gate->cols;
  std::vector<double> g(ffn), u(ffn), act(ffn);
  orc_qmatmul(gate->kind, gate->scales, gate->payload, ffn, d, x, 1, g.data(), threads);
  orc_qmatmul(up->kind, up->scales, up->payload, ffn, d, x, 1, u.data(), threads);
  orc_swiglu_f64(g.data(), u.data(), act.data(), ffn);
  round_bf16_inplace(act);
  orc_qmatmul(down->kind, down->scales, down->payload, down->rows, ffn, act.data(), 1, out, threads);
}

// ---------------------------------------------------------------------------------------------
// Multi-head latent attention, decode step (no reference counterpart; parity unpinned)
//
// Per sequence the cache row of position j is [c_j (kv_lora) | r_j (rope_dim)] in bf16.  The
// projections are stored ABSORBED and quantised per output row (int8 with one f32 scale per row,
// dequantised as crates/tang-infer/src/quantize.rs:73-81 does: v as f32 * scale; matvec order as
// quantize.rs:227-253):
//   W_qk[h] : [kv_lora, nope]   q_lat = W_qk[h] q_nope          (= W_UK[h]^T of the unabsorbed model)
//   W_uv[h] : [v_dim, kv_lora]  o     = W_uv[h] o_lat
//
//   absorbed: q_lat = bf16(W_qk[h] q_nope),  s_j = (q_lat.c_j + q_rope.r_j) * scale,
//             o_lat = bf16(sum_j softmax(s)_j c_j),  o = W_uv[h] o_lat
//   naive:    k_j = W_qk[h]^T c_j,  s_j = (q_nope.k_j + q_rope.r_j) * scale,
//             v_j = W_uv[h] c_j,    o = sum_j softmax(s)_j v_j
// with scale = 1/sqrt(nope + rope_dim).  The two agree exactly in real arithmetic; the absorbed
// form (what the device runs) adds the two bf16 roundings marked above.  `absorbed` selects the
// form, so a test can bound their gap.
// ---------------------------------------------------------------------------------------------

struct OrcMlaDims {
  uint64_t n_heads, kv_lora, nope, rope_dim, v_dim;
};

ORC_API void orc_mla_decode_f64(const OrcMlaDims* dm, const double* q_nope, const double* q_rope,
                                const uint16_t* cache_bf16, uint64_t ctx, const int8_t* w_qk,
                                const float* w_qk_scale, const int8_t* w_uv, const float* w_uv_scale,
                                int absorbed, double* out, int threads) {
  const size_t H = dm->n_heads, C = dm->kv_lora, Dn = dm->nope, Dr = dm->rope_dim, Dv = dm->v_dim;
  const size_t row = C + Dr;
  const double scale = 1.0 / std::sqrt((double)(Dn + Dr));
  (void)threads;
#pragma omp parallel for schedule(static)
  for (long long hh = 0; hh < (long long)H; ++hh) {
    size_t h = (size_t)hh;
    const int8_t* qk = w_qk + h * C * Dn;
    const float* qks = w_qk_scale + h * C;
    const int8_t* uv = w_uv + h * Dv * C;
    const float* uvs = w_uv_scale + h * Dv;
    const double* qn = q_nope + h * Dn;
    const double* qr = q_rope + h * Dr;
    std::vector<double> s(ctx);
    std::vector<double> q_lat(C, 0.0);
    if (absorbed) {
      for (size_t c = 0; c < C; ++c) {
        double acc = 0.0;
        const double sc = (double)qks[c];
        for (size_t dd = 0; dd < Dn; ++dd) acc += (double)qk[c * Dn + dd] * sc * qn[dd];
        q_lat[c] = round_bf16(acc);
      }
    }
    std::vector<double> kj(Dn);
    for (size_t j = 0; j < ctx; ++j) {
      const uint16_t* cr = cache_bf16 + j * row;
      double dot = 0.0;
      if (absorbed) {
        for (size_t c = 0; c < C; ++c) dot += q_lat[c] * (double)orc_bf16_to_f32(cr[c]);
      } else {
        for (size_t dd = 0; dd < Dn; ++dd) kj[dd] = 0.0;
        for (size_t c = 0; c < C; ++c) {
          const double cv = (double)orc_bf16_to_f32(cr[c]) * (double)qks[c];
          for (size_t dd = 0; dd < Dn; ++dd) kj[dd] += (double)qk[c * Dn + dd] * cv;
        }
        for (size_t dd = 0; dd < Dn; ++dd) dot += qn[dd] * kj[dd];
      }
      for (size_t r = 0; r < Dr; ++r) dot += qr[r] * (double)orc_bf16_to_f32(cr[C + r]);
      s[j] = dot * scale;
    }
    double mx = -std::numeric_limits<double>::infinity();
    for (size_t j = 0; j < ctx; ++j) mx = std::fmax(mx, s[j]);
    double sum = 0.0;
    for (size_t j = 0; j < ctx; ++j) {
      s[j] = std::exp(s[j] - mx);
      sum += s[j];
    }
    for (size_t j = 0; j < ctx; ++j) s[j] /= sum;
    if (absorbed) {
      std::vector<double> o_lat(C, 0.0);
      for (size_t j = 0; j < ctx; ++j) {
        const uint16_t* cr = cache_bf16 + j * row;
        for (size_t c = 0; c < C; ++c) o_lat[c] += s[j] * (double)orc_bf16_to_f32(cr[c]);
      }
      for (size_t c = 0; c < C; ++c) o_lat[c] = round_bf16(o_lat[c]);
      for (size_t dv = 0; dv < Dv; ++dv) {
        double acc = 0.0;
        const double sc = (double)uvs[dv];
        for (size_t c = 0; c < C; ++c) acc += (double)uv[dv * C + c] * sc * o_lat[c];
        out[h * Dv + dv] = acc;
      }
    } else {
      for (size_t dv = 0; dv < Dv; ++dv) out[h * Dv + dv] = 0.0;
      std::vector<double> vj(Dv);
      for (size_t j = 0; j < ctx; ++j) {
        const uint16_t* cr = cache_bf16 + j * row;
        for (size_t dv = 0; dv < Dv; ++dv) {
          double acc = 0.0;
          const double sc = (double)uvs[dv];
          for (size_t c = 0; c < C; ++c) acc += (double)uv[dv * C + c] * sc * (double)orc_bf16_to_f32(cr[c]);
          vj[dv] = acc;
        }
        for (size_t dv = 0; dv < Dv; ++dv) out[h * Dv + dv] += s[j] * vj[dv];
      }
    }
  }
}
