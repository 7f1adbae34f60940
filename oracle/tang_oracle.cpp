// tang_oracle — CPU restatement of the reference's quantized decode path.
//
// TEST INFRASTRUCTURE ONLY.  This file is the parity checker for the CUDA library: the test
// suite, the smoke check and the benchmark's CPU-baseline leg load it; the product library
// never links, loads or calls it.
//
// Every function restates, in plain scalar loops, one function of ecto/tang's CPU code and
// names the file:line it follows (paths are relative to the reference project root).  The
// reference is Rust and cannot be compiled in this environment, so nothing here is generated
// from it; arithmetic order, rounding mode and integer rules are reproduced by hand.  Compile
// with -ffp-contract=off and without -ffast-math so that f32/f64 expressions evaluate exactly
// as written (Rust never contracts a*b+c into an FMA).
//
// Parity status: the quantize/dequantize/matvec and CpuDevice functions are pinned against
// the reference's own unit-test cases (tests/test_oracle_pins.py replays them).  The MoE and
// MLA functions have no counterpart in the reference ("parity unpinned"): they are composed
// from the pinned primitives and cross-checked against an independent formulation.
//
// Threading: `threads` arguments parallelise over OUTPUT ROWS only (OpenMP); each row keeps
// the reference's sequential summation order, so results do not depend on the thread count.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t kBlock = 32;  // crates/tang-infer/src/quantize.rs:11  BLOCK_SIZE

inline int clamp_threads(int threads) {
#ifdef _OPENMP
  if (threads <= 0) return omp_get_max_threads();
  return threads;
#else
  (void)threads;
  return 1;
#endif
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Scalar format conversions
// ---------------------------------------------------------------------------------------------

// crates/tang-safetensors/src/lib.rs:262-293  f16_to_f32 (subnormals normalised by shifting,
// inf/nan keep the mantissa bits).
ORC_API float orc_f16_to_f32(uint16_t bits) {
  uint32_t sign = (bits >> 15) & 1u;
  uint32_t exp = (bits >> 10) & 0x1Fu;
  uint32_t mant = bits & 0x3FFu;
  uint32_t out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign << 31;
    } else {
      uint32_t m = mant;
      int e = 0;
      while ((m & 0x400u) == 0) {
        m <<= 1;
        e -= 1;
      }
      m &= 0x3FFu;
      uint32_t f32_exp = (uint32_t)(127 - 15 + 1 + e);
      out = (sign << 31) | (f32_exp << 23) | (m << 13);
    }
  } else if (exp == 31) {
    out = (sign << 31) | (0xFFu << 23) | (mant << 13);
  } else {
    out = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

// crates/tang-compute/src/cuda.rs:22-27  f32_to_bf16: round to nearest even by adding
// 0x7FFF + lsb and truncating (wrapping add, so NaN/inf payloads follow the same rule).
ORC_API uint16_t orc_f32_to_bf16(float v) {
  uint32_t bits;
  std::memcpy(&bits, &v, 4);
  uint32_t lsb = (bits >> 16) & 1u;
  uint32_t rounded = bits + (0x7FFFu + lsb);
  return (uint16_t)(rounded >> 16);
}

// crates/tang-compute/src/cuda.rs:29-31 and crates/tang-safetensors/src/lib.rs:295-297.
ORC_API float orc_bf16_to_f32(uint16_t bits) {
  uint32_t u = (uint32_t)bits << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// f32 -> f16, round to nearest even.  The reference only READS f16; this exists so tests can
// produce f16 scale tables.  It is the inverse of orc_f16_to_f32 on every representable value.
ORC_API uint16_t orc_f32_to_f16(float v) {
  uint32_t x;
  std::memcpy(&x, &v, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
  uint32_t mant = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u | (mant >> 13) : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    mant |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - exp);
    uint32_t half = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) half += 1;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (mant >> 13);
  uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half += 1;
  return (uint16_t)(sign | half);
}

ORC_API void orc_round_to_bf16_f32(const float* in, size_t n, float* out) {
  for (size_t i = 0; i < n; ++i) out[i] = orc_bf16_to_f32(orc_f32_to_bf16(in[i]));
}

// ---------------------------------------------------------------------------------------------
// Block quantisation (crates/tang-infer/src/quantize.rs)
//
// Block storage here is structure-of-arrays: `scales[b]` and 32 (Q8) or 16 (Q4) payload bytes
// per block, blocks in the reference's order (row-major, ceil(cols/32) blocks per row).
// ---------------------------------------------------------------------------------------------

// quantize.rs:47-71  quantize_q8: amax/127 scale (1.0 for an all-zero block), f32 multiply by
// the reciprocal, round half away from zero, clamp to [-128,127]; the ragged tail is zero.
ORC_API void orc_quantize_q8(const float* data, size_t n, float* scales, int8_t* values) {
  size_t n_blocks = (n + kBlock - 1) / kBlock;
  for (size_t b = 0; b < n_blocks; ++b) {
    size_t start = b * kBlock;
    size_t end = std::min(start + kBlock, n);
    float amax = 0.0f;
    for (size_t i = start; i < end; ++i) amax = std::fmax(amax, std::fabs(data[i]));
    float scale = (amax == 0.0f) ? 1.0f : amax / 127.0f;
    float inv_scale = 1.0f / scale;
    int8_t* out = values + b * kBlock;
    for (size_t i = 0; i < kBlock; ++i) out[i] = 0;
    for (size_t i = start; i < end; ++i) {
      float r = std::round(data[i] * inv_scale);
      // f32::clamp keeps NaN and `NaN as i8` is 0; fmin/fmax would turn the NaN into a bound
      out[i - start] = std::isnan(r) ? (int8_t)0 : (int8_t)std::fmin(std::fmax(r, -128.0f), 127.0f);
    }
    scales[b] = scale;
  }
}

// quantize.rs:73-81  dequantize_q8: value as f32 times the block scale.
ORC_API void orc_dequantize_q8(const float* scales, const int8_t* values, size_t n_blocks, float* out) {
  for (size_t b = 0; b < n_blocks; ++b)
    for (size_t i = 0; i < kBlock; ++i) out[b * kBlock + i] = (float)values[b * kBlock + i] * scales[b];
}

// quantize.rs:84-118  quantize_q4: amax/7 scale, round half away, clamp to [-8,7], store q+8;
// byte i = (q[2i]+8) | (q[2i+1]+8)<<4; positions past the end of the data hold q=0 (nibble 8).
ORC_API void orc_quantize_q4(const float* data, size_t n, float* scales, uint8_t* packed) {
  size_t n_blocks = (n + kBlock - 1) / kBlock;
  for (size_t b = 0; b < n_blocks; ++b) {
    size_t start = b * kBlock;
    size_t end = std::min(start + kBlock, n);
    size_t len = end - start;
    float amax = 0.0f;
    for (size_t i = start; i < end; ++i) amax = std::fmax(amax, std::fabs(data[i]));
    float scale = (amax == 0.0f) ? 1.0f : amax / 7.0f;
    float inv_scale = 1.0f / scale;
    for (size_t i = 0; i < kBlock / 2; ++i) {
      size_t idx = i * 2;
      int v0 = 0, v1 = 0;
      if (idx < len) {
        float r = std::round(data[start + idx] * inv_scale);
        v0 = std::isnan(r) ? 0 : (int)std::fmin(std::fmax(r, -8.0f), 7.0f);   // `NaN.clamp(..) as i8` is 0
      }
      if (idx + 1 < len) {
        float r = std::round(data[start + idx + 1] * inv_scale);
        v1 = std::isnan(r) ? 0 : (int)std::fmin(std::fmax(r, -8.0f), 7.0f);
      }
      packed[b * (kBlock / 2) + i] = (uint8_t)((uint8_t)(v0 + 8) | ((uint8_t)(v1 + 8) << 4));
    }
    scales[b] = scale;
  }
}

// quantize.rs:121-132  dequantize_q4: low nibble first, each nibble minus 8, times the scale.
ORC_API void orc_dequantize_q4(const float* scales, const uint8_t* packed, size_t n_blocks, float* out) {
  for (size_t b = 0; b < n_blocks; ++b) {
    for (size_t i = 0; i < kBlock / 2; ++i) {
      uint8_t byte = packed[b * (kBlock / 2) + i];
      int v0 = (int)(int8_t)(byte & 0x0F) - 8;
      int v1 = (int)(int8_t)((byte >> 4) & 0x0F) - 8;
      out[b * kBlock + 2 * i] = (float)v0 * scales[b];
      out[b * kBlock + 2 * i + 1] = (float)v1 * scales[b];
    }
  }
}

// quantize.rs:121-126 integer part only: the signed 4-bit values, for bit-exact unpack checks.
ORC_API void orc_unpack_q4(const uint8_t* packed, size_t n_bytes, int8_t* out) {
  for (size_t i = 0; i < n_bytes; ++i) {
    out[2 * i] = (int8_t)((int)(packed[i] & 0x0F) - 8);
    out[2 * i + 1] = (int8_t)((int)((packed[i] >> 4) & 0x0F) - 8);
  }
}

// quantize.rs:193-205  quantize_matrix_q8: each row quantised on its own so no block spans rows.
ORC_API void orc_quantize_matrix_q8(const float* data, size_t rows, size_t cols, float* scales, int8_t* values) {
  size_t bpr = (cols + kBlock - 1) / kBlock;
  for (size_t r = 0; r < rows; ++r)
    orc_quantize_q8(data + r * cols, cols, scales + r * bpr, values + r * bpr * kBlock);
}

// quantize.rs:208-220  quantize_matrix_q4.
ORC_API void orc_quantize_matrix_q4(const float* data, size_t rows, size_t cols, float* scales, uint8_t* packed) {
  size_t bpr = (cols + kBlock - 1) / kBlock;
  for (size_t r = 0; r < rows; ++r)
    orc_quantize_q4(data + r * cols, cols, scales + r * bpr, packed + r * bpr * (kBlock / 2));
}

// quantize.rs:227-253  q8_matvec: per row, per block, per element, in that order:
// sum += (v as f64) * (scale as f64) * x[k], skipping k >= in_dim; f64 throughout.
ORC_API void orc_q8_matvec(const float* scales, const int8_t* values, size_t rows, size_t cols,
                           const double* x, double* y, int threads) {
  size_t bpr = (cols + kBlock - 1) / kBlock;
  int nt = clamp_threads(threads);
  (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static)
  for (long long row = 0; row < (long long)rows; ++row) {
    double sum = 0.0;
    for (size_t b = 0; b < bpr; ++b) {
      const int8_t* v = values + ((size_t)row * bpr + b) * kBlock;
      double scale = (double)scales[(size_t)row * bpr + b];
      size_t x_start = b * kBlock;
      for (size_t i = 0; i < kBlock; ++i) {
        size_t xi = x_start + i;
        if (xi < cols) sum += (double)v[i] * scale * x[xi];
      }
    }
    y[row] = sum;
  }
}

// quantize.rs:256-289  q4_matvec: as q8_matvec with the nibble unpack of dequantize_q4; the two
// values of a byte are added one after the other (even index first).
ORC_API void orc_q4_matvec(const float* scales, const uint8_t* packed, size_t rows, size_t cols,
                           const double* x, double* y, int threads) {
  size_t bpr = (cols + kBlock - 1) / kBlock;
  int nt = clamp_threads(threads);
  (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static)
  for (long long row = 0; row < (long long)rows; ++row) {
    double sum = 0.0;
    for (size_t b = 0; b < bpr; ++b) {
      const uint8_t* p = packed + ((size_t)row * bpr + b) * (kBlock / 2);
      double scale = (double)scales[(size_t)row * bpr + b];
      size_t x_start = b * kBlock;
      for (size_t i = 0; i < kBlock / 2; ++i) {
        uint8_t byte = p[i];
        double v0 = (double)((int)(int8_t)(byte & 0x0F) - 8);
        double v1 = (double)((int)(int8_t)((byte >> 4) & 0x0F) - 8);
        size_t xi0 = x_start + i * 2;
        size_t xi1 = xi0 + 1;
        if (xi0 < cols) sum += v0 * scale * x[xi0];
        if (xi1 < cols) sum += v1 * scale * x[xi1];
      }
    }
    y[row] = sum;
  }
}

// The two weight forms the benchmark configurations add to tang-infer's native blocks.  They
// follow q4_matvec / q8_matvec term by term; only where the scale comes from differs.

// Q4 blocks whose scale is stored as IEEE half: widen with orc_f16_to_f32, then q4_matvec.
ORC_API void orc_q4_f16scale_matvec(const uint16_t* scales_f16, const uint8_t* packed, size_t rows,
                                    size_t cols, const double* x, double* y, int threads) {
  size_t bpr = (cols + kBlock - 1) / kBlock;
  std::vector<float> scales(rows * bpr);
  for (size_t i = 0; i < rows * bpr; ++i) scales[i] = orc_f16_to_f32(scales_f16[i]);
  orc_q4_matvec(scales.data(), packed, rows, cols, x, y, threads);
}

// int8 weights [rows, cols] with ONE f32 scale per output row: q8_matvec with every block of a
// row sharing that row's scale.
ORC_API void orc_q8_rowscale_matvec(const float* row_scales, const int8_t* w, size_t rows, size_t cols,
                                    const double* x, double* y, int threads) {
  int nt = clamp_threads(threads);
  (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static)
  for (long long row = 0; row < (long long)rows; ++row) {
    double sum = 0.0;
    double scale = (double)row_scales[row];
    const int8_t* v = w + (size_t)row * cols;
    for (size_t k = 0; k < cols; ++k) sum += (double)v[k] * scale * x[k];
    y[row] = sum;
  }
}

// M activation rows = M independent matvecs (the reference has no quantised GEMM; a batch is a
// loop over q4_matvec).  x is [m, cols], y is [m, rows].  kind: 0 = Q4 f32 block scales,
// 1 = Q4 f16 block scales, 2 = Q8 f32 block scales, 3 = int8 with per-row f32 scale.
ORC_API void orc_qmatmul(int kind, const void* scales, const void* payload, size_t rows, size_t cols,
                         const double* x, size_t m, double* y, int threads) {
  for (size_t t = 0; t < m; ++t) {
    const double* xt = x + t * cols;
    double* yt = y + t * rows;
    switch (kind) {
      case 0: orc_q4_matvec((const float*)scales, (const uint8_t*)payload, rows, cols, xt, yt, threads); break;
      case 1: orc_q4_f16scale_matvec((const uint16_t*)scales, (const uint8_t*)payload, rows, cols, xt, yt, threads); break;
      case 2: orc_q8_matvec((const float*)scales, (const int8_t*)payload, rows, cols, xt, yt, threads); break;
      default: orc_q8_rowscale_matvec((const float*)scales, (const int8_t*)payload, rows, cols, xt, yt, threads); break;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// CpuDevice operators (crates/tang-compute/src/cpu.rs), f32 as the reference computes them
// ---------------------------------------------------------------------------------------------

// cpu.rs:99-103,760-770  matmul / naive_matmul: C[m,n] = A[m,k]·B[k,n], f32, k innermost.
ORC_API void orc_matmul_f32(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (size_t p = 0; p < k; ++p) sum += a[i * k + p] * b[p * n + j];
      c[i * n + j] = sum;
    }
}

// device.rs:407-419  matmul_b_transposed default: transpose B[n,k] then matmul; the sums are the
// same sequence as reading B by rows, which is what this does.
ORC_API void orc_matmul_b_transposed_f32(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (size_t p = 0; p < k; ++p) sum += a[i * k + p] * b[j * k + p];
      c[i * n + j] = sum;
    }
}

// cpu.rs:105-124  softmax: subtract the row max, exp, sum, multiply by the reciprocal.
ORC_API void orc_softmax_f32(const float* in, float* out, size_t n_rows, size_t row_len) {
  for (size_t r = 0; r < n_rows; ++r) {
    const float* src = in + r * row_len;
    float* dst = out + r * row_len;
    float mx = -std::numeric_limits<float>::infinity();
    for (size_t i = 0; i < row_len; ++i) mx = std::fmax(mx, src[i]);
    for (size_t i = 0; i < row_len; ++i) dst[i] = std::exp(src[i] - mx);
    float sum = 0.0f;
    for (size_t i = 0; i < row_len; ++i) sum += dst[i];
    float inv = 1.0f / sum;
    for (size_t i = 0; i < row_len; ++i) dst[i] *= inv;
  }
}

// cpu.rs:126-149  rms_norm: x * (1/sqrt(mean(x^2)+eps)) * w, all f32, sum in index order.
ORC_API void orc_rms_norm_f32(const float* data, const float* weight, float* out, size_t n_groups,
                              size_t dim, float eps) {
  for (size_t g = 0; g < n_groups; ++g) {
    const float* s = data + g * dim;
    float sq = 0.0f;
    for (size_t d = 0; d < dim; ++d) sq += s[d] * s[d];
    float rms = std::sqrt(sq / (float)dim + eps);
    float inv = 1.0f / rms;
    for (size_t d = 0; d < dim; ++d) out[g * dim + d] = s[d] * inv * weight[d];
  }
}

// device.rs:546-575  rms_norm_residual default: sum = input + residual, normalise the sum.
ORC_API void orc_rms_norm_residual_f32(const float* input, const float* residual, const float* weight,
                                       float* out, float* sum_out, size_t n_groups, size_t dim, float eps) {
  for (size_t g = 0; g < n_groups; ++g) {
    size_t base = g * dim;
    float sq = 0.0f;
    for (size_t i = 0; i < dim; ++i) {
      float v = input[base + i] + residual[base + i];
      sum_out[base + i] = v;
      sq += v * v;
    }
    float inv = 1.0f / std::sqrt(sq / (float)dim + eps);
    for (size_t i = 0; i < dim; ++i) out[base + i] = sum_out[base + i] * inv * weight[i];
  }
}

// cpu.rs:151-167  embedding: row gather (ids given as integers here, not f32 bit patterns).
ORC_API void orc_embedding_f32(const float* weight, const uint32_t* ids, float* out, size_t seq_len, size_t dim) {
  for (size_t i = 0; i < seq_len; ++i)
    std::memcpy(out + i * dim, weight + (size_t)ids[i] * dim, dim * sizeof(float));
}

// cpu.rs:257-315  kv_attention: per query and head, one pass over positions 0..cache_start+qi
// with a running max / running sum / rescaled accumulator, all f32.  kv_head = head / (n_heads /
// n_kv_heads).  Cache rows are [position, n_kv_heads*head_dim].
ORC_API void orc_kv_attention_f32(const float* q, const float* k_cache, const float* v_cache, float* out,
                                  size_t cache_start, size_t q_len, size_t n_heads, size_t n_kv_heads,
                                  size_t head_dim) {
  size_t total_dim = n_heads * head_dim;
  size_t kv_dim = n_kv_heads * head_dim;
  size_t heads_per_kv = n_heads / n_kv_heads;
  float scale = 1.0f / std::sqrt((float)head_dim);
  std::vector<float> accum(head_dim);
  for (size_t qi = 0; qi < q_len; ++qi) {
    size_t attend_len = cache_start + qi + 1;
    for (size_t h = 0; h < n_heads; ++h) {
      size_t kv_h = h / heads_per_kv;
      size_t q_off = qi * total_dim + h * head_dim;
      size_t kv_off = kv_h * head_dim;
      float running_max = -std::numeric_limits<float>::infinity();
      float running_sum = 0.0f;
      std::fill(accum.begin(), accum.end(), 0.0f);
      for (size_t j = 0; j < attend_len; ++j) {
        float dot = 0.0f;
        for (size_t d = 0; d < head_dim; ++d) dot += q[q_off + d] * k_cache[j * kv_dim + kv_off + d];
        float score = dot * scale;
        float new_max = std::fmax(running_max, score);
        float exp_score = std::exp(score - new_max);
        float rescale = std::exp(running_max - new_max);
        running_sum = running_sum * rescale + exp_score;
        for (size_t d = 0; d < head_dim; ++d)
          accum[d] = accum[d] * rescale + exp_score * v_cache[j * kv_dim + kv_off + d];
        running_max = new_max;
      }
      float inv = 1.0f / running_sum;
      for (size_t d = 0; d < head_dim; ++d) out[q_off + d] = accum[d] * inv;
    }
  }
}

// modules.rs:495-510  InterleavedRoPE::new: freq_i = 1/base^(i/half) in f64, angle = pos*freq,
// cos/sin taken in f64 and stored as f32.  Tables are [max_seq_len, head_dim/2].
ORC_API void orc_rope_tables_f32(size_t head_dim, size_t max_seq_len, double base, float* cos_table, float* sin_table) {
  size_t half = head_dim / 2;
  for (size_t pos = 0; pos < max_seq_len; ++pos)
    for (size_t i = 0; i < half; ++i) {
      double freq = 1.0 / std::pow(base, (double)i / (double)half);
      double angle = (double)pos * freq;
      cos_table[pos * half + i] = (float)std::cos(angle);
      sin_table[pos * half + i] = (float)std::sin(angle);
    }
}

// device.rs:582-610  rope_forward default: input [seq, n_heads, head_dim]; pair (2i, 2i+1) of
// every head rotated by the table entry of position start_pos+s.
ORC_API void orc_rope_forward_f32(const float* in, float* out, const float* cos_table, const float* sin_table,
                                  size_t seq_len, size_t n_heads, size_t head_dim, size_t start_pos) {
  size_t half = head_dim / 2;
  for (size_t s = 0; s < seq_len; ++s) {
    size_t pos = start_pos + s;
    for (size_t h = 0; h < n_heads; ++h) {
      size_t base = (s * n_heads + h) * head_dim;
      for (size_t i = 0; i < half; ++i) {
        float c = cos_table[pos * half + i];
        float sn = sin_table[pos * half + i];
        float x0 = in[base + 2 * i];
        float x1 = in[base + 2 * i + 1];
        out[base + 2 * i] = x0 * c - x1 * sn;
        out[base + 2 * i + 1] = x0 * sn + x1 * c;
      }
    }
  }
}

// device.rs:727-736 with cpu.rs:84-96: swiglu_fused_buf runs through `elementwise`, which
// evaluates the traced expression g * (1/(1+exp(-g))) * u in f64 and narrows the result to f32.
ORC_API void orc_swiglu_f32(const float* gate, const float* up, float* out, size_t numel) {
  for (size_t i = 0; i < numel; ++i) {
    double g = (double)gate[i];
    double u = (double)up[i];
    double sig = 1.0 / (1.0 + std::exp(-g));
    out[i] = (float)(g * sig * u);
  }
}

// ---------------------------------------------------------------------------------------------
// f64 model pieces (crates/tang-train/examples/smollm.rs — the reference's only decode loop)
// ---------------------------------------------------------------------------------------------

// smollm.rs:39-47  rms_norm: ss = sum(x^2)/n, scale = 1/sqrt(ss+eps), out = x*scale*w.
ORC_API void orc_rms_norm_f64(const double* x, const double* w, double* out, size_t n, double eps) {
  double ss = 0.0;
  for (size_t i = 0; i < n; ++i) ss += x[i] * x[i];
  ss /= (double)n;
  double scale = 1.0 / std::sqrt(ss + eps);
  for (size_t i = 0; i < n; ++i) out[i] = x[i] * scale * w[i];
}

// crates/tang-train/src/layers.rs:2134-2200  RotaryEmbedding::with_base + apply, for one
// position: theta_i = pos / base^(2i/dim); even' = e*cos - o*sin, odd' = e*sin + o*cos.
// smollm.rs:311-343 applies it head by head over [heads*head_dim].
ORC_API void orc_rope_heads_f64(const double* x, double* out, size_t n_heads, size_t head_dim, size_t pos, double base) {
  for (size_t h = 0; h < n_heads; ++h)
    for (size_t i = 0; i < head_dim / 2; ++i) {
      double theta = (double)pos / std::pow(base, 2.0 * (double)i / (double)head_dim);
      double c = std::cos(theta), s = std::sin(theta);
      double e = x[h * head_dim + 2 * i], o = x[h * head_dim + 2 * i + 1];
      out[h * head_dim + 2 * i] = e * c - o * s;
      out[h * head_dim + 2 * i + 1] = e * s + o * c;
    }
}

// smollm.rs:101-154  decode attention for one query row (seq_len == 1, so no causal mask):
// scores = q·k * (1/sqrt(head_dim)); softmax by max-subtract, exp, divide by the sum; output =
// sum_k w_k * v_k accumulated in position order.  Caches are [total_seq, n_kv_heads*head_dim].
ORC_API void orc_attention_decode_f64(const double* q, const double* k_cache, const double* v_cache, double* out,
                                      size_t total_seq, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                      int threads) {
  size_t kv_dim = n_kv_heads * head_dim;
  size_t heads_per_kv = n_heads / n_kv_heads;
  double scale = 1.0 / std::sqrt((double)head_dim);
  int nt = clamp_threads(threads);
  (void)nt;
#pragma omp parallel for num_threads(nt) schedule(static)
  for (long long hh = 0; hh < (long long)n_heads; ++hh) {
    size_t h = (size_t)hh;
    size_t kv_h = h / heads_per_kv;
    std::vector<double> scores(total_seq);
    for (size_t ki = 0; ki < total_seq; ++ki) {
      size_t k_off = ki * kv_dim + kv_h * head_dim;
      double dot = 0.0;
      for (size_t d = 0; d < head_dim; ++d) dot += q[h * head_dim + d] * k_cache[k_off + d];
      scores[ki] = dot * scale;
    }
    double mx = -std::numeric_limits<double>::infinity();
    for (size_t ki = 0; ki < total_seq; ++ki) mx = std::fmax(mx, scores[ki]);
    double sum = 0.0;
    for (size_t ki = 0; ki < total_seq; ++ki) {
      scores[ki] = std::exp(scores[ki] - mx);
      sum += scores[ki];
    }
    for (size_t ki = 0; ki < total_seq; ++ki) scores[ki] /= sum;
    double* o = out + h * head_dim;
    for (size_t d = 0; d < head_dim; ++d) o[d] = 0.0;
    for (size_t ki = 0; ki < total_seq; ++ki) {
      size_t v_off = ki * kv_dim + kv_h * head_dim;
      double w = scores[ki];
      for (size_t d = 0; d < head_dim; ++d) o[d] += w * v_cache[v_off + d];
    }
  }
}

// smollm.rs:181-191  SwiGLU in f64: v * (1/(1+exp(-v))) * up.
ORC_API void orc_swiglu_f64(const double* gate, const double* up, double* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = gate[i] * (1.0 / (1.0 + std::exp(-gate[i]))) * up[i];
}

// ---------------------------------------------------------------------------------------------
// Selection rules (crates/tang-infer/src/sampling.rs)
// ---------------------------------------------------------------------------------------------

// sampling.rs:183-194  argmax: strict '>' scan, so the FIRST maximum wins.
ORC_API size_t orc_argmax_f64(const double* v, size_t n) {
  size_t best = 0;
  double best_val = -std::numeric_limits<double>::infinity();
  for (size_t i = 0; i < n; ++i)
    if (v[i] > best_val) {
      best_val = v[i];
      best = i;
    }
  return best;
}

// sampling.rs:176-181  kth_largest: sort descending, take element k-1.
ORC_API double orc_kth_largest_f64(const double* v, size_t n, size_t k) {
  std::vector<double> s(v, v + n);
  std::stable_sort(s.begin(), s.end(), [](double a, double b) { return a > b; });
  return s[std::min(k, n) - 1];
}

// sampling.rs:119-133  the sampler's softmax numerators and top-k filter: exp(l - max), then
// zero everything below the k-th largest value (entries equal to the threshold all survive).
ORC_API void orc_topk_filter_f64(const double* logits, size_t n, size_t k, double* probs_out) {
  double mx = -std::numeric_limits<double>::infinity();
  for (size_t i = 0; i < n; ++i) mx = std::fmax(mx, logits[i]);
  for (size_t i = 0; i < n; ++i) probs_out[i] = std::exp(logits[i] - mx);
  if (k > 0 && k < n) {
    double thr = orc_kth_largest_f64(probs_out, n, k);
    for (size_t i = 0; i < n; ++i)
      if (probs_out[i] < thr) probs_out[i] = 0.0;
  }
}

// Exactly-k selection used for expert routing.  The reference has no router; this fixes the
// rule its top-k precedents leave open: larger value first, LOWER INDEX first among equal
// values, exactly k winners, returned in that order.
ORC_API void orc_topk_indices_f64(const double* v, size_t n, size_t k, int32_t* idx_out) {
  std::vector<int32_t> idx(n);
  for (size_t i = 0; i < n; ++i) idx[i] = (int32_t)i;
  std::stable_sort(idx.begin(), idx.end(), [&](int32_t a, int32_t b) { return v[a] > v[b]; });
  for (size_t i = 0; i < k && i < n; ++i) idx_out[i] = idx[i];
}

// sampling.rs:72-79  rand_f64: 64-bit LCG (Knuth's MMIX constants), top 53 bits as a fraction in [0, 1).
ORC_API double orc_lcg_next_f64(uint64_t* state) {
  *state = *state * 6364136223846793005ULL + 1442695040888963407ULL;
  return (double)(*state >> 11) / (double)(1ULL << 53);
}

// sampling.rs:196-218  top_p_filter: indices sorted by probability, descending (Rust's sort_by is stable, so
// equal probabilities keep ascending index order); the cumulative sum runs in that order and everything after
// the first rank at which it reaches p is zeroed.
static void top_p_filter(std::vector<double>& probs, double p) {
  std::vector<size_t> idx(probs.size());
  for (size_t i = 0; i < idx.size(); ++i) idx[i] = i;
  std::stable_sort(idx.begin(), idx.end(), [&](size_t a, size_t b) { return probs[a] > probs[b]; });
  double cumsum = 0.0;
  size_t cutoff = probs.size();
  for (size_t rank = 0; rank < idx.size(); ++rank) {
    cumsum += probs[idx[rank]];
    if (cumsum >= p) {
      cutoff = rank + 1;
      break;
    }
  }
  for (size_t rank = cutoff; rank < idx.size(); ++rank) probs[idx[rank]] = 0.0;
}

// sampling.rs:86-158  Sampler::sample, step for step: f64 copy of the logits; repetition penalty once per
// occurrence in past_tokens (divide positive logits, multiply the others); temperature 0 -> argmax; scale by
// 1/temperature; exp(l - max); top-k threshold (ties at the threshold survive); normalise (sum <= 0 -> argmax);
// top-p filter and re-normalise; categorical draw with one LCG step (sampling.rs:161-174: first index whose
// running sum exceeds r, else the last index).
struct OrcSamplerConfig {
  double temperature;
  uint64_t top_k;
  double top_p;
  double repetition_penalty;
};

ORC_API int64_t orc_sampler_sample(const double* logits, size_t n, const int64_t* past, size_t n_past,
                                   const OrcSamplerConfig* cfg, uint64_t* rng_state) {
  std::vector<double> probs(logits, logits + n);
  if (cfg->repetition_penalty != 1.0) {
    for (size_t j = 0; j < n_past; ++j) {
      if (past[j] >= 0 && (size_t)past[j] < n) {
        double& v = probs[(size_t)past[j]];
        if (v > 0.0) v /= cfg->repetition_penalty;
        else v *= cfg->repetition_penalty;
      }
    }
  }
  if (cfg->temperature == 0.0) return (int64_t)orc_argmax_f64(probs.data(), n);
  if (cfg->temperature != 1.0) {
    const double inv_t = 1.0 / cfg->temperature;
    for (double& v : probs) v *= inv_t;
  }
  double mx = -std::numeric_limits<double>::infinity();
  for (double v : probs) mx = std::fmax(mx, v);
  for (double& v : probs) v = std::exp(v - mx);
  if (cfg->top_k > 0 && cfg->top_k < n) {
    const double thr = orc_kth_largest_f64(probs.data(), n, (size_t)cfg->top_k);
    for (double& v : probs)
      if (v < thr) v = 0.0;
  }
  double sum = 0.0;
  for (double v : probs) sum += v;
  if (sum <= 0.0) return (int64_t)orc_argmax_f64(probs.data(), n);
  for (double& v : probs) v /= sum;
  if (cfg->top_p < 1.0) {
    top_p_filter(probs, cfg->top_p);
    double s2 = 0.0;
    for (double v : probs) s2 += v;
    if (s2 > 0.0)
      for (double& v : probs) v /= s2;
  }
  const double r = orc_lcg_next_f64(rng_state);
  double cumsum = 0.0;
  for (size_t i = 0; i < n; ++i) {
    cumsum += probs[i];
    if (r < cumsum) return (int64_t)i;
  }
  return (int64_t)n - 1;
}

ORC_API int orc_max_threads(void) { return clamp_threads(0); }
