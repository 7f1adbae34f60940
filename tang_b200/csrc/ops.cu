// Small bandwidth-trivial operators of the decode step (include/tangq.h): RMSNorm (+residual),
// interleaved RoPE, SwiGLU, embedding gather, and the fused q/k/v post-processing that rotates
// q and k and appends k, v to the bf16 KV cache.
#include <cuda_bf16.h>

#include <cmath>
#include <vector>

#include "common.cuh"
#include "internal.h"

namespace tq {

__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
  return dtype == TQ_F32 ? reinterpret_cast<const float*>(p)[i]
                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, int dtype, size_t i, float v) {
  if (dtype == TQ_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Block-wide sum; `red` holds one float per warp.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// rms_norm / rms_norm_residual (crates/tang-compute/src/cpu.rs:126-149, device.rs:546-575):
//   v = x (+ residual);  out = v * (1/sqrt(mean(v^2) + eps)) * w;  sum_out = v (optional).
// One CTA per row; the row is read once into registers (dim <= 256*32).
constexpr int kNormThreads = 256;
constexpr int kNormMaxPerThread = 32;

__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const void* x, int x_dt, const float* residual,
                                                                const void* w, int w_dt, int dim, float eps, void* out,
                                                                int out_dt, float* sum_out) {
  __shared__ float red[kNormThreads / 32];
  const size_t row = blockIdx.x;
  float v[kNormMaxPerThread];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxPerThread; ++i) {
    const int d = threadIdx.x + i * kNormThreads;
    v[i] = 0.f;
    if (d < dim) {
      float t = load_as_float(x, x_dt, row * dim + d);
      if (residual) t += residual[row * dim + d];
      v[i] = t;
      sq += t * t;
    }
  }
  const float total = block_sum(sq, red);
  const float inv = 1.0f / sqrtf(total / (float)dim + eps);
#pragma unroll
  for (int i = 0; i < kNormMaxPerThread; ++i) {
    const int d = threadIdx.x + i * kNormThreads;
    if (d < dim) {
      store_from_float(out, out_dt, row * dim + d, v[i] * inv * load_as_float(w, w_dt, d));
      if (sum_out) sum_out[row * dim + d] = v[i];
    }
  }
}

// rope_forward (crates/tang-compute/src/device.rs:582-610): x [rows, n_heads, head_dim]; pair
// (2i, 2i+1) of every head rotated by table row `pos`; pos = positions[row] or start_pos + row.
__global__ void rope_kernel(const void* x, int x_dt, void* out, int out_dt, const float* cos_t, const float* sin_t,
                            const int* positions, int start_pos, size_t rows, int n_heads, int head_dim) {
  const int half = head_dim / 2;
  const size_t total = rows * n_heads * half;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int i = (int)(idx % half);
  const size_t rh = idx / half;  // row * n_heads + head
  const size_t row = rh / n_heads;
  const int pos = positions ? positions[row] : start_pos + (int)row;
  const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
  const size_t base = rh * head_dim + 2 * i;
  const float x0 = load_as_float(x, x_dt, base), x1 = load_as_float(x, x_dt, base + 1);
  store_from_float(out, out_dt, base, x0 * c - x1 * s);
  store_from_float(out, out_dt, base + 1, x0 * s + x1 * c);
}

// swiglu_fused_buf (device.rs:727-736): out = g * (1/(1+exp(-g))) * u.  gate and up may be the two
// halves of one fused projection: element (row, i) of gate sits at gate[row*ld + i].
__global__ void swiglu_kernel(const void* gate, const void* up, int in_dt, size_t ld, size_t rows, size_t n, void* out,
                              int out_dt) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * n) return;
  const size_t row = idx / n, i = idx % n;
  const float g = load_as_float(gate, in_dt, row * ld + i), u = load_as_float(up, in_dt, row * ld + i);
  const float sig = 1.0f / (1.0f + expf(-g));
  store_from_float(out, out_dt, idx, g * sig * u);
}

// embedding (cpu.rs:151-167): out[i, :] = weight[ids[i], :].
__global__ void embedding_kernel(const void* weight, int w_dt, const int* ids, size_t n_ids, size_t dim, size_t vocab,
                                 void* out, int out_dt) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_ids * dim) return;
  const size_t r = idx / dim, d = idx % dim;
  const int id = ids[r];
  const float v = (id >= 0 && (size_t)id < vocab) ? load_as_float(weight, w_dt, (size_t)id * dim + d) : 0.f;
  store_from_float(out, out_dt, idx, v);
}

// Fused epilogue of the q/k/v projection for one decode token per sequence
// (crates/tang-train/examples/smollm.rs:84-95: RoPE on q and k, then cache.append(k_roped, v)):
//   qkv [B, (n_heads + 2*n_kv) * hd] f32  ->  q_out [B, n_heads*hd] bf16 (rotated),
//   k_cache[b, pos_b, :] = bf16(rot(k)),  v_cache[b, pos_b, :] = bf16(v).
// Cache layout per sequence is [max_seq, n_kv*hd] (crates/tang-infer/src/kv_cache.rs:12-24).
__global__ void qkv_post_kernel(const float* qkv, const float* cos_t, const float* sin_t, const int* positions, int B,
                                int n_heads, int n_kv, int hd, int max_seq, __nv_bfloat16* q_out,
                                __nv_bfloat16* k_cache, __nv_bfloat16* v_cache, size_t seq_stride) {
  const int half = hd / 2;
  const int pairs_per_row = (n_heads + 2 * n_kv) * half;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)B * pairs_per_row) return;
  const int b = (int)(idx / pairs_per_row);
  const int pr = (int)(idx % pairs_per_row);
  const int head = pr / half, i = pr % half;
  const int pos = positions[b];
  const size_t src = (size_t)b * (n_heads + 2 * n_kv) * hd + (size_t)head * hd + 2 * i;
  const float x0 = qkv[src], x1 = qkv[src + 1];
  if (head < n_heads + n_kv) {
    const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
    const float r0 = x0 * c - x1 * s, r1 = x0 * s + x1 * c;
    const __nv_bfloat162 pk = __floats2bfloat162_rn(r0, r1);
    if (head < n_heads) {
      *reinterpret_cast<__nv_bfloat162*>(q_out + (size_t)b * n_heads * hd + (size_t)head * hd + 2 * i) = pk;
    } else if (pos < max_seq) {
      const int kh = head - n_heads;
      *reinterpret_cast<__nv_bfloat162*>(k_cache + (size_t)b * seq_stride + (size_t)pos * n_kv * hd + (size_t)kh * hd + 2 * i) = pk;
    }
  } else if (pos < max_seq) {
    const int vh = head - n_heads - n_kv;
    *reinterpret_cast<__nv_bfloat162*>(v_cache + (size_t)b * seq_stride + (size_t)pos * n_kv * hd + (size_t)vh * hd + 2 * i) =
        __floats2bfloat162_rn(x0, x1);
  }
}

int launch_qkv_post(tq_ctx* ctx, const float* qkv, const float* cos_t, const float* sin_t, const int* positions, int B,
                    int n_heads, int n_kv, int hd, int max_seq, void* q_out, void* k_cache, void* v_cache,
                    size_t seq_stride) {
  const size_t n = (size_t)B * (n_heads + 2 * n_kv) * (hd / 2);
  qkv_post_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
      qkv, cos_t, sin_t, positions, B, n_heads, n_kv, hd, max_seq, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), seq_stride);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

}  // namespace tq

using namespace tq;

static bool io_dtype(int d) { return d == TQ_F32 || d == TQ_BF16; }

extern "C" {

int tq_rms_norm(tq_ctx* ctx, const void* x_dev, int x_dtype, const float* residual_dev, const void* weight_dev,
                int w_dtype, size_t n_groups, size_t dim, float eps, void* out_dev, int out_dtype, float* sum_out_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, io_dtype(x_dtype) && io_dtype(w_dtype) && io_dtype(out_dtype), "tq_rms_norm: dtypes must be f32 or bf16");
  TQ_REQUIRE(ctx, dim > 0 && dim <= (size_t)kNormThreads * kNormMaxPerThread, "tq_rms_norm: dim must be in 1..%d",
             kNormThreads * kNormMaxPerThread);
  if (n_groups == 0) return TQ_OK;
  TQ_REQUIRE(ctx, x_dev && weight_dev && out_dev, "tq_rms_norm: null pointer");
  rms_norm_kernel<<<(unsigned)n_groups, kNormThreads, 0, ctx->stream>>>(x_dev, x_dtype, residual_dev, weight_dev, w_dtype,
                                                                       (int)dim, eps, out_dev, out_dtype, sum_out_dev);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

int tq_rope_tables(tq_ctx* ctx, size_t head_dim, size_t max_seq_len, double base, float* cos_dev, float* sin_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, head_dim >= 2 && head_dim % 2 == 0 && max_seq_len > 0 && base > 0, "tq_rope_tables: bad shape");
  TQ_REQUIRE(ctx, cos_dev && sin_dev, "tq_rope_tables: null pointer");
  // InterleavedRoPE::new (crates/tang-compute/src/modules.rs:495-510): f64 on the host, stored f32.
  const size_t half = head_dim / 2;
  std::vector<float> c(max_seq_len * half), s(max_seq_len * half);
  std::vector<double> freq(half);
  for (size_t i = 0; i < half; ++i) freq[i] = 1.0 / std::pow(base, (double)i / (double)half);
  for (size_t pos = 0; pos < max_seq_len; ++pos)
    for (size_t i = 0; i < half; ++i) {
      const double angle = (double)pos * freq[i];
      c[pos * half + i] = (float)std::cos(angle);
      s[pos * half + i] = (float)std::sin(angle);
    }
  TQ_CUDA(ctx, cudaMemcpyAsync(cos_dev, c.data(), c.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  TQ_CUDA(ctx, cudaMemcpyAsync(sin_dev, s.data(), s.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return TQ_OK;
}

int tq_rope_forward(tq_ctx* ctx, const void* x_dev, int x_dtype, const float* cos_dev, const float* sin_dev,
                    const int* positions_dev, size_t seq_len, size_t n_heads, size_t head_dim, size_t start_pos,
                    void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, io_dtype(x_dtype) && io_dtype(out_dtype), "tq_rope_forward: dtypes must be f32 or bf16");
  TQ_REQUIRE(ctx, head_dim >= 2 && head_dim % 2 == 0, "tq_rope_forward: head_dim must be even");
  const size_t n = seq_len * n_heads * (head_dim / 2);
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(ctx, x_dev && out_dev && cos_dev && sin_dev, "tq_rope_forward: null pointer");
  rope_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x_dev, x_dtype, out_dev, out_dtype, cos_dev, sin_dev,
                                                                   positions_dev, (int)start_pos, seq_len, (int)n_heads,
                                                                   (int)head_dim);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

int tq_swiglu(tq_ctx* ctx, const void* gate_dev, const void* up_dev, int in_dtype, size_t ld, size_t rows, size_t n,
              void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, io_dtype(in_dtype) && io_dtype(out_dtype), "tq_swiglu: dtypes must be f32 or bf16");
  if (rows * n == 0) return TQ_OK;
  TQ_REQUIRE(ctx, gate_dev && up_dev && out_dev, "tq_swiglu: null pointer");
  if (ld == 0) ld = n;
  swiglu_kernel<<<(unsigned)((rows * n + 255) / 256), 256, 0, ctx->stream>>>(gate_dev, up_dev, in_dtype, ld, rows, n, out_dev,
                                                                            out_dtype);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

int tq_embedding(tq_ctx* ctx, const void* weight_dev, int w_dtype, const int* ids_dev, size_t seq_len, size_t dim,
                 size_t vocab, void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, io_dtype(w_dtype) && io_dtype(out_dtype), "tq_embedding: dtypes must be f32 or bf16");
  if (seq_len * dim == 0) return TQ_OK;
  TQ_REQUIRE(ctx, weight_dev && ids_dev && out_dev, "tq_embedding: null pointer");
  embedding_kernel<<<(unsigned)((seq_len * dim + 255) / 256), 256, 0, ctx->stream>>>(weight_dev, w_dtype, ids_dev, seq_len,
                                                                                    dim, vocab, out_dev, out_dtype);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

}  // extern "C"
