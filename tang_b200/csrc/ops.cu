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
// One CTA per row.  The row is read once, four elements per load, ALL loads issued before any of
// them is used (the row lives in registers), so the kernel costs one memory round trip per phase.
constexpr int kNormThreads = 256;
constexpr int kNormVecs = 8;  // float4 chunks per thread: dim <= 256 * 8 * 4 = 8192

template <typename T>
__device__ __forceinline__ float4 load4(const T* p, size_t i);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p, size_t i) {
  return *reinterpret_cast<const float4*>(p + i);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  const uint2 u = *reinterpret_cast<const uint2*>(p + i);
  return make_float4(bf16_bits_to_float(u.x & 0xFFFFu), bf16_bits_to_float(u.x >> 16), bf16_bits_to_float(u.y & 0xFFFFu),
                     bf16_bits_to_float(u.y >> 16));
}
__device__ __forceinline__ void store4(float* p, size_t i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, size_t i, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p + i) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

// dim % 4 == 0 and 16-byte aligned rows.
template <typename XT, typename WT, typename OT>
__global__ void __launch_bounds__(kNormThreads) rms_norm_vec_kernel(const XT* x, const float* residual, const WT* w, int dim,
                                                                    float eps, OT* out, float* sum_out) {
  __shared__ float red[kNormThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t base = (size_t)blockIdx.x * dim;
  const bool has_res = residual != nullptr;
  float4 v[kNormVecs], r[kNormVecs], g[kNormVecs];
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    const int d = 4 * (threadIdx.x + i * kNormThreads);
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    r[i] = v[i];
    g[i] = v[i];
    if (d < dim) {
      v[i] = load4<XT>(x, base + d);
      if (has_res) r[i] = load4<float>(residual, base + d);
      g[i] = load4<WT>(w, d);
    }
  }
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    v[i].x += r[i].x;
    v[i].y += r[i].y;
    v[i].z += r[i].z;
    v[i].w += r[i].w;
    sq += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  const float total = block_sum(sq, red);
  const float inv = 1.0f / sqrtf(total / (float)dim + eps);
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    const int d = 4 * (threadIdx.x + i * kNormThreads);
    if (d < dim) {
      store4(out, base + d, make_float4(v[i].x * inv * g[i].x, v[i].y * inv * g[i].y, v[i].z * inv * g[i].z, v[i].w * inv * g[i].w));
      if (sum_out) store4(sum_out, base + d, v[i]);
    }
  }
}

// Any dim <= 8192, any alignment: one element per step (the rarely used fallback).
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const void* x, int x_dt, const float* residual,
                                                                const void* w, int w_dt, int dim, float eps, void* out,
                                                                int out_dt, float* sum_out) {
  __shared__ float red[kNormThreads / 32];
  __shared__ float row_s[8192];
  pdl_wait();
  pdl_launch_dependents();
  const size_t base = (size_t)blockIdx.x * dim;
  float sq = 0.f;
  for (int d = threadIdx.x; d < dim; d += kNormThreads) {
    float t = load_as_float(x, x_dt, base + d);
    if (residual) t += residual[base + d];
    row_s[d] = t;
    sq += t * t;
  }
  const float total = block_sum(sq, red);
  const float inv = 1.0f / sqrtf(total / (float)dim + eps);
  for (int d = threadIdx.x; d < dim; d += kNormThreads) {
    store_from_float(out, out_dt, base + d, row_s[d] * inv * load_as_float(w, w_dt, d));
    if (sum_out) sum_out[base + d] = row_s[d];
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
  pdl_wait();
  pdl_launch_dependents();
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
  pdl_wait();
  pdl_launch_dependents();
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
// With q_len > 1 (prefill) the rows are [sequence][i] and row i of sequence b sits at position positions[b] + i.
// `rope_positions` (optional) gives the position each sequence's rotation uses when that is not its cache row any
// more (after KVCache::trim_to, crates/tang-infer/src/kv_cache.rs:138-149, rows move to the front of the cache
// while the caller's position count runs on).
__global__ void qkv_post_kernel(const float* qkv, const float* cos_t, const float* sin_t, const int* positions,
                                const int* rope_positions, int B,
                                int n_heads, int n_kv, int hd, int max_seq, __nv_bfloat16* q_out,
                                __nv_bfloat16* k_cache, __nv_bfloat16* v_cache, size_t seq_stride, int q_len, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int half = hd / 2;
  const int pairs_per_row = (n_heads + 2 * n_kv) * half;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)B * pairs_per_row) return;
  const int row = (int)(idx / pairs_per_row);   // B counts rows (sequences x q_len)
  const int pr = (int)(idx % pairs_per_row);
  const int head = pr / half, i = pr % half;
  const int b = row / q_len;
  const int pos = positions[b] + row % q_len;
  // The position comes from device memory (a generation loop advances it inside a replayed graph): one outside
  // the cache / the tables is not followed.  The row's outputs stay unwritten and the status word says why.
  const int rpos = rope_positions ? rope_positions[b] + row % q_len : pos;
  if (pos < 0 || pos >= max_seq || rpos < 0 || rpos >= max_seq) {
    if (pr == 0) atomicCAS(err, 0, (int)DERR_POSITION);
    return;
  }
  const size_t src = (size_t)row * (n_heads + 2 * n_kv) * hd + (size_t)head * hd + 2 * i;
  const float x0 = qkv[src], x1 = qkv[src + 1];
  if (head < n_heads + n_kv) {
    const float c = cos_t[(size_t)rpos * half + i], s = sin_t[(size_t)rpos * half + i];
    const float r0 = x0 * c - x1 * s, r1 = x0 * s + x1 * c;
    const __nv_bfloat162 pk = __floats2bfloat162_rn(r0, r1);
    if (head < n_heads) {
      *reinterpret_cast<__nv_bfloat162*>(q_out + (size_t)row * n_heads * hd + (size_t)head * hd + 2 * i) = pk;
    } else {
      const int kh = head - n_heads;
      *reinterpret_cast<__nv_bfloat162*>(k_cache + (size_t)b * seq_stride + (size_t)pos * n_kv * hd + (size_t)kh * hd + 2 * i) = pk;
    }
  } else {
    const int vh = head - n_heads - n_kv;
    *reinterpret_cast<__nv_bfloat162*>(v_cache + (size_t)b * seq_stride + (size_t)pos * n_kv * hd + (size_t)vh * hd + 2 * i) =
        __floats2bfloat162_rn(x0, x1);
  }
}

int launch_qkv_post(tq_ctx* ctx, const float* qkv, const float* cos_t, const float* sin_t, const int* positions,
                    const int* rope_positions, int B, int n_heads, int n_kv, int hd, int max_seq, void* q_out, void* k_cache,
                    void* v_cache, size_t seq_stride, int q_len) {
  const size_t n = (size_t)B * (n_heads + 2 * n_kv) * (hd / 2);
  TQ_CUDA(ctx, launch_k(ctx, qkv_post_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, qkv, cos_t, sin_t, positions, rope_positions, B,
                        n_heads, n_kv, hd, max_seq, static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                        static_cast<__nv_bfloat16*>(v_cache), seq_stride, q_len, ctx->dev_err));
  return TQ_OK;
}

// Index of the first maximum of each row (strict '>' scan from index 0: NaN is never chosen, an all-NaN or
// all -inf row gives 0), crates/tang-infer/src/sampling.rs:183-194.  x is [slices][rows][cols]; the index is
// slice * cols + column.  One CTA per row; each thread scans ascending indices, then (value, index) pairs meet
// with "larger value, else smaller index".
__global__ void argmax_rows_kernel(const float* x, int slices, int rows, int cols, int* idx_out) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int total = slices * cols;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int sl = i / cols, c = i - sl * cols;
    const float v = x[((size_t)sl * rows + r) * cols + c];
    if (v > best) {
      best = v;
      best_i = i;
    }
  }
  auto meet = [](float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) meet(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
  __shared__ float sv[32];
  __shared__ int si[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    best_i = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) meet(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    if (lane == 0) idx_out[r] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

// Between two decode steps of a generation loop: record the chosen tokens, make them the next input, advance the
// positions.  The step counter lives on the device so that the same captured graph can be replayed.
__global__ void generate_advance_kernel(const int* chosen, int rows, int* tokens_io, int* positions_io, int* out_tokens,
                                        int out_ld, int* step_io, int* lens_io) {
  pdl_wait();
  pdl_launch_dependents();
  const int step = *step_io;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) {
    if (step < out_ld) out_tokens[(size_t)i * out_ld + step] = chosen[i];
    tokens_io[i] = chosen[i];
    positions_io[i] += 1;
    if (lens_io) lens_io[i] += 1;
  }
  __syncthreads();                       // a single block (rows <= 1024): every thread has read `step`
  if (threadIdx.x == 0) *step_io = step + 1;
}

}  // namespace tq

using namespace tq;

static bool io_dtype(int d) { return d == TQ_F32 || d == TQ_BF16; }

extern "C" {

int tq_rms_norm(tq_ctx* ctx, const void* x_dev, int x_dtype, const float* residual_dev, const void* weight_dev,
                int w_dtype, size_t n_groups, size_t dim, float eps, void* out_dev, int out_dtype, float* sum_out_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, io_dtype(x_dtype) && io_dtype(w_dtype) && io_dtype(out_dtype), "tq_rms_norm: dtypes must be f32 or bf16");
  TQ_REQUIRE(ctx, dim > 0 && dim <= 8192, "tq_rms_norm: dim must be in 1..8192");
  if (n_groups == 0) return TQ_OK;
  TQ_REQUIRE(ctx, x_dev && weight_dev && out_dev, "tq_rms_norm: null pointer");
  const dim3 grid((unsigned)n_groups), block(kNormThreads);
  const bool vec = dim % 4 == 0 && (((uintptr_t)x_dev | (uintptr_t)weight_dev | (uintptr_t)out_dev | (uintptr_t)residual_dev |
                                     (uintptr_t)sum_out_dev) & 15) == 0;
  using bf = __nv_bfloat16;
#define TQ_NORM(XT, WT, OT)                                                                                           \
  TQ_CUDA(ctx, launch_k(ctx, rms_norm_vec_kernel<XT, WT, OT>, grid, block, 0, static_cast<const XT*>(x_dev), residual_dev, \
                        static_cast<const WT*>(weight_dev), (int)dim, eps, static_cast<OT*>(out_dev), sum_out_dev))
  const int key = (x_dtype == TQ_BF16) * 4 + (w_dtype == TQ_BF16) * 2 + (out_dtype == TQ_BF16);
  if (!vec) {
    TQ_CUDA(ctx, launch_k(ctx, rms_norm_kernel, grid, block, 0, x_dev, x_dtype, residual_dev, weight_dev, w_dtype, (int)dim, eps,
                          out_dev, out_dtype, sum_out_dev));
  } else {
    switch (key) {
      case 0: TQ_NORM(float, float, float); break;
      case 1: TQ_NORM(float, float, bf); break;
      case 2: TQ_NORM(float, bf, float); break;
      case 3: TQ_NORM(float, bf, bf); break;
      case 4: TQ_NORM(bf, float, float); break;
      case 5: TQ_NORM(bf, float, bf); break;
      case 6: TQ_NORM(bf, bf, float); break;
      default: TQ_NORM(bf, bf, bf); break;
    }
  }
#undef TQ_NORM
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
  TQ_CUDA(ctx, launch_k(ctx, swiglu_kernel, dim3((unsigned)((rows * n + 255) / 256)), dim3(256), 0, gate_dev, up_dev, in_dtype,
                        ld, rows, n, out_dev, out_dtype));
  return TQ_OK;
}

int tq_embedding(tq_ctx* ctx, const void* weight_dev, int w_dtype, const int* ids_dev, size_t seq_len, size_t dim,
                 size_t vocab, void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, io_dtype(w_dtype) && io_dtype(out_dtype), "tq_embedding: dtypes must be f32 or bf16");
  if (seq_len * dim == 0) return TQ_OK;
  TQ_REQUIRE(ctx, weight_dev && ids_dev && out_dev, "tq_embedding: null pointer");
  TQ_CUDA(ctx, launch_k(ctx, embedding_kernel, dim3((unsigned)((seq_len * dim + 255) / 256)), dim3(256), 0, weight_dev, w_dtype,
                        ids_dev, seq_len, dim, vocab, out_dev, out_dtype));
  return TQ_OK;
}

int tq_argmax_rows(tq_ctx* ctx, const float* x_dev, size_t slices, size_t rows, size_t cols, int* idx_out_dev) {
  if (int st = bind(ctx)) return st;
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(ctx, x_dev && idx_out_dev && slices > 0 && cols > 0, "tq_argmax_rows: null pointer or empty row");
  TQ_REQUIRE(ctx, slices * cols < (1ull << 31), "tq_argmax_rows: row too long");
  TQ_CUDA(ctx, launch_k(ctx, argmax_rows_kernel, dim3((unsigned)rows), dim3(1024), 0, x_dev, (int)slices, (int)rows, (int)cols,
                        idx_out_dev));
  return TQ_OK;
}

int tq_generate_advance(tq_ctx* ctx, const int* chosen_dev, size_t rows, int* tokens_io_dev, int* positions_io_dev,
                        int* out_tokens_dev, size_t out_ld, int* step_io_dev, int* lens_io_dev) {
  if (int st = bind(ctx)) return st;
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(ctx, chosen_dev && tokens_io_dev && positions_io_dev && out_tokens_dev && step_io_dev, "tq_generate_advance: null pointer");
  TQ_REQUIRE(ctx, rows <= 1024, "tq_generate_advance: at most 1024 sequences");
  TQ_CUDA(ctx, launch_k(ctx, generate_advance_kernel, dim3(1), dim3(1024), 0, chosen_dev, (int)rows, tokens_io_dev,
                        positions_io_dev, out_tokens_dev, (int)out_ld, step_io_dev, lens_io_dev));
  return TQ_OK;
}

}  // extern "C"
