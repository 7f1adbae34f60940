// Quantised weights and the quantised linear layer of the C ABI (include/tangq.h).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "internal.h"
#include "qgemm_mma.cuh"

namespace tq {

static inline bool is_q4(int kind) { return kind == TQ_Q4_F32 || kind == TQ_Q4_F16; }
static inline size_t scale_elem(int kind) { return kind == TQ_Q4_F16 ? 2 : 4; }

// ---------------------------------------------------------------------------------------------
// dequantize_q4 / dequantize_q8 (crates/tang-infer/src/quantize.rs:73-81,121-132) through the same
// register dequantisers the GEMM uses, so a bit-exact check of this kernel's integers is a check
// of the GEMM's unpack.  One thread per 8 consecutive k.
// ---------------------------------------------------------------------------------------------
__global__ void dequantize_kernel(const uint8_t* payload, const uint8_t* scales, size_t ldw, size_t lds, int kind,
                                  size_t rows, size_t cols, size_t kpad, float* out, int8_t* ints) {
  const size_t per_row = kpad / 8;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const size_t row = idx / per_row, oct = idx % per_row;
  const size_t k0 = oct * 8;
  uint32_t v[4];
  if (kind == TQ_Q4_F32 || kind == TQ_Q4_F16) {
    dequant_q4_word(*reinterpret_cast<const uint32_t*>(payload + row * ldw + k0 / 2), v);
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(payload + row * ldw + k0);
    dequant_i8_words(u.x, u.y, v);
  }
  float scale;
  if (kind == TQ_I8_ROW) scale = reinterpret_cast<const float*>(scales)[row];
  else if (kind == TQ_Q4_F16) scale = __half2float(*reinterpret_cast<const __half*>(scales + row * lds + 2 * (k0 / 32)));
  else scale = *reinterpret_cast<const float*>(scales + row * lds + 4 * (k0 / 32));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = bf16_bits_to_float(v[i] & 0xFFFFu), hi = bf16_bits_to_float(v[i] >> 16);  // k0+i, k0+i+4
    if (k0 + i < cols) {
      if (out) out[row * cols + k0 + i] = lo * scale;
      if (ints) ints[row * cols + k0 + i] = (int8_t)(int)lo;
    }
    if (k0 + i + 4 < cols) {
      if (out) out[row * cols + k0 + i + 4] = hi * scale;
      if (ints) ints[row * cols + k0 + i + 4] = (int8_t)(int)hi;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Activation staging: produces the bf16 [mx][kpad] operand of the GEMM kernel (zero beyond the
// true K).  bf16 input is copied; f32 input is split exactly into three bf16 terms
// hi = bf16(x), mid = bf16(x - hi), lo = x - hi - mid, stored as rows 3m, 3m+1, 3m+2.
// ---------------------------------------------------------------------------------------------
__global__ void prep_x_kernel(const void* x, int x_dtype, size_t ldx, size_t m, size_t k, size_t kpad,
                              __nv_bfloat16* out) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= m * kpad) return;
  const size_t row = idx / kpad, col = idx % kpad;
  if (x_dtype == TQ_BF16) {
    out[row * kpad + col] =
        col < k ? reinterpret_cast<const __nv_bfloat16*>(x)[row * ldx + col] : __float2bfloat16_rn(0.f);
  } else {
    float v = col < k ? reinterpret_cast<const float*>(x)[row * ldx + col] : 0.f;
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(mid);
    out[(3 * row + 0) * kpad + col] = hi;
    out[(3 * row + 1) * kpad + col] = mid;
    out[(3 * row + 2) * kpad + col] = __float2bfloat16_rn(r2);
  }
}

template <int KIND>
static cudaError_t launch_nt(int nt, const QGemmParams& p, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  auto go = [&](auto kern) -> cudaError_t {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    kern<<<grid, block, smem, st>>>(p);
    return cudaGetLastError();
  };
  switch (nt) {
    case 1: return go(qgemm_mma_kernel<KIND, 1>);
    case 2: return go(qgemm_mma_kernel<KIND, 2>);
    case 4: return go(qgemm_mma_kernel<KIND, 4>);
    default: return go(qgemm_mma_kernel<KIND, 8>);
  }
}

struct QgConfig {
  int nt, wr, wk, stages;
};

// Launch shape: enough CTAs to cover the SMs about twice with every CTA resident at once (the
// HBM stream is then shared evenly and no tail wave forms), eight consumer warps per CTA, and a
// ring deep enough to keep tens of KB per SM in flight.
static QgConfig choose_config(const tq_ctx* ctx, const tq_qweight* w, int mx) {
  QgConfig c;
  c.nt = mx <= 8 ? 1 : mx <= 16 ? 2 : mx <= 32 ? 4 : 8;
  const int kind = w->kind;
  int wr = c.nt >= 4 ? 4 : 2;
  while (wr > 1 && (long long)((w->rows + 16 * wr - 1) / (16 * wr)) < 2LL * ctx->sm_count) wr >>= 1;
  c.wr = wr;
  c.wk = 8 / wr;
  if (c.nt == 8 && c.wk > 2) c.wk = 2;
  c.stages = 4;
  if (ctx->cfg_wr > 0) {
    c.wr = ctx->cfg_wr;
    c.wk = ctx->cfg_wk;
    c.stages = ctx->cfg_stages;
  }
  // shrink until the CTA fits in shared memory
  while (qg_smem_bytes(kind, c.nt, c.wr, c.wk, c.stages, mx, (int)w->kpad) > 200 * 1024 && c.stages > 2) c.stages--;
  while (qg_smem_bytes(kind, c.nt, c.wr, c.wk, c.stages, mx, (int)w->kpad) > 200 * 1024 && c.wk > 1) c.wk >>= 1;
  return c;
}

// One GEMM launch over <= 64 staged activation rows.
static int launch_qgemm(tq_ctx* ctx, const tq_qweight* w, const __nv_bfloat16* xs, size_t ldxs, int mx, int combine,
                        void* y, int y_dtype, size_t ldy, const float* residual) {
  QgConfig c = choose_config(ctx, w, mx);
  QGemmParams p;
  p.payload = w->payload;
  p.scales = w->scales;
  p.x = xs;
  p.y = y;
  p.residual = residual;
  p.ldw = (long long)w->ldw;
  p.lds = (long long)w->lds;
  p.ldx = (long long)ldxs;
  p.ldy = (long long)ldy;
  p.n_rows = (int)w->rows;
  p.kpad = (int)w->kpad;
  p.mx = mx;
  p.m_out = mx / combine;
  p.combine = combine;
  p.y_bf16 = y_dtype == TQ_BF16;
  p.wr = c.wr;
  p.wk = c.wk;
  p.stages = c.stages;
  p.err = ctx->dev_err;
  const size_t smem = qg_smem_bytes(w->kind, c.nt, c.wr, c.wk, c.stages, mx, p.kpad);
  if (smem > 227 * 1024) return fail(ctx, TQ_EUNSUPPORTED, "tq_qlinear: K=%zu needs %zu bytes of shared memory", w->cols, smem);
  dim3 grid((unsigned)((w->rows + 16 * c.wr - 1) / (16 * c.wr)));
  dim3 block((unsigned)(32 * (c.wr * c.wk + 1)));
  cudaError_t e;
  switch (w->kind) {
    case TQ_Q4_F32: e = launch_nt<Q4_F32>(c.nt, p, grid, block, smem, ctx->stream); break;
    case TQ_Q4_F16: e = launch_nt<Q4_F16>(c.nt, p, grid, block, smem, ctx->stream); break;
    case TQ_Q8_F32: e = launch_nt<Q8_F32>(c.nt, p, grid, block, smem, ctx->stream); break;
    default: e = launch_nt<I8_ROW>(c.nt, p, grid, block, smem, ctx->stream); break;
  }
  ctx->launches++;
  TQ_CUDA(ctx, e);
  return TQ_OK;
}

}  // namespace tq

using namespace tq;

static int make_weight(tq_ctx* ctx, int kind, size_t rows, size_t cols, tq_qweight** out) {
  TQ_REQUIRE(ctx, out != nullptr, "null output handle");
  *out = nullptr;
  TQ_REQUIRE(ctx, kind >= TQ_Q4_F32 && kind <= TQ_I8_ROW, "unknown weight kind %d", kind);
  TQ_REQUIRE(ctx, rows > 0 && cols > 0, "empty weight matrix");
  TQ_REQUIRE(ctx, rows < (1u << 30) && cols < (1u << 30), "weight matrix too large");
  tq_qweight* w = new (std::nothrow) tq_qweight();
  if (!w) return fail(ctx, TQ_ENOMEM, "out of host memory");
  w->kind = kind;
  w->rows = rows;
  w->cols = cols;
  w->kpad = (cols + 31) / 32 * 32;
  w->ldw = is_q4(kind) ? w->kpad / 2 : w->kpad;
  w->lds = kind == TQ_I8_ROW ? 4 : ((w->kpad / 32) * scale_elem(kind) + 15) / 16 * 16;
  *out = w;
  return TQ_OK;
}

static int alloc_weight(tq_ctx* ctx, tq_qweight* w) {
  // 16 spare bytes: the scale-row bulk copy of the last row may read up to the padded row end
  TQ_CUDA(ctx, cudaMalloc(&w->payload, w->rows * w->ldw + 16));
  TQ_CUDA(ctx, cudaMalloc(&w->scales, w->rows * w->lds + 16));
  w->owns = true;
  return TQ_OK;
}

extern "C" {

int tq_qweight_from_arrays(tq_ctx* ctx, int kind, const void* payload_host, const void* scales_host, size_t rows,
                           size_t cols, tq_qweight** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, payload_host && scales_host, "tq_qweight_from_arrays: null array");
  tq_qweight* w = nullptr;
  if (int st = make_weight(ctx, kind, rows, cols, &w)) return st;
  if (int st = alloc_weight(ctx, w)) {
    tq_qweight_free(ctx, w);
    return st;
  }
  const size_t bpr = w->kpad / 32;
  // payload: host rows are whole blocks (Q4/Q8) or exactly `cols` bytes (I8_ROW)
  const size_t host_ldw = kind == TQ_I8_ROW ? cols : w->ldw;
  cudaError_t e = cudaSuccess;
  if (host_ldw != w->ldw) e = cudaMemsetAsync(w->payload, 0, rows * w->ldw, ctx->stream);
  if (e == cudaSuccess)
    e = cudaMemcpy2DAsync(w->payload, w->ldw, payload_host, host_ldw, host_ldw, rows, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) {
    if (kind == TQ_I8_ROW) {
      e = cudaMemcpyAsync(w->scales, scales_host, rows * 4, cudaMemcpyHostToDevice, ctx->stream);
    } else {
      const size_t host_lds = bpr * scale_elem(kind);
      if (host_lds != w->lds) e = cudaMemsetAsync(w->scales, 0, rows * w->lds, ctx->stream);
      if (e == cudaSuccess)
        e = cudaMemcpy2DAsync(w->scales, w->lds, scales_host, host_lds, host_lds, rows, cudaMemcpyHostToDevice, ctx->stream);
    }
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) {
    tq_qweight_free(ctx, w);
    return fail(ctx, TQ_ECUDA, "tq_qweight_from_arrays: %s", cudaGetErrorString(e));
  }
  *out = w;
  return TQ_OK;
}

int tq_qweight_from_blocks(tq_ctx* ctx, int kind, const void* blocks_host, size_t rows, size_t cols,
                           tq_qweight** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, kind == TQ_Q4_F32 || kind == TQ_Q8_F32, "tq_qweight_from_blocks: kind must be TQ_Q4_F32 or TQ_Q8_F32");
  TQ_REQUIRE(ctx, blocks_host != nullptr, "tq_qweight_from_blocks: null blocks");
  TQ_REQUIRE(ctx, rows > 0 && cols > 0, "empty weight matrix");
  const size_t bpr = (cols + 31) / 32, pb = kind == TQ_Q4_F32 ? 16 : 32, bs = 4 + pb;
  std::vector<uint8_t> payload(rows * bpr * pb);
  std::vector<float> scales(rows * bpr);
  const uint8_t* src = static_cast<const uint8_t*>(blocks_host);
  for (size_t b = 0; b < rows * bpr; ++b) {
    std::memcpy(&scales[b], src + b * bs, 4);
    std::memcpy(&payload[b * pb], src + b * bs + 4, pb);
  }
  return tq_qweight_from_arrays(ctx, kind, payload.data(), scales.data(), rows, cols, out);
}

int tq_qweight_wrap_device(tq_ctx* ctx, int kind, const void* payload_dev, const void* scales_dev, size_t rows,
                           size_t cols, tq_qweight** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, payload_dev && scales_dev, "tq_qweight_wrap_device: null array");
  TQ_REQUIRE(ctx, cols % 32 == 0, "tq_qweight_wrap_device: cols must be a multiple of 32");
  tq_qweight* w = nullptr;
  if (int st = make_weight(ctx, kind, rows, cols, &w)) return st;
  const size_t dense_lds = kind == TQ_I8_ROW ? 4 : (cols / 32) * scale_elem(kind);
  if (dense_lds != w->lds || ((uintptr_t)payload_dev & 15) || ((uintptr_t)scales_dev & 15)) {
    delete w;
    return fail(ctx, TQ_EINVAL, "tq_qweight_wrap_device: rows of both arrays must start on 16-byte boundaries");
  }
  w->payload = const_cast<uint8_t*>(static_cast<const uint8_t*>(payload_dev));
  w->scales = const_cast<uint8_t*>(static_cast<const uint8_t*>(scales_dev));
  w->owns = false;
  *out = w;
  return TQ_OK;
}

int tq_qweight_free(tq_ctx* ctx, tq_qweight* w) {
  if (!w) return TQ_OK;
  if (int st = bind(ctx)) return st;
  if (w->owns) {
    cudaStreamSynchronize(ctx->stream);
    if (w->payload) cudaFree(w->payload);
    if (w->scales) cudaFree(w->scales);
  }
  delete w;
  return TQ_OK;
}

int tq_qweight_shape(const tq_qweight* w, size_t* rows, size_t* cols, int* kind) {
  if (!w) return TQ_EINVAL;
  if (rows) *rows = w->rows;
  if (cols) *cols = w->cols;
  if (kind) *kind = w->kind;
  return TQ_OK;
}

size_t tq_qweight_bytes(const tq_qweight* w) {
  if (!w) return 0;
  const size_t bpr = w->kpad / 32;
  const size_t pay = w->rows * (is_q4(w->kind) ? w->kpad / 2 : w->kpad);
  const size_t sc = w->kind == TQ_I8_ROW ? w->rows * 4 : w->rows * bpr * scale_elem(w->kind);
  return pay + sc;
}

int tq_dequantize(tq_ctx* ctx, const tq_qweight* w, float* out_dev, int8_t* ints_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, w != nullptr, "tq_dequantize: null weight");
  TQ_REQUIRE(ctx, out_dev || ints_dev, "tq_dequantize: nothing to write");
  const size_t n = w->rows * (w->kpad / 8);
  dequantize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(w->payload, w->scales, w->ldw, w->lds, w->kind,
                                                                         w->rows, w->cols, w->kpad, out_dev, ints_dev);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

int tq_qlinear_set_config(tq_ctx* ctx, int wr, int wk, int stages) {
  if (!ctx) return TQ_EINVAL;
  if (wr == 0) {
    ctx->cfg_wr = ctx->cfg_wk = ctx->cfg_stages = 0;
    return TQ_OK;
  }
  TQ_REQUIRE(ctx, wr > 0 && wk > 0 && wr * wk <= 8 && stages >= 2 && stages <= 8,
             "tq_qlinear_set_config: need wr*wk <= 8 and 2 <= stages <= 8");
  ctx->cfg_wr = wr;
  ctx->cfg_wk = wk;
  ctx->cfg_stages = stages;
  return TQ_OK;
}

int tq_qlinear(tq_ctx* ctx, const tq_qweight* w, const void* x_dev, int x_dtype, size_t ldx, size_t m, void* y_dev,
               int y_dtype, size_t ldy, const float* residual_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, w != nullptr, "tq_qlinear: null weight");
  TQ_REQUIRE(ctx, x_dtype == TQ_BF16 || x_dtype == TQ_F32, "tq_qlinear: x must be bf16 or f32");
  TQ_REQUIRE(ctx, y_dtype == TQ_BF16 || y_dtype == TQ_F32, "tq_qlinear: y must be bf16 or f32");
  if (m == 0) return TQ_OK;  // empty batch: nothing to do (Linear::forward_2d on zero rows)
  TQ_REQUIRE(ctx, x_dev && y_dev, "tq_qlinear: null activation pointer");
  if (ldx == 0) ldx = w->cols;
  if (ldy == 0) ldy = w->rows;
  TQ_REQUIRE(ctx, ldx >= w->cols && ldy >= w->rows, "tq_qlinear: row stride smaller than the row");
  TQ_REQUIRE(ctx, !(residual_dev && y_dtype == TQ_BF16 && (const void*)residual_dev == y_dev),
             "tq_qlinear: residual may alias y only for f32 output");

  const int combine = x_dtype == TQ_F32 ? 3 : 1;
  const size_t chunk = x_dtype == TQ_F32 ? 21 : 64;
  const bool direct = x_dtype == TQ_BF16 && w->cols == w->kpad && ldx % 8 == 0 && ((uintptr_t)x_dev & 15) == 0;
  if (!direct) {
    const size_t rows_staged = (m < chunk ? m : chunk) * combine;
    if (int st = ensure_xprep(ctx, rows_staged * w->kpad * 2)) return st;
  }
  const size_t xe = x_dtype == TQ_F32 ? 4 : 2, ye = y_dtype == TQ_F32 ? 4 : 2;
  for (size_t m0 = 0; m0 < m; m0 += chunk) {
    const size_t mc = m - m0 < chunk ? m - m0 : chunk;
    const uint8_t* xc = static_cast<const uint8_t*>(x_dev) + m0 * ldx * xe;
    uint8_t* yc = static_cast<uint8_t*>(y_dev) + m0 * ldy * ye;
    const float* rc = residual_dev ? residual_dev + m0 * ldy : nullptr;
    const __nv_bfloat16* xs;
    size_t ldxs;
    if (direct) {
      xs = reinterpret_cast<const __nv_bfloat16*>(xc);
      ldxs = ldx;
    } else {
      const size_t n = mc * w->kpad;
      prep_x_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(xc, x_dtype, ldx, mc, w->cols, w->kpad,
                                                                         static_cast<__nv_bfloat16*>(ctx->xprep));
      ctx->launches++;
      TQ_CUDA(ctx, cudaGetLastError());
      xs = static_cast<const __nv_bfloat16*>(ctx->xprep);
      ldxs = w->kpad;
    }
    if (int st = launch_qgemm(ctx, w, xs, ldxs, (int)(mc * combine), combine, yc, y_dtype, ldy, rc)) return st;
  }
  return TQ_OK;
}

int tq_q_matvec_host(tq_ctx* ctx, const tq_qweight* w, const void* x_host, void* y_host, int dtype, size_t m) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, w != nullptr, "tq_q_matvec_host: null weight");
  TQ_REQUIRE(ctx, dtype == TQ_F64 || dtype == TQ_F32 || dtype == TQ_BF16, "tq_q_matvec_host: dtype must be f64, f32 or bf16");
  if (m == 0) return TQ_OK;
  TQ_REQUIRE(ctx, x_host && y_host, "tq_q_matvec_host: null vector");
  const size_t nx = m * w->cols, ny = m * w->rows;
  const size_t es = dtype == TQ_F64 ? 8 : dtype == TQ_F32 ? 4 : 2;
  const size_t dev_es = dtype == TQ_BF16 ? 2 : 4;
  // scratch: [x as uploaded][x as consumed][y as produced][y as downloaded]
  const size_t off_x2 = (nx * es + 255) / 256 * 256;
  const size_t off_y = off_x2 + (nx * dev_es + 255) / 256 * 256;
  const size_t off_y2 = off_y + (ny * dev_es + 255) / 256 * 256;
  if (int st = ensure_scratch(ctx, off_y2 + ny * es)) return st;
  uint8_t* s = static_cast<uint8_t*>(ctx->scratch);
  TQ_CUDA(ctx, cudaMemcpyAsync(s, x_host, nx * es, cudaMemcpyHostToDevice, ctx->stream));
  const void* xd = s;
  if (dtype == TQ_F64) {
    if (int st = tq_convert(ctx, s, TQ_F64, s + off_x2, TQ_F32, nx)) return st;
    xd = s + off_x2;
  }
  const int dev_dt = dtype == TQ_BF16 ? TQ_BF16 : TQ_F32;
  if (int st = tq_qlinear(ctx, w, xd, dev_dt, 0, m, s + off_y, dev_dt, 0, nullptr)) return st;
  const void* yd = s + off_y;
  if (dtype == TQ_F64) {
    if (int st = tq_convert(ctx, s + off_y, TQ_F32, s + off_y2, TQ_F64, ny)) return st;
    yd = s + off_y2;
  }
  TQ_CUDA(ctx, cudaMemcpyAsync(y_host, yd, ny * es, cudaMemcpyDeviceToHost, ctx->stream));
  return tq_sync(ctx);
}

}  // extern "C"
