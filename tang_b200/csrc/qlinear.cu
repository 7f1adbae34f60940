// Quantised weights and the quantised linear layer of the C ABI (include/tangq.h).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "internal.h"
#include "qgemm_mma.cuh"
#include "qgemv_sk.cuh"
#include "qgemm_sk.cuh"
#include "qgemm_skg.cuh"

namespace tq {

static inline bool is_q4(int kind) { return kind == TQ_Q4_F32 || kind == TQ_Q4_F16; }
static inline size_t scale_elem(int kind) { return kind == TQ_Q4_F16 ? 2 : 4; }

// ---------------------------------------------------------------------------------------------
// Repack: plain block arrays (payload [rows][ld_pay], scales [rows][ld_sc]) -> fragment tiles.
// One thread per (tile, half, lane, block): it moves the eight weights of one lane-block and,
// for t == 0, the block's scale.  Integer codes and scale bits are copied, never recomputed.
// ---------------------------------------------------------------------------------------------
__global__ void repack_kernel(const uint8_t* pay, const uint8_t* sc, size_t ld_pay, size_t ld_sc, int kind, size_t rows,
                              size_t cols, int n_rb, int n_kc, uint8_t* tiles) {
  const size_t total = (size_t)n_rb * n_kc * 2 * 32 * 4;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int j = idx & 3;
  const int lane = (idx >> 2) & 31;
  const int h = (idx >> 7) & 1;
  const size_t tile_idx = idx >> 8;
  const int kc = (int)(tile_idx % n_kc);
  const size_t rb = tile_idx / n_kc;
  const int g = lane >> 2, t = lane & 3;
  const size_t row = rb * 16 + g + 8 * h;
  const size_t k0 = (size_t)kc * kTileK + 32 * j + 8 * t;   // first of this thread's eight k
  const size_t kblocks = (cols + 31) / 32;                   // blocks present per input row
  const bool live = row < rows && (k0 / 32) < kblocks;
  uint8_t* tile = tiles + tile_idx * qk_tile_bytes(kind);
  if (kind == Q4_F32 || kind == Q4_F16) {
    uint32_t w = 0x88888888u;  // eight zeros (stored q+8)
    if (live) w = *reinterpret_cast<const uint32_t*>(pay + row * ld_pay + k0 / 2);
    // nibble i of w is k0+i; output nibble order k0+{0,2,4,6,1,3,5,7}
    uint32_t o = 0;
#pragma unroll
    for (int pos = 0; pos < 8; ++pos) {
      const int src = pos < 4 ? 2 * pos : 2 * (pos - 4) + 1;
      o |= ((w >> (4 * src)) & 0xFu) << (4 * pos);
    }
    *reinterpret_cast<uint32_t*>(tile + h * 512 + 16 * lane + 4 * j) = o;
  } else {
    uint2 w = make_uint2(0u, 0u);
    if (live) {
      if (kind == I8_ROW) {  // rows are exactly `cols` bytes: guard the tail byte by byte
        uint8_t b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = (k0 + i < cols) ? pay[row * ld_pay + k0 + i] : 0;
        w.x = b[0] | (b[1] << 8) | (b[2] << 16) | ((uint32_t)b[3] << 24);
        w.y = b[4] | (b[5] << 8) | (b[6] << 16) | ((uint32_t)b[7] << 24);
      } else {
        w = *reinterpret_cast<const uint2*>(pay + row * ld_pay + k0);
      }
    }
    // bytes k0..k0+7 -> [k0,k2,k4,k6][k1,k3,k5,k7]
    const uint32_t even = prmt(w.x, w.y, 0x6420u), odd = prmt(w.x, w.y, 0x7531u);
    const int pl = j >> 1;
    *reinterpret_cast<uint2*>(tile + h * 1024 + pl * 512 + 16 * lane + 8 * (j & 1)) = make_uint2(even, odd);
  }
  if (t == 0 && kind != I8_ROW) {
    const int off = qk_scale_offset(kind, g + 8 * h, j);
    if (kind == Q4_F16) {
      uint16_t v = 0;
      if (live) v = *reinterpret_cast<const uint16_t*>(sc + row * ld_sc + 2 * (k0 / 32));
      *reinterpret_cast<uint16_t*>(tile + off) = v;
    } else {
      uint32_t v = 0;
      if (live) v = *reinterpret_cast<const uint32_t*>(sc + row * ld_sc + 4 * (k0 / 32));
      *reinterpret_cast<uint32_t*>(tile + off) = v;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// dequantize_q4 / dequantize_q8 (crates/tang-infer/src/quantize.rs:73-81,121-132) through the same
// register dequantisers the GEMM uses, reading the fragment tiles: a bit-exact check of this
// kernel's integers is a check of the repack and of the GEMM's unpack.  One thread per eight k.
// ---------------------------------------------------------------------------------------------
__global__ void dequantize_kernel(const uint8_t* tiles, const float* row_scales, int kind, size_t rows, size_t cols,
                                  int n_kc, float* out, int8_t* ints) {
  const size_t per_row = (size_t)n_kc * 16;  // eight-k units per row
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const size_t row = idx / per_row, oct = idx % per_row;
  const int kc = (int)(oct / 16), j = (int)(oct % 16) / 4, t = (int)(oct % 4);
  const size_t k0 = (size_t)kc * kTileK + 32 * j + 8 * t;
  const int r = (int)(row % 16), h = r >> 3, g = r & 7, lane = 4 * g + t;
  const uint8_t* tile = tiles + ((row / 16) * n_kc + kc) * qk_tile_bytes(kind);
  uint32_t v[4];
  if (kind == Q4_F32 || kind == Q4_F16) {
    dequant_q4_word(*reinterpret_cast<const uint32_t*>(tile + h * 512 + 16 * lane + 4 * j), v);
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(tile + h * 1024 + (j >> 1) * 512 + 16 * lane + 8 * (j & 1));
    dequant_i8_words(u.x, u.y, v);
  }
  float scale;
  if (kind == I8_ROW) scale = row_scales[row];
  else if (kind == Q4_F16) scale = __half2float(*reinterpret_cast<const __half*>(tile + qk_scale_offset(kind, r, j)));
  else scale = *reinterpret_cast<const float*>(tile + qk_scale_offset(kind, r, j));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = bf16_bits_to_float(v[i] & 0xFFFFu), hi = bf16_bits_to_float(v[i] >> 16);  // k0+2i, k0+2i+1
    if (k0 + 2 * i < cols) {
      if (out) out[row * cols + k0 + 2 * i] = lo * scale;
      if (ints) ints[row * cols + k0 + 2 * i] = (int8_t)(int)lo;
    }
    if (k0 + 2 * i + 1 < cols) {
      if (out) out[row * cols + k0 + 2 * i + 1] = hi * scale;
      if (ints) ints[row * cols + k0 + 2 * i + 1] = (int8_t)(int)hi;
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
static cudaError_t launch_nt(tq_ctx* ctx, int nt, const QGemmParams& p, dim3 grid, dim3 block, size_t smem) {
  auto go = [&](auto kern) -> cudaError_t {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    return launch_k(ctx, kern, grid, block, smem, p);
  };
  switch (nt) {
    case 1: return go(qgemm_mma_kernel<KIND, 1>);
    case 2: return go(qgemm_mma_kernel<KIND, 2>);
    case 4: return go(qgemm_mma_kernel<KIND, 4>);
    default: return go(qgemm_mma_kernel<KIND, 8>);
  }
}

struct QgConfig {
  int nt, wr, wk, tpw, stages;
};

// Launch shape: enough CTAs to cover the SMs about twice with every CTA resident at once (the
// HBM stream is then shared evenly and no tail wave forms), eight consumer warps per CTA, and a
// ring deep enough to keep tens of KB per SM in flight.
static QgConfig choose_config(const tq_ctx* ctx, const tq_qweight* w, int mx, int n_rb, int n_groups) {
  QgConfig c;
  c.nt = mx <= 8 ? 1 : mx <= 16 ? 2 : mx <= 32 ? 4 : 8;
  int wr = c.nt >= 4 ? 4 : 2;
  while (wr > 1 && (long long)((n_rb + wr - 1) / wr) * n_groups < 2LL * ctx->sm_count) wr >>= 1;
  c.wr = wr;
  c.wk = 8 / wr;
  if (c.nt == 8 && c.wk > 2) c.wk = 2;
  c.stages = 4;
  c.tpw = 1;
  while (c.wk > 1 && c.wk > w->n_kc) c.wk >>= 1;
  while (c.tpw > 1 && c.wk * c.tpw > w->n_kc) c.tpw >>= 1;
  // shrink until the CTA fits in shared memory
  while (qg_smem_bytes(w->kind, c.nt, c.wr, c.wk, c.tpw, c.stages, mx) > 200 * 1024 && c.stages > 2) c.stages--;
  while (qg_smem_bytes(w->kind, c.nt, c.wr, c.wk, c.tpw, c.stages, mx) > 200 * 1024 && c.tpw > 1) c.tpw >>= 1;
  while (qg_smem_bytes(w->kind, c.nt, c.wr, c.wk, c.tpw, c.stages, mx) > 200 * 1024 && c.wk > 1) c.wk >>= 1;
  return c;
}

struct QgGroup {
  int n_groups = 1;
  const int* counts = nullptr;    // device: rows routed to each group (expert batches)
  const int* offsets = nullptr;   // device: first row of each group in x / y
  long long x_stride = 0, y_stride = 0;  // elements between groups when counts == nullptr
  int max_rows = 0;               // upper bound of counts[e] (sizes gridDim.z)
  const int* active = nullptr;    // device: ids of the groups that have rows, then -1s
  int max_active = 0;             // upper bound of how many groups can have rows (sizes gridDim.y)
};

// ---------------------------------------------------------------------------------------------
// Persistent GEMV (qgemv_sk.cuh) for up to eight staged activation rows of an ungrouped weight.
// Returns false when the shape does not fit it (the ring would be shorter than three stages);
// the caller then uses the general kernel.
// ---------------------------------------------------------------------------------------------
// Two CTA shapes, both with 16 tiles per stage: 8 warps x 2 tiles for a kernel that has an SM to itself (it waits
// for its activations: only its ring fills early), 4 warps x 4 tiles for kernels that run four to an SM.
template <int KIND, bool M1, int W, int TPW, int MINB>
static cudaError_t launch_sk_kernel(tq_ctx* ctx, const QGemvParams& p, unsigned grid, size_t smem) {
  auto kern = qgemv_sk_kernel<KIND, W, TPW, M1, MINB>;
  static size_t attr_bytes[64] = {};   // per device: the attribute belongs to the device's copy of the kernel
  const int dev = ctx->device & 63;
  if (smem > 48 * 1024 && attr_bytes[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_bytes[dev] = smem;
  }
  return launch_k(ctx, kern, dim3(grid), dim3(32 * (W + 2)), smem, p);
}

template <int KIND>
static cudaError_t launch_sk_kind(tq_ctx* ctx, const QGemvParams& p, unsigned grid, size_t smem, bool m1, bool small) {
  if (small) return m1 ? launch_sk_kernel<KIND, true, 4, 4, 4>(ctx, p, grid, smem) : launch_sk_kernel<KIND, false, 4, 4, 4>(ctx, p, grid, smem);
  return m1 ? launch_sk_kernel<KIND, true, 8, 2, 3>(ctx, p, grid, smem) : launch_sk_kernel<KIND, false, 8, 2, 3>(ctx, p, grid, smem);
}

// ---------------------------------------------------------------------------------------------
// Persistent GEMM for 2..8 staged activation rows (qgemm_sk.cuh): K in slabs, so that a CTA holds
// only a slab of the activation rows beside its weight ring.  Returns false when the shape does
// not fit; the caller then uses another kernel.
// ---------------------------------------------------------------------------------------------
template <int KIND, int TPW, bool SS>
static cudaError_t launch_skw_kernel(tq_ctx* ctx, const QGemvParams& p, unsigned grid, size_t smem) {
  auto kern = qgemm_sk_kernel<KIND, 8, TPW, 1, 2, SS>;
  static size_t attr_bytes[64] = {};   // per device
  const int dev = ctx->device & 63;
  if (smem > 48 * 1024 && attr_bytes[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_bytes[dev] = smem;
  }
  return launch_k(ctx, kern, dim3(grid), dim3(32 * 10), smem, p);
}

template <int KIND>
static cudaError_t launch_skw_kind(tq_ctx* ctx, const QGemvParams& p, unsigned grid, size_t smem, int tpw, int nt) {
  (void)nt;   // one column tile of eight rows: the launcher takes up to eight rows
  // (the variant that hands sums of squares over is a kernel of its own: the plain one pays nothing for it)
  if (p.ss_out || p.ss_in)
    return tpw == 2 ? launch_skw_kernel<KIND, 2, true>(ctx, p, grid, smem) : launch_skw_kernel<KIND, 1, true>(ctx, p, grid, smem);
  return tpw == 2 ? launch_skw_kernel<KIND, 2, false>(ctx, p, grid, smem) : launch_skw_kernel<KIND, 1, false>(ctx, p, grid, smem);
}

static bool launch_qgemm_sk(tq_ctx* ctx, const tq_qweight* w, const __nv_bfloat16* xs, size_t ldxs, int mx, int combine,
                            void* y, int y_dtype, size_t ldy, const float* residual, int* status, const QlinearNorm* norm,
                            bool swiglu, const unsigned* x_tag, unsigned x_seq, const unsigned* x_epoch) {
  // (measured per 14336 x 4096 launch in a dependent chain: 12-15 us for 4-8 rows, but 26 us for 16 rows with their
  // eight-tile stages, against about 20 us for the general kernel: more than eight rows stay there)
  if (mx < 2 || mx > 8) return false;
  if (w->cols != (size_t)w->n_kc * kTileK && norm) return false;
  const int nt = (mx + 7) / 8;
  const int kc_total = w->n_kc;
  // slab width: the largest divisor of the chunk count whose slab of activation rows stays near 36 KB
  int skc_max = 36864 / (mx * 256);
  if (skc_max > 32) skc_max = 32;
  int skc = 0;
  for (int d = skc_max < kc_total ? skc_max : kc_total; d >= 1; --d)
    if (kc_total % d == 0) {
      skc = d;
      break;
    }
  if (skc < 4 && skc != kc_total) return false;
  const int n_slabs = kc_total / skc;
  const long long units = (long long)w->n_rb * skc;
  long long cps = 2LL * ctx->sm_count / n_slabs;
  if (cps < 1) cps = 1;
  if (cps > units) cps = units;
  const long long grid = cps * n_slabs;
  if (grid > kGemvMaxGrid || grid * 2 * nt > (long long)kGemvSets * kGemvMaxGrid * 2) return false;
  const int tpw = skc >= 16 ? 2 : 1;
  const size_t stage = (size_t)8 * tpw * qk_tile_bytes(w->kind);
  const size_t fixed = skw_fixed_bytes(w->kind, 8, skc, mx, nt);
  const size_t budget = 113 * 1024;
  if (fixed + 3 * stage > budget) return false;
  int stages = (int)((budget - fixed) / stage);
  if (stages > kSkMaxStages) stages = kSkMaxStages;
  const size_t smem = fixed + (size_t)stages * stage;
  if (n_slabs > 1) {
    *status = ensure_gemm_ws2(ctx, (size_t)n_slabs * w->n_rb * nt * 128 * sizeof(unsigned long long));
    if (*status != TQ_OK) return true;
  }
  const int kx = kc_total * kTileK;
  const int m_out = mx / combine;
  // the kernel may read its activations at once when nothing that may still be running writes them
  struct R { uintptr_t lo, hi; };
  const R rx = norm ? R{(uintptr_t)norm->h, (uintptr_t)norm->h + ((size_t)(mx - 1) * kx + kx) * 4}
                    : R{(uintptr_t)xs, (uintptr_t)xs + ((size_t)(mx - 1) * ldxs + kx) * 2};
  const R ry = {(uintptr_t)y, (uintptr_t)y + ((size_t)(m_out - 1) * ldy + w->rows) * (y_dtype == TQ_BF16 ? 2 : 4)};
  const R rr = {(uintptr_t)residual, residual ? (uintptr_t)residual + ((size_t)(m_out - 1) * ldy + w->rows) * 4 : (uintptr_t)residual};
  auto hit = [](const R& a, const tq_ctx::Range& b) { return a.lo < b.hi && b.lo < a.hi; };
  int mode = (ctx->owns_stream && ctx->pdl && !ctx->inflight_unknown && ctx->n_inflight + 3 <= 96 && !norm) ? 1 : 0;
  for (int i = 0; mode && i < ctx->n_inflight; ++i)
    if (ctx->inflight[i].written && hit(rx, ctx->inflight[i])) mode = 0;
  QGemvParams p;
  p.tiles = w->tiles;
  p.row_scales = w->row_scales;
  p.x = xs;
  p.y = y;
  p.residual = residual;
  p.ldx = (long long)ldxs;
  p.ldy = (long long)ldy;
  p.n_units = units;
  p.n_rows = (int)w->rows;
  p.n_row_blocks = w->n_rb;
  p.kc_total = kc_total;
  p.kx = kx;
  p.mx = mx;
  p.m_out = m_out;
  p.combine = combine;
  p.y_bf16 = y_dtype == TQ_BF16;
  p.stages = stages;
  p.nh = norm ? norm->h : nullptr;
  p.ndelta = norm ? norm->delta : nullptr;
  p.norm_w = norm ? static_cast<const __nv_bfloat16*>(norm->gain_bf16) : nullptr;
  p.nh_out = norm ? norm->h_out : nullptr;
  p.ld_h = kx;
  p.norm_eps = norm ? norm->eps : 0.f;
  p.ss_in = norm ? norm->sumsq : nullptr;
  p.ss_n = norm ? norm->n_sumsq : 0;
  // (asked for by the caller of the enclosing operator: the row sums of squares of what this launch stores)
  p.ss_out = (ctx->ss_req && !swiglu && combine == 1 && y_dtype == TQ_F32) ? ctx->ss_req : nullptr;
  if (p.ss_out) ctx->ss_written = true;
  p.swiglu = swiglu ? 1 : 0;
  p.x_tag = x_tag;
  p.x_seq = x_seq;
  p.x_epoch = x_epoch;
  p.x_early = mode;
  p.skc = skc;
  p.n_slabs = n_slabs;
  p.cps = (int)cps;
  p.ws = ctx->gemv_ws;
  p.ws2 = ctx->gemm_ws2;
  p.err = ctx->dev_err;
  cudaError_t e;
  switch (w->kind) {
    case TQ_Q4_F32: e = launch_skw_kind<Q4_F32>(ctx, p, (unsigned)grid, smem, tpw, nt); break;
    case TQ_Q4_F16: e = launch_skw_kind<Q4_F16>(ctx, p, (unsigned)grid, smem, tpw, nt); break;
    case TQ_Q8_F32: e = launch_skw_kind<Q8_F32>(ctx, p, (unsigned)grid, smem, tpw, nt); break;
    default: e = launch_skw_kind<I8_ROW>(ctx, p, (unsigned)grid, smem, tpw, nt); break;
  }
  *status = e == cudaSuccess ? TQ_OK : fail(ctx, TQ_ECUDA, "persistent GEMM launch failed: %s", cudaGetErrorString(e));
  if (e == cudaSuccess && !norm) {   // (launch_k has just marked the stream's state unknown)
    if (mode == 0) ctx->n_inflight = 0;
    ctx->inflight_unknown = false;
    ctx->inflight[ctx->n_inflight++] = {rx.lo, rx.hi, false};
    ctx->inflight[ctx->n_inflight++] = {ry.lo, ry.hi, true};
    if (residual) ctx->inflight[ctx->n_inflight++] = {rr.lo, rr.hi, false};
  }
  return true;
}

static bool launch_qgemv_sk(tq_ctx* ctx, const tq_qweight* w, const __nv_bfloat16* xs, size_t ldxs, int mx, int combine,
                            void* y, int y_dtype, size_t ldy, const float* residual, int* status,
                            const QlinearNorm* norm = nullptr, bool swiglu = false, const unsigned* x_tag = nullptr,
                            unsigned x_seq = 0, const unsigned* x_epoch = nullptr) {
  if (mx >= 2 && launch_qgemm_sk(ctx, w, xs, ldxs, mx, combine, y, y_dtype, ldy, residual, status, norm, swiglu, x_tag, x_seq, x_epoch)) return true;
  if (mx > 8) return false;
  if (norm && (w->cols != (size_t)w->n_kc * kTileK)) return false;   // the fused norm wants whole 128-k chunks
  const bool m1 = mx == 1;
  const int kx = w->n_kc * kTileK;
  const size_t stage = (size_t)16 * qk_tile_bytes(w->kind);
  const long long units = (long long)w->n_rb * w->n_kc;
  long long grid = ctx->sm_count;
  if (grid > kGemvMaxGrid) grid = kGemvMaxGrid;
  if (grid > units) grid = units;
  // What may still be running when this kernel starts decides how it is launched: 0 = it waits for its
  // activations, 1 = it reads them at once and only its stores wait, 2 = nothing in flight touches its operands.
  // Only on a stream of the context's own: on an adopted stream a foreign kernel that lets its dependents start
  // early could sit between two of these launches.
  struct R { uintptr_t lo, hi; };
  const int m_out = mx / combine;
  const R rx = norm ? R{(uintptr_t)norm->h, (uintptr_t)norm->h + ((size_t)(mx - 1) * kx + kx) * 4}
                    : R{(uintptr_t)xs, (uintptr_t)xs + ((size_t)(mx - 1) * ldxs + kx) * 2};
  const R ry = {(uintptr_t)y, (uintptr_t)y + ((size_t)(m_out - 1) * ldy + w->rows) * (y_dtype == TQ_BF16 ? 2 : 4)};
  const R rr = {(uintptr_t)residual, residual ? (uintptr_t)residual + ((size_t)(m_out - 1) * ldy + w->rows) * 4 : (uintptr_t)residual};
  auto hit = [](const R& a, const tq_ctx::Range& b) { return a.lo < b.hi && b.lo < a.hi; };
  int mode = (ctx->owns_stream && ctx->pdl && !ctx->inflight_unknown && ctx->n_inflight + 3 <= 96 && !norm) ? 2 : 0;
  for (int i = 0; mode && i < ctx->n_inflight; ++i) {
    const tq_ctx::Range& f = ctx->inflight[i];
    if (f.written && hit(rx, f)) mode = 0;                                     // x comes from a kernel that may still run
    else if (hit(ry, f) || (f.written && hit(rr, f))) mode = 1;                // only the stores / the residual have to wait
  }
  // Shared memory per CTA.  Kernels that wait for nothing run side by side: four small CTAs per SM (a two-stage
  // ring each) keep the most copies in flight and the most warps busy (measured per 14336 x 4096 launch: 5.8 us,
  // against 6.3 us for three CTAs of eight warps and 6.9 us for two).
  const size_t quarter = 56 * 1024, third = 74 * 1024, half = 113 * 1024, most = 150 * 1024, whole = 226 * 1024;
  // (with nothing in flight the kernel has the GPU to itself, like one that waits: the larger shape below)
  const bool small = mode == 2 && ctx->n_inflight > 0 && sk_fixed_bytes(w->kind, 4, kx, mx, m1) + 2 * stage <= quarter;
  const size_t fixed = sk_fixed_bytes(w->kind, small ? 4 : 8, kx, mx, m1);
  size_t budget = whole;
  if (small) budget = quarter;
  else if (mode == 2 && ctx->n_inflight > 0 && fixed + 3 * stage <= third) budget = third;
  else if (fixed + 3 * stage <= half) {
    // A kernel that waits (for its activations or before its stores): two CTAs per SM, and a grid that fills both
    // slots of every SM so that none is handed two while another gets none (a grid of one CTA per SM with room for
    // two measured 2.48 ms per decode step; one large CTA per SM 1.89 ms; this 1.79 ms).
    budget = half;
    if (units >= 2LL * ctx->sm_count * 8) grid = 2LL * ctx->sm_count;
    // A short matrix with 1.5 to 2 row blocks per SM (the 4096 x 4096 output projection): one whole row block per
    // CTA.  No row block is cut, so nothing is parked and nobody waits at the end, which for so few bytes is worth
    // more than the last 14 % of the slots (same-box decode step at one row: 1.82 -> 1.78 ms).  Fewer row blocks or
    // shorter rows (the tensor-parallel shards) measured no better that way and keep the even split.
    if (w->n_kc >= 24 && w->n_kc <= 48 && 2 * w->n_rb >= 3 * ctx->sm_count && w->n_rb <= 2 * ctx->sm_count) grid = w->n_rb;
  } else if (fixed + 3 * stage <= most) budget = most;
  if (fixed + 2 * stage > budget) return false;
  int stages = (int)((budget - fixed) / stage);
  if (stages > kSkMaxStages) stages = kSkMaxStages;
  const size_t smem = fixed + (size_t)stages * stage;
  // Running entirely unordered relies on the rotating workspace sets: a CTA only leaves once the kernel before
  // its own has completed, so kernel n and kernel n + kGemvSets can both have resident CTAs only if kGemvSets - 1
  // whole grids fit on the GPU beside one more CTA.  Grids of at least one CTA per SM rule that out.
  const long long resident = (long long)(233472 / (smem + 1024)) * ctx->sm_count;   // CTAs of this shape the GPU can hold
  if (mode == 2 && !(grid >= ctx->sm_count && (long long)(kGemvSets - 1) * grid >= resident)) mode = 1;
  QGemvParams p;
  p.tiles = w->tiles;
  p.row_scales = w->row_scales;
  p.x = xs;
  p.y = y;
  p.residual = residual;
  p.ldx = (long long)ldxs;
  p.ldy = (long long)ldy;
  p.n_units = units;
  p.n_rows = (int)w->rows;
  p.n_row_blocks = w->n_rb;
  p.kc_total = w->n_kc;
  p.kx = kx;
  p.mx = mx;
  p.m_out = m_out;
  p.combine = combine;
  p.y_bf16 = y_dtype == TQ_BF16;
  p.stages = stages;
  p.nh = norm ? norm->h : nullptr;
  p.ndelta = norm ? norm->delta : nullptr;
  p.norm_w = norm ? static_cast<const __nv_bfloat16*>(norm->gain_bf16) : nullptr;
  p.nh_out = norm ? norm->h_out : nullptr;
  p.ld_h = kx;
  p.norm_eps = norm ? norm->eps : 0.f;
  p.ss_in = nullptr;   // (this kernel neither reads nor leaves sums of squares)
  p.ss_n = 0;
  p.ss_out = nullptr;
  p.swiglu = swiglu ? 1 : 0;
  p.x_tag = x_tag;
  p.x_seq = x_seq;
  p.x_epoch = x_epoch;
  p.x_early = mode;
  const unsigned set = ctx->gemv_seq++ % kGemvSets;
  p.ws = ctx->gemv_ws + (size_t)set * kGemvMaxGrid * 2 * 128;
  p.err = ctx->dev_err;
  cudaError_t e;
  switch (w->kind) {
    case TQ_Q4_F32: e = launch_sk_kind<Q4_F32>(ctx, p, (unsigned)grid, smem, m1, small); break;
    case TQ_Q4_F16: e = launch_sk_kind<Q4_F16>(ctx, p, (unsigned)grid, smem, m1, small); break;
    case TQ_Q8_F32: e = launch_sk_kind<Q8_F32>(ctx, p, (unsigned)grid, smem, m1, small); break;
    default: e = launch_sk_kind<I8_ROW>(ctx, p, (unsigned)grid, smem, m1, small); break;
  }
  *status = e == cudaSuccess ? TQ_OK : fail(ctx, TQ_ECUDA, "persistent GEMV launch failed: %s", cudaGetErrorString(e));
  if (e == cudaSuccess && !norm) {   // (launch_k has just marked the stream's state unknown; a fused norm also writes
                                     // h_out, so what follows it simply waits)
    if (mode == 0) ctx->n_inflight = 0;   // this kernel waits for everything before it
    ctx->inflight_unknown = false;
    ctx->inflight[ctx->n_inflight++] = {rx.lo, rx.hi, false};
    ctx->inflight[ctx->n_inflight++] = {ry.lo, ry.hi, true};
    if (residual) ctx->inflight[ctx->n_inflight++] = {rr.lo, rr.hi, false};
  }
  return true;
}

// One GEMM launch over <= 64 staged activation rows (per group, for grouped launches).
static int launch_qgemm(tq_ctx* ctx, const tq_qweight* w, const __nv_bfloat16* xs, size_t ldxs, int mx, int combine,
                        void* y, int y_dtype, size_t ldy, const float* residual, const QgGroup* grp = nullptr) {
  if (!grp) {
    int st = TQ_OK;
    if (launch_qgemv_sk(ctx, w, xs, ldxs, mx, combine, y, y_dtype, ldy, residual, &st)) return st;
  }
  const int n_groups = grp ? grp->n_groups : 1;
  const int n_rb = w->n_rb / n_groups;
  const size_t rows_g = w->rows / n_groups;
  QgConfig c = choose_config(ctx, w, mx, n_rb, n_groups);
  QGemmParams p;
  p.tiles = w->tiles;
  p.row_scales = w->row_scales;
  p.x = xs;
  p.y = y;
  p.residual = residual;
  p.ldx = (long long)ldxs;
  p.ldy = (long long)ldy;
  p.n_rows = (int)rows_g;
  p.n_row_blocks = n_rb;
  p.kc_total = w->n_kc;
  p.kx = w->n_kc * kTileK;
  p.mx = mx;
  p.m_out = mx / combine;
  p.combine = combine;
  p.y_bf16 = y_dtype == TQ_BF16;
  p.wr = c.wr;
  p.wk = c.wk;
  p.stages = c.stages;
  p.tpw = c.tpw;
  p.err = ctx->dev_err;
  p.grouped = grp ? 1 : 0;
  p.g_counts = grp ? grp->counts : nullptr;
  p.g_offsets = grp ? grp->offsets : nullptr;
  p.g_active = grp ? grp->active : nullptr;
  p.g_tile_stride = (long long)n_rb * w->n_kc * qk_tile_bytes(w->kind);
  p.g_x_stride = grp ? grp->x_stride : 0;
  p.g_y_stride = grp ? grp->y_stride : 0;
  const size_t smem = qg_smem_bytes(w->kind, c.nt, c.wr, c.wk, c.tpw, c.stages, mx);
  if (smem > 227 * 1024) return fail(ctx, TQ_EUNSUPPORTED, "tq_qlinear: launch needs %zu bytes of shared memory", smem);
  const int chunk = 8 * c.nt;
  const unsigned gz = (grp && grp->counts) ? (unsigned)((grp->max_rows + chunk - 1) / chunk) : 1u;
  const int gy = (grp && grp->active && grp->max_active < n_groups) ? grp->max_active : n_groups;
  dim3 grid((unsigned)((n_rb + c.wr - 1) / c.wr), (unsigned)gy, gz ? gz : 1u);
  dim3 block((unsigned)(32 * (c.wr * c.wk + 1)));
  cudaError_t e;
  switch (w->kind) {
    case TQ_Q4_F32: e = launch_nt<Q4_F32>(ctx, c.nt, p, grid, block, smem); break;
    case TQ_Q4_F16: e = launch_nt<Q4_F16>(ctx, c.nt, p, grid, block, smem); break;
    case TQ_Q8_F32: e = launch_nt<Q8_F32>(ctx, c.nt, p, grid, block, smem); break;
    default: e = launch_nt<I8_ROW>(ctx, c.nt, p, grid, block, smem); break;
  }
  TQ_CUDA(ctx, e);
  return TQ_OK;
}

// Grouped launch entry for the other translation units (MoE experts, per-head MLA projections).
// ---------------------------------------------------------------------------------------------
// Grouped persistent kernel (qgemm_skg.cuh) for expert batches / per-head matrices with 8..17 k chunks.
// Returns false when the shape does not fit; the caller then uses the general kernel.
// ---------------------------------------------------------------------------------------------
template <int KIND, int TPW>
static cudaError_t launch_skg_kernel(tq_ctx* ctx, const QGroupParams& p, dim3 grid, size_t smem) {
  auto kern = qgemm_skg_kernel<KIND, 8, TPW>;
  static size_t attr_bytes[64] = {};   // per device
  const int dev = ctx->device & 63;
  if (smem > 48 * 1024 && attr_bytes[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_bytes[dev] = smem;
  }
  return launch_k(ctx, kern, grid, dim3(32 * 10), smem, p);
}

static bool launch_qgemm_skg(tq_ctx* ctx, const tq_qweight* w, int n_groups, const __nv_bfloat16* x, size_t ldx, int mx, const int* counts,
                             const int* offsets, int max_rows, long long x_stride, long long y_stride, void* y, int y_dtype, size_t ldy,
                             const int* active, int max_active, size_t total_rows, int* status) {
  const int kc = w->n_kc, n_rb = w->n_rb / n_groups;
  if (kc < 8 || kc > 17 || n_rb < 1 || n_groups > 65535) return false;
  const int rows_bound = counts ? max_rows : mx;
  if (rows_bound < 1) return false;
  int gz = (rows_bound + 7) / 8;
  int gy = (active && max_active < n_groups) ? max_active : n_groups;
  // With the row counts on the device, a one-thread kernel first lists the (group, row chunk) jobs that exist, so
  // that the grid need not cover every chunk of every group (CTAs without a job cost a scheduling slot each): there
  // are at most (groups with rows) + (rows / 8) of them.
  bool listed = false;
  if (counts && total_rows > 0) {
    const long long bound = (long long)gy + (long long)(total_rows / 8);
    if (bound < (long long)gy * gz && bound <= kSkgJobs && bound <= 65535) {
      if (launch_k(ctx, skg_jobs_kernel, dim3(1), dim3(256), 0, counts, (active && max_active < n_groups) ? active : (const int*)nullptr, gy,
                   ctx->skg_jobs, (int)bound) != cudaSuccess) {
        *status = fail(ctx, TQ_ECUDA, "grouped persistent GEMM: job list launch failed");
        return true;
      }
      listed = true;
      gy = (int)bound;
      gz = 1;
    }
  }
  // CTAs per job: about two per SM over the jobs that are expected to have rows (mx is the caller's row chunk, about
  // twice the expected rows of a group, when the counts live on the device)
  const int est_chunks = listed ? 1 : counts ? (mx > 16 ? (mx / 2 + 7) / 8 : 1) : gz;
  long long est_jobs = (long long)gy * est_chunks;
  if (listed) est_jobs = (long long)((active && max_active < n_groups) ? max_active : n_groups) + (long long)(total_rows / 32);   // (the bound is loose)
  if (est_jobs < 1) est_jobs = 1;
  // (rounded down: with every slot of the GPU spoken for, a job or two more than estimated would put whole CTAs --
  // tens of microseconds each -- into a second wave)
  long long cps = 2LL * ctx->sm_count / est_jobs;
  const long long units = (long long)n_rb * kc;
  if (cps > 32) cps = 32;
  if (cps > units / 16) cps = units / 16;
  if (cps < 1) cps = 1;
  while (cps > 1 && cps * gy * gz > (long long)kGemvSets * kGemvMaxGrid * 2) cps >>= 1;   // one 128-word slot per CTA
  if (cps * gy * gz > (long long)kGemvSets * kGemvMaxGrid * 2 || gz > 65535 || gy > 65535) return false;
  const int tpw = kc >= 16 ? 2 : 1;
  const size_t stage = (size_t)8 * tpw * qk_tile_bytes(w->kind);
  const size_t fixed = (size_t)kSkwHeaderBytes + skw_red_bytes(8, 1) + (size_t)8 * skw_x_stride(kc) + skw_csum_bytes(w->kind, kc, 1);
  const size_t budget = 113 * 1024;
  if (fixed + 3 * stage > budget) return false;
  int stages = (int)((budget - fixed) / stage);
  if (stages > kSkMaxStages) stages = kSkMaxStages;
  QGroupParams p;
  p.tiles = w->tiles;
  p.row_scales = w->row_scales;
  p.x = x;
  p.y = y;
  p.ldx = (long long)ldx;
  p.ldy = (long long)ldy;
  p.n_rows = (int)(w->rows / n_groups);
  p.n_row_blocks = n_rb;
  p.kc_total = kc;
  p.mx = mx;
  p.y_bf16 = y_dtype == TQ_BF16;
  p.stages = stages;
  p.counts = counts;
  p.offsets = offsets;
  p.active = (active && max_active < n_groups) ? active : nullptr;
  p.jobs = listed ? ctx->skg_jobs : nullptr;
  p.x_stride = x_stride;
  p.y_stride = y_stride;
  p.ws = ctx->gemv_ws;
  p.err = ctx->dev_err;
  const size_t smem = fixed + (size_t)stages * stage;
  const dim3 grid((unsigned)cps, (unsigned)gy, (unsigned)gz);
  cudaError_t e;
  switch (w->kind) {
    case TQ_Q4_F32: e = tpw == 2 ? launch_skg_kernel<Q4_F32, 2>(ctx, p, grid, smem) : launch_skg_kernel<Q4_F32, 1>(ctx, p, grid, smem); break;
    case TQ_Q4_F16: e = tpw == 2 ? launch_skg_kernel<Q4_F16, 2>(ctx, p, grid, smem) : launch_skg_kernel<Q4_F16, 1>(ctx, p, grid, smem); break;
    case TQ_Q8_F32: e = tpw == 2 ? launch_skg_kernel<Q8_F32, 2>(ctx, p, grid, smem) : launch_skg_kernel<Q8_F32, 1>(ctx, p, grid, smem); break;
    default: e = tpw == 2 ? launch_skg_kernel<I8_ROW, 2>(ctx, p, grid, smem) : launch_skg_kernel<I8_ROW, 1>(ctx, p, grid, smem); break;
  }
  *status = e == cudaSuccess ? TQ_OK : fail(ctx, TQ_ECUDA, "grouped persistent GEMM launch failed: %s", cudaGetErrorString(e));
  return true;
}

int launch_qgemm_grouped(tq_ctx* ctx, const tq_qweight* w, int n_groups, const void* x_bf16, size_t ldx, int mx,
                         const int* counts, const int* offsets, int max_rows, long long x_stride, long long y_stride,
                         void* y, int y_dtype, size_t ldy, const int* active, int max_active, size_t total_rows) {
  TQ_REQUIRE(ctx, w && n_groups > 0 && w->rows % n_groups == 0 && (w->rows / n_groups) % kTileRows == 0,
             "grouped qlinear: rows per group must be a multiple of 16");
  TQ_REQUIRE(ctx, w->cols == (size_t)w->n_kc * kTileK && ldx % 8 == 0 && ((uintptr_t)x_bf16 & 15) == 0 && (x_stride % 8) == 0,
             "grouped qlinear: K must be a multiple of 128 and activation rows 16-byte aligned");
  {
    int st = TQ_OK;
    if (launch_qgemm_skg(ctx, w, n_groups, static_cast<const __nv_bfloat16*>(x_bf16), ldx, mx, counts, offsets, max_rows, x_stride, y_stride, y,
                         y_dtype, ldy, active, max_active, total_rows, &st))
      return st;
  }
  QgGroup g;
  g.n_groups = n_groups;
  g.counts = counts;
  g.offsets = offsets;
  g.x_stride = x_stride;
  g.y_stride = y_stride;
  g.max_rows = max_rows;
  g.active = active;
  g.max_active = max_active;
  return launch_qgemm(ctx, w, static_cast<const __nv_bfloat16*>(x_bf16), ldx, mx, 1, y, y_dtype, ldy, nullptr, &g);
}

bool umma_supported(const tq_qweight* w, size_t m);
struct UmmaGroups;
int launch_qgemm_umma(tq_ctx* ctx, const tq_qweight* w, const void* x_bf16, size_t ldx, size_t m, void* y, int y_dtype,
                      size_t ldy, int terms, const UmmaGroups* grp, bool swiglu = false);

// ---------------------------------------------------------------------------------------------
// Gate/up weights in the row order the fused SwiGLU epilogue wants: out row block b = gate rows 8b..8b+7 then up
// rows 8b..8b+7.  A half of a fragment tile (eight rows: its packed weights and its scales) is contiguous, so the
// regrouping is a copy of half-tiles; no number changes.
// ---------------------------------------------------------------------------------------------
__global__ void interleave_gate_up_kernel(const uint8_t* src, uint8_t* dst, int kind, int n_kc, int n_rb_out, int f_rows) {
  const int tile_bytes = qk_tile_bytes(kind), wb = qk_weight_bytes(kind), sb = qk_scale_bytes(kind);
  const size_t t = blockIdx.x;                      // (out row block, k chunk)
  const int rb = (int)(t / n_kc), kc = (int)(t % n_kc);
  if (rb >= n_rb_out) return;
  uint8_t* out = dst + t * tile_bytes;
  for (int h = 0; h < 2; ++h) {
    const int src_row = (h == 0 ? 0 : f_rows) + 8 * rb;                 // first of the eight source rows
    const int srb = src_row / 16, sh = (src_row / 8) & 1;
    const uint8_t* in = src + ((size_t)srb * n_kc + kc) * tile_bytes;
    for (int i = threadIdx.x * 16; i < wb / 2; i += blockDim.x * 16)
      *reinterpret_cast<uint4*>(out + h * (wb / 2) + i) = *reinterpret_cast<const uint4*>(in + sh * (wb / 2) + i);
    for (int i = threadIdx.x * 16; i < sb / 2; i += blockDim.x * 16)
      *reinterpret_cast<uint4*>(out + wb + h * (sb / 2) + i) = *reinterpret_cast<const uint4*>(in + wb + sh * (sb / 2) + i);
  }
}

// silu(gate) * up over a projection output in the interleaved order: gu [rows][2n] f32, out [rows][n].
__global__ void swiglu_interleaved_kernel(const float* gu, size_t rows, size_t n, void* out, int out_dt) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * n) return;
  const size_t row = idx / n, i = idx % n;
  const size_t src = row * 2 * n + (i / 8) * 16 + (i % 8);
  const float g = gu[src], u = gu[src + 8];
  const float v = g * (1.0f / (1.0f + expf(-g))) * u;
  if (out_dt == TQ_BF16) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else static_cast<float*>(out)[idx] = v;
}

// Activation rows from which the tcgen05 kernel takes over from the mma.sync kernel.
// Rows from which the tcgen05 kernel takes over from the mma.sync kernel (Llama-3-8B decode step, 32 layers, f32
// outputs: 4.87 against 4.98 ms at 16 rows, 5.63 against 5.30 ms at 20, 6.10 against 5.50 ms at 24).
static int umma_min_m(int y_dtype) {
  (void)y_dtype;
  return 17;
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
  w->n_rb = (int)((rows + kTileRows - 1) / kTileRows);
  w->n_kc = (int)((cols + kTileK - 1) / kTileK);
  w->tile_bytes = (size_t)w->n_rb * w->n_kc * qk_tile_bytes(kind);
  cudaError_t e = cudaMalloc(&w->tiles, w->tile_bytes);
  if (e == cudaSuccess && kind == TQ_I8_ROW) e = cudaMalloc(&w->row_scales, rows * sizeof(float));
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (w->tiles) cudaFree(w->tiles);
    delete w;
    return fail(ctx, e == cudaErrorMemoryAllocation ? TQ_ENOMEM : TQ_ECUDA, "weight allocation failed: %s",
                cudaGetErrorString(e));
  }
  *out = w;
  return TQ_OK;
}

// ---------------------------------------------------------------------------------------------
// quantize_q4 / quantize_q8 of tang-infer (crates/tang-infer/src/quantize.rs:47-71, 84-118) on the device,
// row by row as quantize_matrix_q4/q8 do (:193-220).  One warp per (row, 32-block), one lane per value:
// amax = max |v| (NaN ignored, as f32::max does), scale = amax / 7 (or / 127), 1.0 for an all-zero block,
// q = round(v * (1 / scale)) with ties away from zero, clamped; a ragged tail is padded with q = 0.
// Every operation is a correctly rounded f32 operation with no fusing, so codes and scales are the reference's
// bit for bit.  Writes the plain structure-of-arrays form the repack reads.
// ---------------------------------------------------------------------------------------------
__global__ void quantize_rows_kernel(const void* src, int src_dtype, size_t ld, size_t rows, size_t cols, int is4,
                                     uint8_t* pay, float* scales) {
  const size_t bpr = (cols + 31) / 32;
  const size_t blk = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (blk >= rows * bpr) return;
  const int lane = threadIdx.x & 31;
  const size_t row = blk / bpr, b = blk - row * bpr, k = b * 32 + lane;
  float v = 0.f;
  const bool live = k < cols;
  if (live) {
    if (src_dtype == TQ_F32) v = static_cast<const float*>(src)[row * ld + k];
    else if (src_dtype == TQ_BF16) v = __bfloat162float(static_cast<const __nv_bfloat16*>(src)[row * ld + k]);
    else v = __half2float(static_cast<const __half*>(src)[row * ld + k]);
  }
  float amax = live ? fabsf(v) : 0.f;
  if (!(amax == amax)) amax = 0.f;                       // f32::max(acc, NaN) keeps acc
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax == 0.f ? 1.0f : __fdiv_rn(amax, is4 ? 7.0f : 127.0f);
  const float inv = __fdiv_rn(1.0f, scale);
  const float pr = __fmul_rn(v, inv);                    // NaN for a NaN weight, and for inf * 0 in a block with an infinity
  float q = roundf(pr);                                  // ties away from zero, like f32::round
  q = fminf(fmaxf(q, is4 ? -8.0f : -128.0f), is4 ? 7.0f : 127.0f);
  // Rust's `NaN.round().clamp(..) as i8` is 0; fminf/fmaxf would have turned the NaN into a bound, so test the product
  int qi = (live && pr == pr) ? (int)q : 0;
  if (is4) {
    const int hi = __shfl_down_sync(0xffffffffu, qi, 1);
    if ((lane & 1) == 0) pay[blk * 16 + (lane >> 1)] = (uint8_t)((qi + 8) | ((hi + 8) << 4));
  } else {
    pay[blk * 32 + lane] = (uint8_t)(int8_t)qi;
  }
  if (lane == 0) scales[blk] = scale;
}

// Input strides of the plain arrays for a given kind.
static void plain_strides(int kind, size_t cols, size_t* ld_pay, size_t* ld_sc) {
  const size_t bpr = (cols + 31) / 32;
  *ld_pay = kind == TQ_I8_ROW ? cols : is_q4(kind) ? bpr * 16 : bpr * 32;
  *ld_sc = kind == TQ_I8_ROW ? 0 : bpr * scale_elem(kind);
}

// Repacks plain device arrays into w->tiles.
static int repack_from_device(tq_ctx* ctx, tq_qweight* w, const uint8_t* pay, const uint8_t* sc) {
  size_t ld_pay, ld_sc;
  plain_strides(w->kind, w->cols, &ld_pay, &ld_sc);
  const size_t n = (size_t)w->n_rb * w->n_kc * 256;
  repack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(pay, sc, ld_pay, ld_sc, w->kind, w->rows, w->cols,
                                                                     w->n_rb, w->n_kc, w->tiles);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  if (w->kind == TQ_I8_ROW)
    TQ_CUDA(ctx, cudaMemcpyAsync(w->row_scales, sc, w->rows * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
  return TQ_OK;
}

extern "C" {

int tq_qweight_from_device_arrays(tq_ctx* ctx, int kind, const void* payload_dev, const void* scales_dev, size_t rows,
                                  size_t cols, tq_qweight** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, payload_dev && scales_dev, "tq_qweight_from_device_arrays: null array");
  TQ_REQUIRE(ctx, ((uintptr_t)payload_dev & 7) == 0 && ((uintptr_t)scales_dev & 3) == 0,
             "tq_qweight_from_device_arrays: payload must be 8-byte and scales 4-byte aligned");
  TQ_REQUIRE(ctx, kind == TQ_I8_ROW || kind == TQ_Q4_F32 || kind == TQ_Q8_F32 || ((cols + 31) / 32) % 2 == 0 || rows == 1,
             "tq_qweight_from_device_arrays: f16 scale rows must stay 4-byte aligned (even block count)");
  tq_qweight* w = nullptr;
  if (int st = make_weight(ctx, kind, rows, cols, &w)) return st;
  if (int st = repack_from_device(ctx, w, static_cast<const uint8_t*>(payload_dev), static_cast<const uint8_t*>(scales_dev))) {
    tq_qweight_free(ctx, w);
    return st;
  }
  *out = w;
  return TQ_OK;
}

int tq_quantize_matrix(tq_ctx* ctx, const void* src_dev, int src_dtype, size_t ld, size_t rows, size_t cols, int kind,
                       tq_qweight** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, out != nullptr, "null output handle");
  *out = nullptr;
  TQ_REQUIRE(ctx, kind == TQ_Q4_F32 || kind == TQ_Q8_F32, "tq_quantize_matrix: kind must be TQ_Q4_F32 or TQ_Q8_F32 (the reference's block formats)");
  TQ_REQUIRE(ctx, src_dtype == TQ_F32 || src_dtype == TQ_BF16 || src_dtype == TQ_F16, "tq_quantize_matrix: source must be f32, bf16 or f16");
  TQ_REQUIRE(ctx, src_dev && rows > 0 && cols > 0, "tq_quantize_matrix: null source or empty matrix");
  if (ld == 0) ld = cols;
  TQ_REQUIRE(ctx, ld >= cols, "tq_quantize_matrix: row stride smaller than the row");
  size_t ld_pay, ld_sc;
  plain_strides(kind, cols, &ld_pay, &ld_sc);
  uint8_t* pay = nullptr;
  float* sc = nullptr;
  cudaError_t e = cudaMalloc(&pay, rows * ld_pay + 16);
  if (e == cudaSuccess) e = cudaMalloc(&sc, rows * ld_sc + 16);
  int st = TQ_OK;
  tq_qweight* w = nullptr;
  if (e != cudaSuccess) st = fail(ctx, e == cudaErrorMemoryAllocation ? TQ_ENOMEM : TQ_ECUDA, "tq_quantize_matrix: %s", cudaGetErrorString(e));
  if (st == TQ_OK) st = make_weight(ctx, kind, rows, cols, &w);
  if (st == TQ_OK) {
    const size_t n_blocks = rows * ((cols + 31) / 32);
    quantize_rows_kernel<<<(unsigned)((n_blocks + 7) / 8), 256, 0, ctx->stream>>>(src_dev, src_dtype, ld, rows, cols, is_q4(kind) ? 1 : 0,
                                                                                pay, sc);
    ctx->launches++;
    if (cudaGetLastError() != cudaSuccess) st = fail(ctx, TQ_ECUDA, "tq_quantize_matrix: launch failed");
  }
  if (st == TQ_OK) st = repack_from_device(ctx, w, pay, reinterpret_cast<const uint8_t*>(sc));
  if (cudaStreamSynchronize(ctx->stream) != cudaSuccess && st == TQ_OK) st = fail(ctx, TQ_ECUDA, "tq_quantize_matrix: failed");
  if (pay) cudaFree(pay);
  if (sc) cudaFree(sc);
  if (st != TQ_OK) {
    if (w) tq_qweight_free(ctx, w);
    cudaGetLastError();
    return st;
  }
  *out = w;
  return TQ_OK;
}

int tq_qweight_from_arrays(tq_ctx* ctx, int kind, const void* payload_host, const void* scales_host, size_t rows,
                           size_t cols, tq_qweight** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, out != nullptr, "null output handle");
  *out = nullptr;
  TQ_REQUIRE(ctx, payload_host && scales_host, "tq_qweight_from_arrays: null array");
  TQ_REQUIRE(ctx, kind >= TQ_Q4_F32 && kind <= TQ_I8_ROW, "unknown weight kind %d", kind);
  TQ_REQUIRE(ctx, rows > 0 && cols > 0, "empty weight matrix");
  size_t ld_pay, ld_sc;
  plain_strides(kind, cols, &ld_pay, &ld_sc);
  const size_t pay_bytes = rows * ld_pay, sc_bytes = kind == TQ_I8_ROW ? rows * 4 : rows * ld_sc;
  uint8_t *dpay = nullptr, *dsc = nullptr;
  cudaError_t e = cudaMalloc(&dpay, pay_bytes + 16);
  if (e == cudaSuccess) e = cudaMalloc(&dsc, sc_bytes + 16);
  if (e == cudaSuccess) e = cudaMemcpyAsync(dpay, payload_host, pay_bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(dsc, scales_host, sc_bytes, cudaMemcpyHostToDevice, ctx->stream);
  int st = TQ_OK;
  tq_qweight* w = nullptr;
  if (e != cudaSuccess) st = fail(ctx, TQ_ECUDA, "tq_qweight_from_arrays: %s", cudaGetErrorString(e));
  if (st == TQ_OK) st = make_weight(ctx, kind, rows, cols, &w);
  if (st == TQ_OK) st = repack_from_device(ctx, w, dpay, dsc);
  if (st == TQ_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) st = fail(ctx, TQ_ECUDA, "repack failed");
  else cudaStreamSynchronize(ctx->stream);
  if (dpay) cudaFree(dpay);
  if (dsc) cudaFree(dsc);
  if (st != TQ_OK) {
    if (w) tq_qweight_free(ctx, w);
    cudaGetLastError();
    return st;
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

int tq_qweight_free(tq_ctx* ctx, tq_qweight* w) {
  if (!w) return TQ_OK;
  if (int st = bind(ctx)) return st;
  cudaStreamSynchronize(ctx->stream);
  if (w->tiles) cudaFree(w->tiles);
  if (w->row_scales) cudaFree(w->row_scales);
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
  const size_t n = w->rows * (size_t)w->n_kc * 16;
  dequantize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(w->tiles, w->row_scales, w->kind, w->rows,
                                                                         w->cols, w->n_kc, out_dev, ints_dev);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
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
  const size_t kx = (size_t)w->n_kc * kTileK;  // the kernel consumes whole 128-k chunks
  const bool direct = x_dtype == TQ_BF16 && w->cols == kx && ldx % 8 == 0 && ((uintptr_t)x_dev & 15) == 0;
  if (!direct) {
    const size_t rows_staged = (m < chunk ? m : chunk) * combine;
    if (int st = ensure_xprep(ctx, rows_staged * kx * 2)) return st;
  }
  if (direct && !residual_dev && m >= (size_t)umma_min_m(y_dtype) && umma_supported(w, m))
    return launch_qgemm_umma(ctx, w, x_dev, ldx, m, y_dev, y_dtype, ldy, y_dtype == TQ_F32 ? 2 : 1, nullptr);
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
      const size_t n = mc * kx;
      prep_x_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(xc, x_dtype, ldx, mc, w->cols, kx,
                                                                         static_cast<__nv_bfloat16*>(ctx->xprep));
      ctx->launches++;
      TQ_CUDA(ctx, cudaGetLastError());
      xs = static_cast<const __nv_bfloat16*>(ctx->xprep);
      ldxs = kx;
    }
    if (int st = launch_qgemm(ctx, w, xs, ldxs, (int)(mc * combine), combine, yc, y_dtype, ldy, rc)) return st;
  }
  return TQ_OK;
}

}  // extern "C"

// Stages the activations of a host-vector matvec: x (bf16 or f32, in PINNED host memory, read through its device
// alias) -> bf16 rows of kx elements in a ring slot, zero beyond `cols`; f32 values as three bf16 terms (rows 3r, 3r+1,
// 3r+2, as prep_x_kernel).  It waits for nothing until its last instruction, so it runs beside whatever is in flight;
// the GEMV that consumes the slot looks at the tag word instead of waiting for this kernel to finish.
__global__ void __launch_bounds__(256) stage_host_x_kernel(const void* x, int dtype, size_t m, size_t cols, size_t kx,
                                                           __nv_bfloat16* slot, unsigned* tag, unsigned seq, const unsigned* epoch) {
  pdl_launch_dependents();
  // Every load below crosses the bus: 16 bytes per load, all of a thread's loads issued before any is used.
  if (dtype == TQ_BF16 && cols == kx && ((uintptr_t)x & 15) == 0) {
    const size_t n16 = m * kx / 8;
    const uint4* src = static_cast<const uint4*>(x);
    uint4* dst = reinterpret_cast<uint4*>(slot);
    for (size_t i0 = threadIdx.x; i0 < n16; i0 += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * blockDim.x < n16) v[u] = src[i0 + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * blockDim.x < n16) dst[i0 + u * blockDim.x] = v[u];
    }
  } else if (dtype == TQ_F32 && cols == kx && ((uintptr_t)x & 15) == 0) {
    const size_t n4 = m * kx / 4;
    const float4* src = static_cast<const float4*>(x);
    for (size_t i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * blockDim.x < n4) v[u] = src[i0 + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t i = i0 + u * blockDim.x;
        if (i >= n4) continue;
        const size_t row = (4 * i) / kx, col = (4 * i) % kx;
        const float f[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat16 hi = __float2bfloat16_rn(f[e]);
          const float r1 = f[e] - __bfloat162float(hi);
          const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
          slot[(3 * row + 0) * kx + col + e] = hi;
          slot[(3 * row + 1) * kx + col + e] = mid;
          slot[(3 * row + 2) * kx + col + e] = __float2bfloat16_rn(r1 - __bfloat162float(mid));
        }
      }
    }
  } else
  for (size_t idx = threadIdx.x; idx < m * kx; idx += blockDim.x) {
    const size_t row = idx / kx, col = idx % kx;
    if (dtype == TQ_BF16) {
      slot[row * kx + col] = col < cols ? static_cast<const __nv_bfloat16*>(x)[row * cols + col] : __float2bfloat16_rn(0.f);
    } else {
      const float v = col < cols ? static_cast<const float*>(x)[row * cols + col] : 0.f;
      const __nv_bfloat16 hi = __float2bfloat16_rn(v);
      const float r1 = v - __bfloat162float(hi);
      const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
      slot[(3 * row + 0) * kx + col] = hi;
      slot[(3 * row + 1) * kx + col] = mid;
      slot[(3 * row + 2) * kx + col] = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(tag), "r"(sk_x_tag_value(seq, epoch)) : "memory");
  pdl_wait();   // kernels of a stream still complete in launch order
}

static void* pinned_alias(const void* host) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer) return attr.devicePointer;
  cudaGetLastError();   // an unregistered pointer is not an error here
  return nullptr;
}

// Host vectors in pinned memory, bf16 or f32, up to eight staged rows: no copy is queued on the stream at all.  A
// one-CTA kernel pulls x over the bus into a ring slot, the persistent GEMV stores y straight into the pinned result,
// and consecutive calls overlap on the GPU like any other run of independent GEMVs.  Returns false when the call
// does not qualify (the caller then takes the copying path).
// First staging call of a captured graph: one thread advances the replay count.  It lets nothing start early, so every
// kernel recorded after it starts after it has finished.
__global__ void hostx_epoch_kernel(unsigned* epoch) { *epoch = *epoch + 1; }

static bool matvec_host_pinned(tq_ctx* ctx, const tq_qweight* w, const void* x_host, void* y_host, int dtype, size_t m, int* status) {
  if (dtype == TQ_F64 || !ctx->owns_stream || !ctx->pdl) return false;
  const int combine = dtype == TQ_F32 ? 3 : 1;
  const size_t mx = m * combine, kx = (size_t)w->n_kc * kTileK;
  if (mx > 8 || mx * kx * 2 > kHostXSlotBytes) return false;
  void* xa = pinned_alias(x_host);
  void* ya = xa ? pinned_alias(y_host) : nullptr;
  if (!xa || !ya) return false;
  if (!ctx->hostx_ring) {
    if (ctx->capturing) return false;   // (no allocation inside a capture: one eager call first sets the ring up)
    if (cudaMalloc(&ctx->hostx_ring, (size_t)kHostXSlots * kHostXSlotBytes) != cudaSuccess ||
        cudaMalloc(&ctx->hostx_tags, (kHostXSlots + 1) * sizeof(unsigned)) != cudaSuccess ||
        cudaMemsetAsync(ctx->hostx_tags, 0, (kHostXSlots + 1) * sizeof(unsigned), ctx->stream) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    ctx->hostx_epoch = ctx->hostx_tags + kHostXSlots;
  }
  const unsigned* epoch = nullptr;
  if (ctx->capturing) {
    // A replay runs the same launches with the same sequence numbers: the tags carry the replay count as well.
    epoch = ctx->hostx_epoch;
    if (ctx->hostx_epoch_pending) {
      if (launch_k(ctx, hostx_epoch_kernel, dim3(1), dim3(1), 0, ctx->hostx_epoch) != cudaSuccess) {
        *status = fail(ctx, TQ_ECUDA, "tq_q_matvec_host: launch failed");
        return true;
      }
      ctx->hostx_epoch_pending = false;
    }
  }
  const unsigned seq = ++ctx->hostx_seq;                 // never 0: a zeroed tag matches nothing
  const unsigned slot = seq % kHostXSlots;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ctx->hostx_ring + (size_t)slot * kHostXSlotBytes);
  if (launch_k_independent(ctx, stage_host_x_kernel, dim3(1), dim3(256), 0, (const void*)xa, dtype, m, w->cols, kx, xs, ctx->hostx_tags + slot,
                           seq, epoch) != cudaSuccess) {
    *status = fail(ctx, TQ_ECUDA, "tq_q_matvec_host: staging kernel launch failed");
    return true;
  }
  if (!launch_qgemv_sk(ctx, w, xs, kx, (int)mx, combine, ya, dtype == TQ_BF16 ? TQ_BF16 : TQ_F32, w->rows, nullptr, status, nullptr, false,
                       ctx->hostx_tags + slot, seq, epoch))
    return false;   // (the staged slot is simply not used)
  return true;
}

// The host-vector call; `wait` = return only when y_host holds the result.
static int matvec_host(tq_ctx* ctx, const tq_qweight* w, const void* x_host, void* y_host, int dtype, size_t m, bool wait) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, w != nullptr, "tq_q_matvec_host: null weight");
  TQ_REQUIRE(ctx, dtype == TQ_F64 || dtype == TQ_F32 || dtype == TQ_BF16, "tq_q_matvec_host: dtype must be f64, f32 or bf16");
  if (m == 0) return TQ_OK;
  TQ_REQUIRE(ctx, x_host && y_host, "tq_q_matvec_host: null vector");
  {
    int st = TQ_OK;
    if (matvec_host_pinned(ctx, w, x_host, y_host, dtype, m, &st)) return st != TQ_OK ? st : (wait ? tq_sync(ctx) : TQ_OK);
  }
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
  if (dtype != TQ_F64) {
    // A pinned result vector is visible to the device: the kernel stores y straight into it (posted writes over
    // the bus) and the separate device-to-host copy disappears.  x is still copied once: every CTA reads all of it.
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, y_host) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer) {
      if (int st = tq_qlinear(ctx, w, xd, dev_dt, 0, m, attr.devicePointer, dev_dt, 0, nullptr)) return st;
      return wait ? tq_sync(ctx) : TQ_OK;
    }
    cudaGetLastError();   // an unregistered pointer is not an error here
  }
  if (int st = tq_qlinear(ctx, w, xd, dev_dt, 0, m, s + off_y, dev_dt, 0, nullptr)) return st;
  const void* yd = s + off_y;
  if (dtype == TQ_F64) {
    if (int st = tq_convert(ctx, s + off_y, TQ_F32, s + off_y2, TQ_F64, ny)) return st;
    yd = s + off_y2;
  }
  TQ_CUDA(ctx, cudaMemcpyAsync(y_host, yd, ny * es, cudaMemcpyDeviceToHost, ctx->stream));
  return wait ? tq_sync(ctx) : TQ_OK;
}

extern "C" {

int tq_q_matvec_host(tq_ctx* ctx, const tq_qweight* w, const void* x_host, void* y_host, int dtype, size_t m) {
  return matvec_host(ctx, w, x_host, y_host, dtype, m, true);
}

int tq_q_matvec_host_async(tq_ctx* ctx, const tq_qweight* w, const void* x_host, void* y_host, int dtype, size_t m) {
  return matvec_host(ctx, w, x_host, y_host, dtype, m, false);
}

}  // extern "C"


namespace tq {

int launch_swiglu_interleaved(tq_ctx* ctx, const float* gu, size_t rows, size_t n, void* out, int out_dtype) {
  TQ_CUDA(ctx, launch_k(ctx, swiglu_interleaved_kernel, dim3((unsigned)((rows * n + 255) / 256)), dim3(256), 0, gu, rows, n, out, out_dtype));
  return TQ_OK;
}

int qlinear_fused(tq_ctx* ctx, const tq_qweight* w, const void* x_bf16, const QlinearNorm* norm, size_t m, void* y, int y_dtype,
                  size_t ldy, bool swiglu, float* gu_tmp) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, w && y && (norm || x_bf16), "fused linear: null argument");
  TQ_REQUIRE(ctx, !swiglu || w->gate_up_interleaved, "fused linear: the SwiGLU epilogue needs a weight from tq_qweight_interleave_gate_up");
  if (m == 0) return TQ_OK;
  const size_t cols = w->cols;
  if (m <= 8 && w->cols == (size_t)w->n_kc * kTileK) {
    int st = TQ_OK;
    if (launch_qgemv_sk(ctx, w, static_cast<const __nv_bfloat16*>(x_bf16), cols, (int)m, 1, y, y_dtype, ldy, nullptr, &st, norm, swiglu))
      return st;
  }
  // the separate operators
  const void* xin = x_bf16;
  if (norm) {
    TQ_REQUIRE(ctx, norm->xn_tmp != nullptr, "fused linear: no buffer for the normalised rows");
    if (int st = tq_rms_norm(ctx, norm->delta ? (const void*)norm->delta : (const void*)norm->h, TQ_F32, norm->delta ? norm->h : nullptr,
                             norm->gain_bf16, TQ_BF16, m, cols, norm->eps, norm->xn_tmp, TQ_BF16, norm->h_out))
      return st;
    xin = norm->xn_tmp;
  }
  if (!swiglu) return tq_qlinear(ctx, w, xin, TQ_BF16, cols, m, y, y_dtype, ldy, nullptr);
  // many rows: the tcgen05 kernel applies silu(gate) * up to its f32 sums itself.  As for every projection, the
  // result type decides the operand terms: exact products (two terms) for f32 results, the product rounded once to
  // bf16 (at most 2^-8 relative, half a step of the result type) for bf16 results.
  if (m >= (size_t)umma_min_m(TQ_F32) && umma_supported(w, m) && w->cols == (size_t)w->n_kc * kTileK && ((uintptr_t)xin & 15) == 0)
    return launch_qgemm_umma(ctx, w, xin, cols, m, y, y_dtype, ldy, y_dtype == TQ_F32 ? 2 : 1, nullptr, true);
  TQ_REQUIRE(ctx, gu_tmp != nullptr, "fused linear: no buffer for the gate/up projection");
  if (int st = tq_qlinear(ctx, w, xin, TQ_BF16, cols, m, gu_tmp, TQ_F32, w->rows, nullptr)) return st;
  const size_t n = w->rows / 2;
  TQ_REQUIRE(ctx, ldy == n, "fused linear: the SwiGLU output must be dense");
  return launch_swiglu_interleaved(ctx, gu_tmp, m, n, y, y_dtype);
}

}  // namespace tq

extern "C" int tq_qweight_interleave_gate_up(tq_ctx* ctx, const tq_qweight* w_gate_up, tq_qweight** out) {
  if (int st = tq::bind(ctx)) return st;
  TQ_REQUIRE(ctx, w_gate_up && out, "tq_qweight_interleave_gate_up: null argument");
  *out = nullptr;
  TQ_REQUIRE(ctx, !w_gate_up->gate_up_interleaved, "tq_qweight_interleave_gate_up: the weight is interleaved already");
  TQ_REQUIRE(ctx, w_gate_up->rows % 32 == 0, "tq_qweight_interleave_gate_up: gate and up need a multiple of 16 rows each");
  tq_qweight* w = new (std::nothrow) tq_qweight();
  if (!w) return tq::fail(ctx, TQ_ENOMEM, "out of host memory");
  *w = *w_gate_up;
  w->tiles = nullptr;
  w->row_scales = nullptr;
  w->gate_up_interleaved = true;
  cudaError_t e = cudaMalloc(&w->tiles, w->tile_bytes);
  if (e == cudaSuccess && w->kind == TQ_I8_ROW) e = cudaMalloc(&w->row_scales, w->rows * sizeof(float));
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (w->tiles) cudaFree(w->tiles);
    delete w;
    return tq::fail(ctx, TQ_ENOMEM, "tq_qweight_interleave_gate_up: allocation failed");
  }
  const int f = (int)(w->rows / 2);
  tq::interleave_gate_up_kernel<<<(unsigned)((size_t)w->n_rb * w->n_kc), 64, 0, ctx->stream>>>(w_gate_up->tiles, w->tiles, w->kind, w->n_kc,
                                                                                       w->n_rb, f);
  ctx->launches++;
  e = cudaGetLastError();
  if (e == cudaSuccess && w->kind == TQ_I8_ROW) {
    // row scales follow their rows: out row 16b + i (i < 8) is gate row 8b + i, out row 16b + 8 + i is up row 8b + i
    for (int b = 0; b < w->n_rb && e == cudaSuccess; ++b) {
      e = cudaMemcpyAsync(w->row_scales + 16 * (size_t)b, w_gate_up->row_scales + 8 * (size_t)b, 8 * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(w->row_scales + 16 * (size_t)b + 8, w_gate_up->row_scales + f + 8 * (size_t)b, 8 * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream);
    }
  }
  if (e != cudaSuccess) {
    tq_qweight_free(ctx, w);
    return tq::fail(ctx, TQ_ECUDA, "tq_qweight_interleave_gate_up: %s", cudaGetErrorString(e));
  }
  *out = w;
  return TQ_OK;
}
