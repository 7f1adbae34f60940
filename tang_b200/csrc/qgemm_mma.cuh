// Weight-only quantised linear layer for 1..64 activation rows (decode):
//     y[m, n] = sum_k x[m, k] * q[n, k] * scale[n, k/32]
// restating crates/tang-infer/src/quantize.rs:227-289 (q8_matvec / q4_matvec) for the GPU.
//
// The kernel is bound by the HBM stream of the packed weights, so everything is arranged
// around that stream:
//   * one producer warp per CTA moves [R rows x KB k] weight tiles and the matching activation
//     chunk into shared memory with 1-D bulk (TMA) copies through an S-stage mbarrier ring;
//     weights carry an L2 evict-first hint, activations evict-last;
//   * WR x WK consumer warps each own 16 output rows and one 128-wide K slice of the stage.
//     A lane reads its eight 4-bit (or 8-bit) weights of a 32-block as ONE 32-bit word (two for
//     int8), turns them into exact bf16 integers in registers and feeds mma.sync m16n8k16; the
//     32-block's scale multiplies the f32 partial sum afterwards, so integer unpack and products
//     are exact and only the f32 accumulation rounds;
//   * the K permutation inside a 32-block that the register dequantiser produces is undone on the
//     activation side with two byte-permutes per MMA, so weights stay in tang-infer's nibble order;
//   * the WK partial sums of a row meet in shared memory (split-K inside the CTA).
// f32 activations are supported by the caller splitting every value into three bf16 terms
// (exactly) and asking for combine=3: three adjacent token columns are summed in the epilogue.
#pragma once

#include "common.cuh"

namespace tq {

enum QKind : int { Q4_F32 = 0, Q4_F16 = 1, Q8_F32 = 2, I8_ROW = 3 };

constexpr int kWarpK = 128;   // k handled by one consumer warp per stage (four 32-blocks)

struct QGemmParams {
  const uint8_t* payload;   // [n_rows][ldw] bytes
  const uint8_t* scales;    // [n_rows][lds] bytes (I8_ROW: one f32 per row, lds = 4)
  const __nv_bfloat16* x;   // [mx][ldx] bf16, rows 16-byte aligned, zero beyond the true K
  void* y;                  // [m_out][ldy] f32 or bf16
  const float* residual;    // optional f32 [m_out][ldy] added before the store (may alias y)
  long long ldw, lds, ldx, ldy;
  int n_rows;               // output features
  int kpad;                 // K rounded up to a multiple of 32
  int mx;                   // activation rows present in x (<= 8*NT)
  int m_out;                // rows of y = mx / combine
  int combine;              // 1, or 3 for split-f32 activations
  int y_bf16;               // 0: f32 output, 1: bf16 output
  int wr, wk, stages;       // consumer grid inside the CTA and ring depth
  int* err;
};

__host__ __device__ inline int qg_rows_per_cta(int wr) { return 16 * wr; }
__host__ __device__ inline int qg_stage_k(int wk) { return kWarpK * wk; }
// Shared-memory row strides.  Padding keeps the 8 row groups of a warp on different banks:
// 4-byte weight reads want stride = 16 (mod 128), 8-byte reads 32 (mod 128), the 16-byte
// activation reads 64 (mod 128).
__host__ __device__ inline int qg_w_stride(int kind, int wk) {
  return (kind == Q8_F32 || kind == I8_ROW) ? qg_stage_k(wk) + 32 : qg_stage_k(wk) / 2 + 16;
}
__host__ __device__ inline int qg_x_stride(int wk) { return qg_stage_k(wk) * 2 + 64; }
__host__ __device__ inline int qg_scale_elem(int kind) { return kind == Q4_F16 ? 2 : 4; }
__host__ __device__ inline int qg_scale_stride(int kind, int kpad) {
  if (kind == I8_ROW) return 16;
  int bytes = (kpad / 32) * qg_scale_elem(kind);
  int s = (bytes + 127) / 128 * 128 + 16;
  return s;
}
__host__ __device__ inline int qg_stage_bytes(int kind, int wr, int wk, int mx) {
  return qg_rows_per_cta(wr) * qg_w_stride(kind, wk) + mx * qg_x_stride(wk);
}
__host__ __device__ inline int qg_epilogue_bytes(int wr, int wk, int nt) {
  return wk * 8 * nt * (qg_rows_per_cta(wr) + 4) * 4;
}
constexpr int kQgHeaderBytes = 256;  // barriers + failure flag
__host__ __device__ inline size_t qg_smem_bytes(int kind, int nt, int wr, int wk, int stages, int mx, int kpad) {
  size_t pipe = (size_t)stages * qg_stage_bytes(kind, wr, wk, mx);
  size_t epi = (size_t)qg_epilogue_bytes(wr, wk, nt);
  size_t body = pipe > epi ? pipe : epi;
  return kQgHeaderBytes + (size_t)qg_rows_per_cta(wr) * qg_scale_stride(kind, kpad) + body;
}

template <int KIND, int NT>
__global__ void __launch_bounds__(288) qgemm_mma_kernel(const QGemmParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool kIs8 = (KIND == Q8_F32 || KIND == I8_ROW);
  constexpr int kMaxStages = 8;

  const int WR = p.wr, WK = p.wk, S = p.stages;
  const int R = qg_rows_per_cta(WR);
  const int KB = qg_stage_k(WK);
  const int w_stride = qg_w_stride(KIND, WK);
  const int x_stride = qg_x_stride(WK);
  const int sc_stride = qg_scale_stride(KIND, p.kpad);
  const int stage_bytes = qg_stage_bytes(KIND, WR, WK, p.mx);

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* scale_bar = empty_bar + kMaxStages;
  volatile int* failed = reinterpret_cast<volatile int*>(scale_bar + 1);
  uint8_t* sc_smem = smem + kQgHeaderBytes;
  uint8_t* body = sc_smem + (size_t)R * sc_stride;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_consumers = WR * WK;
  const int row0 = blockIdx.x * R;
  const int rows_valid = min(R, p.n_rows - row0);
  const int n_iters = (p.kpad + KB - 1) / KB;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], n_consumers);
    }
    mbar_init(scale_bar, 1);
    *failed = 0;
    mbar_init_fence();
  }
  __syncthreads();

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;

  if (warp == n_consumers) {
    // ------------------------------------------------------------------ producer warp
    const uint64_t pol_w = l2_policy_evict_first();
    const uint64_t pol_x = l2_policy_evict_last();
    {  // scale rows of this CTA, whole K, once
      const uint32_t row_bytes = (KIND == I8_ROW) ? 0u : (uint32_t)((p.kpad / 32) * qg_scale_elem(KIND));
      if constexpr (KIND != I8_ROW) {
        // bulk copies need a multiple of 16 bytes; the packer pads scale rows to 16 bytes
        const uint32_t copy_bytes = (row_bytes + 15u) & ~15u;
        if (lane == 0) mbar_arrive_expect_tx(scale_bar, copy_bytes * (uint32_t)rows_valid);
        __syncwarp();
        for (int r = lane; r < rows_valid; r += 32)
          bulk_g2s(sc_smem + (size_t)r * sc_stride, p.scales + (size_t)(row0 + r) * p.lds, copy_bytes, scale_bar,
                   pol_x);
      } else {
        if (lane == 0) mbar_arrive(scale_bar);
      }
    }
    for (int it = 0; it < n_iters; ++it) {
      const int s = it % S;
      const uint32_t ph = (uint32_t)(it / S) & 1u;
      if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, failed, p.err, DERR_EMPTY_WAIT)) break;
      const int k0 = it * KB;
      const int kv = min(KB, p.kpad - k0);
      const uint32_t wbytes = kIs8 ? (uint32_t)kv : (uint32_t)(kv / 2);
      const uint32_t xbytes = (uint32_t)kv * 2u;
      uint8_t* st = body + (size_t)s * stage_bytes;
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[s], wbytes * (uint32_t)rows_valid + xbytes * (uint32_t)p.mx);
      __syncwarp();
      const size_t koff = kIs8 ? (size_t)k0 : (size_t)(k0 / 2);
      for (int r = lane; r < rows_valid; r += 32)
        bulk_g2s(st + (size_t)r * w_stride, p.payload + (size_t)(row0 + r) * p.ldw + koff, wbytes, &full_bar[s], pol_w);
      uint8_t* xs = st + (size_t)R * w_stride;
      for (int m = lane; m < p.mx; m += 32)
        bulk_g2s(xs + (size_t)m * x_stride, p.x + (size_t)m * p.ldx + k0, xbytes, &full_bar[s], pol_x);
    }
  } else if (warp < n_consumers) {
    // ------------------------------------------------------------------ consumer warps
    const int wr_i = warp / WK, wk_i = warp % WK;
    const int g = lane >> 2, t = lane & 3;
    const int lr0 = wr_i * 16 + g;  // local rows lr0 and lr0 + 8
    bool ok = mbar_wait_bounded(scale_bar, 0, failed, p.err, DERR_SCALE_WAIT);
    float row_scale0 = 1.f, row_scale1 = 1.f;
    if constexpr (KIND == I8_ROW) {
      if (row0 + lr0 < p.n_rows) row_scale0 = reinterpret_cast<const float*>(p.scales)[row0 + lr0];
      if (row0 + lr0 + 8 < p.n_rows) row_scale1 = reinterpret_cast<const float*>(p.scales)[row0 + lr0 + 8];
    }
    const uint8_t* sc0 = sc_smem + (size_t)lr0 * sc_stride;
    const uint8_t* sc1 = sc0 + 8 * (size_t)sc_stride;

    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it % S;
      const uint32_t ph = (uint32_t)(it / S) & 1u;
      ok = mbar_wait_bounded(&full_bar[s], ph, failed, p.err, DERR_FULL_WAIT);
      if (!ok) break;
      const int k0 = it * KB;
      const int kv = min(KB, p.kpad - k0);
      const int kw0 = wk_i * kWarpK;
      const uint8_t* st = body + (size_t)s * stage_bytes;
      const uint8_t* w0p = st + (size_t)lr0 * w_stride;
      const uint8_t* w1p = w0p + 8 * (size_t)w_stride;
      const uint8_t* xs = st + (size_t)R * w_stride;
#pragma unroll
      for (int j = 0; j < kWarpK / 32; ++j) {
        const int kk = kw0 + 32 * j;  // k offset of this 32-block inside the stage
        if (kk < kv) {
          uint32_t a_lo[4], a_hi[4];  // rows lr0 and lr0+8: [0]=(q0,q4) [1]=(q1,q5) [2]=(q2,q6) [3]=(q3,q7)
          if constexpr (kIs8) {
            const uint2 u0 = *reinterpret_cast<const uint2*>(w0p + kk + 8 * t);
            const uint2 u1 = *reinterpret_cast<const uint2*>(w1p + kk + 8 * t);
            dequant_i8_words(u0.x, u0.y, a_lo);
            dequant_i8_words(u1.x, u1.y, a_hi);
          } else {
            const uint32_t u0 = *reinterpret_cast<const uint32_t*>(w0p + kk / 2 + 4 * t);
            const uint32_t u1 = *reinterpret_cast<const uint32_t*>(w1p + kk / 2 + 4 * t);
            dequant_q4_word(u0, a_lo);
            dequant_q4_word(u1, a_hi);
          }
          float s0, s1;
          const int gi = (k0 + kk) >> 5;
          if constexpr (KIND == Q4_F16) {
            s0 = __half2float(*reinterpret_cast<const __half*>(sc0 + 2 * gi));
            s1 = __half2float(*reinterpret_cast<const __half*>(sc1 + 2 * gi));
          } else if constexpr (KIND == I8_ROW) {
            s0 = 1.f;
            s1 = 1.f;
          } else {
            s0 = *reinterpret_cast<const float*>(sc0 + 4 * gi);
            s1 = *reinterpret_cast<const float*>(sc1 + 4 * gi);
          }
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            const int tok = 8 * i + g;
            uint4 xv = make_uint4(0u, 0u, 0u, 0u);
            if (tok < p.mx) xv = *reinterpret_cast<const uint4*>(xs + (size_t)tok * x_stride + 2 * (kk + 8 * t));
            // xv = (x0,x1)(x2,x3)(x4,x5)(x6,x7); pair them as the dequantiser pairs the weights
            const uint32_t b04 = prmt(xv.x, xv.z, 0x5410u), b15 = prmt(xv.x, xv.z, 0x7632u);
            const uint32_t b26 = prmt(xv.y, xv.w, 0x5410u), b37 = prmt(xv.y, xv.w, 0x7632u);
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            mma_bf16_16816(part, a_lo[0], a_hi[0], a_lo[1], a_hi[1], b04, b15);
            mma_bf16_16816(part, a_lo[2], a_hi[2], a_lo[3], a_hi[3], b26, b37);
            if constexpr (KIND == I8_ROW) {
              acc[i][0] += part[0];
              acc[i][1] += part[1];
              acc[i][2] += part[2];
              acc[i][3] += part[3];
            } else {
              acc[i][0] = fmaf(s0, part[0], acc[i][0]);
              acc[i][1] = fmaf(s0, part[1], acc[i][1]);
              acc[i][2] = fmaf(s1, part[2], acc[i][2]);
              acc[i][3] = fmaf(s1, part[3], acc[i][3]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    if constexpr (KIND == I8_ROW) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        acc[i][0] *= row_scale0;
        acc[i][1] *= row_scale0;
        acc[i][2] *= row_scale1;
        acc[i][3] *= row_scale1;
      }
    }
  }

  // ------------------------------------------------------------------ split-K meet + store
  __syncthreads();  // every stage consumed (or the CTA has failed and no copy is awaited)
  const int RS = R + 4;
  float* red = reinterpret_cast<float*>(body);  // [WK][8*NT cols][RS]
  if (warp < n_consumers) {
    const int wr_i = warp / WK, wk_i = warp % WK;
    const int g = lane >> 2, t = lane & 3;
    float* base = red + (size_t)wk_i * (8 * NT) * RS + wr_i * 16 + g;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      base[(size_t)(8 * i + 2 * t) * RS] = acc[i][0];
      base[(size_t)(8 * i + 2 * t + 1) * RS] = acc[i][1];
      base[(size_t)(8 * i + 2 * t) * RS + 8] = acc[i][2];
      base[(size_t)(8 * i + 2 * t + 1) * RS + 8] = acc[i][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.m_out * R; idx += blockDim.x) {
    const int r = idx % R, m = idx / R;
    if (r >= rows_valid) continue;
    float v = 0.f;
    for (int c = 0; c < p.combine; ++c) {
      const int col = m * p.combine + c;
      for (int w = 0; w < WK; ++w) v += red[((size_t)w * (8 * NT) + col) * RS + r];
    }
    const size_t o = (size_t)m * p.ldy + row0 + r;
    if (p.residual) v += p.residual[o];
    if (p.y_bf16)
      reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
    else
      reinterpret_cast<float*>(p.y)[o] = v;
  }
}

}  // namespace tq
