// Weight-only quantised linear layer for 1..64 activation rows (decode):
//     y[m, n] = sum_k x[m, k] * q[n, k] * scale[n, k/32]
// restating crates/tang-infer/src/quantize.rs:227-289 (q8_matvec / q4_matvec) for the GPU.
//
// The kernel is bound by the HBM stream of the packed weights, so everything is arranged
// around that stream:
//   * weights live in HBM as fragment tiles (qlayout.cuh); the tiles one CTA needs for a
//     pipeline stage are contiguous, so ONE elected lane moves them with one bulk (TMA) copy per
//     16-row block through an S-stage mbarrier ring (L2 evict-first); the activation chunk of
//     the stage follows as one bulk copy per token row (L2 evict-last);
//   * WR x WK consumer warps each own 16 output rows and one 128-wide K slice of the stage.  A
//     lane reads its weights for four 32-blocks as two 16-byte vectors, turns each 32-bit word
//     (eight 4-bit values; or two words of int8) into exact bf16 integers in registers and feeds
//     mma.sync m16n8k16; the 32-block's scale multiplies the f32 partial sum afterwards, so
//     integer unpack and products are exact and only the f32 accumulation rounds;
//   * the WK partial sums of a row meet in shared memory (split-K inside the CTA).
// f32 activations are supported by the caller splitting every value into three bf16 terms
// (exactly) and asking for combine=3: three adjacent token columns are summed in the epilogue.
#pragma once

#include "common.cuh"
#include "qlayout.cuh"

namespace tq {

struct QGemmParams {
  const uint8_t* tiles;     // fragment tiles, [n_row_blocks][kc_total][tile_bytes]
  const float* row_scales;  // I8_ROW only: one f32 per output row
  const __nv_bfloat16* x;   // [mx][ldx] bf16, rows 16-byte aligned, kx valid elements per row
  void* y;                  // [m_out][ldy] f32 or bf16
  const float* residual;    // optional f32 [m_out][ldy] added before the store (may alias y)
  long long ldx, ldy;
  int n_rows;               // output features
  int n_row_blocks;         // ceil(n_rows / 16)
  int kc_total;             // ceil(K / 128)
  int kx;                   // activation row length, a multiple of 128 (K rounded up; zero beyond K)
  int mx;                   // activation rows present in x (<= 8*NT)
  int m_out;                // rows of y = mx / combine
  int combine;              // 1, or 3 for split-f32 activations
  int y_bf16;               // 0: f32 output, 1: bf16 output
  int wr, wk, stages;       // consumer grid inside the CTA and ring depth
  int tpw;                  // 128-k tiles each consumer warp handles per stage
  // Grouped launches (blockIdx.y = group): every group has its own weight of the same shape, `g_tile_stride`
  // bytes apart (row scales n_rows apart).  With g_counts, group e owns activation rows
  // g_offsets[e] .. +g_counts[e] of x / y and blockIdx.z walks them in chunks of 8*NT (expert batches);
  // without, group e's rows start g_x_stride / g_y_stride elements into x / y (one matrix per head).
  int grouped;
  const int* g_counts;
  const int* g_offsets;
  const int* g_active;    // optional: blockIdx.y indexes this list of group ids (-1 = unused entry)
  long long g_tile_stride, g_x_stride, g_y_stride;
  int* err;
};

// `kt` = 128-k tiles per stage (K slices x tiles per warp).
__host__ __device__ inline int qg_x_stride(int kt) { return kTileK * kt * 2 + 64; }  // 64 (mod 128): no bank conflicts
__host__ __device__ inline int qg_stage_bytes(int kind, int wr, int kt, int mx) {
  return wr * kt * qk_tile_bytes(kind) + mx * qg_x_stride(kt);
}
__host__ __device__ inline int qg_epilogue_bytes(int wr, int wk, int nt) { return wk * 8 * nt * (16 * wr + 4) * 4; }
constexpr int kQgHeaderBytes = 256;  // barriers + failure flag
constexpr int kQgMaxStages = 8;
__host__ __device__ inline size_t qg_smem_bytes(int kind, int nt, int wr, int wk, int tpw, int stages, int mx) {
  size_t pipe = (size_t)stages * qg_stage_bytes(kind, wr, wk * tpw, mx);
  size_t epi = (size_t)qg_epilogue_bytes(wr, wk, nt);
  return kQgHeaderBytes + qg_x_stride(wk * tpw) + (pipe > epi ? pipe : epi);
}

// mma with a zero accumulator input (the compiler then needs no registers for it)
__device__ __forceinline__ void mma_bf16_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

template <int KIND, int NT>
__global__ void __launch_bounds__(288, (NT == 1 ? 4 : (NT == 2 ? 3 : 1))) qgemm_mma_kernel(const QGemmParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool kIs8 = (KIND == Q8_F32 || KIND == I8_ROW);
  // Removing the +8 nibble bias with two constant-operand MMAs per block instead of eight subtractions was
  // measured SLOWER (12.6 -> 13.5 us at M = 1): the legacy HMMA pipe is already half busy on this kernel.
  constexpr bool kBiasByMma = false;
  constexpr int TB = kIs8 ? (KIND == I8_ROW ? 2048 : 2304) : (KIND == Q4_F16 ? 1152 : 1280);
  constexpr int WB = kIs8 ? 2048 : 1024;  // weight bytes of a tile; scales follow

  const int WR = p.wr, WK = p.wk, S = p.stages, TPW = p.tpw;
  const int KT = WK * TPW;             // 128-k tiles per stage
  const int R = 16 * WR;
  const int KB = kTileK * KT;
  const int x_stride = qg_x_stride(KT);
  const int stage_bytes = qg_stage_bytes(KIND, WR, KT, p.mx);
  const int x_region = WR * KT * TB;   // activations follow the tiles inside a stage

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kQgMaxStages;
  volatile int* failed = reinterpret_cast<volatile int*>(empty_bar + kQgMaxStages);
  uint8_t* zero_row = smem + kQgHeaderBytes;          // x_stride bytes of zeros: the "token" of idle lanes
  uint8_t* body = zero_row + x_stride;

  // per-launch or per-group operands
  int mx = p.mx;
  const uint8_t* tiles = p.tiles;
  const __nv_bfloat16* xg = p.x;
  const float* row_scales = p.row_scales;
  size_t y_off = 0;
  if (p.grouped) {
    pdl_wait();   // group tables and row offsets come from earlier kernels of the stream
    int e = blockIdx.y;
    if (p.g_active) {
      e = p.g_active[blockIdx.y];
      if (e < 0) return;                  // fewer groups have rows than the grid allowed for
    }
    tiles += (size_t)e * p.g_tile_stride;
    if (row_scales) row_scales += (size_t)e * p.n_rows;
    if (p.g_counts) {
      const int cnt = p.g_counts[e];
      const int m0 = blockIdx.z * 8 * NT;
      if (m0 >= cnt) return;              // whole CTA: nothing routed to this chunk
      mx = min(8 * NT, cnt - m0);
      const size_t row = (size_t)p.g_offsets[e] + m0;
      xg += row * p.ldx;
      y_off = row * p.ldy;
    } else {
      xg += (size_t)e * p.g_x_stride;
      y_off = (size_t)e * p.g_y_stride;
    }
  }
  const int m_out = p.grouped ? mx / p.combine : p.m_out;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_consumers = WR * WK;
  const int rb0 = blockIdx.x * WR;                       // first 16-row block of this CTA
  const int row0 = rb0 * 16;
  const int rbs_valid = min(WR, p.n_row_blocks - rb0);
  const int n_iters = (p.kc_total + KT - 1) / KT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], n_consumers);
    }
    *failed = 0;
    mbar_init_fence();
  }
  for (int i = threadIdx.x * 16; i < x_stride; i += blockDim.x * 16)
    *reinterpret_cast<uint4*>(zero_row + i) = make_uint4(0u, 0u, 0u, 0u);
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
    // The weights do not depend on the previous kernel of the stream, the activations do: the first
    // ring-full of weight tiles is requested before griddepcontrol.wait, the activation rows after.
    auto issue = [&](int it, int s, bool weights, bool acts) {
      const int kc0 = it * KT;
      const int kcs = min(KT, p.kc_total - kc0);                 // tiles along K in this stage
      const int kxv = max(0, min(KB, p.kx - kc0 * kTileK));       // activation elements in this stage
      const uint32_t wbytes = (uint32_t)(kcs * TB);
      const uint32_t xbytes = (uint32_t)kxv * 2u;
      uint8_t* st = body + (size_t)s * stage_bytes;
      if (weights) {
        if (lane == 0)
          mbar_arrive_expect_tx(&full_bar[s], wbytes * (uint32_t)rbs_valid + (xbytes ? xbytes * (uint32_t)mx : 0u));
        __syncwarp();
        for (int i = lane; i < rbs_valid; i += 32)
          bulk_g2s(st + (size_t)i * KT * TB, tiles + ((size_t)(rb0 + i) * p.kc_total + kc0) * TB, wbytes, &full_bar[s], pol_w);
      }
      if (acts && xbytes)
        for (int m = lane; m < mx; m += 32)
          bulk_g2s(st + x_region + (size_t)m * x_stride, xg + (size_t)m * p.ldx + (size_t)kc0 * kTileK, xbytes, &full_bar[s],
                   pol_x);
    };
    const int n_pre = min(S, n_iters);
    for (int it = 0; it < n_pre; ++it) issue(it, it, true, false);
    pdl_wait();
    pdl_launch_dependents();
    for (int it = 0; it < n_pre; ++it) issue(it, it, false, true);
    int s = n_pre == S ? 0 : n_pre;
    uint32_t ph = n_pre == S ? 1u : 0u;
    for (int it = n_pre; it < n_iters; ++it) {
      if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, failed, p.err, DERR_EMPTY_WAIT)) break;
      issue(it, s, true, true);
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
    }
  } else if (warp < n_consumers) {
    // ------------------------------------------------------------------ consumer warps
    // All shared-memory addressing below is "smem + 32-bit offset" so it costs one integer add.
    const int wr_i = warp / WK, wk_i = warp - wr_i * WK;
    const int g = lane >> 2, t = lane & 3;
    const bool rb_ok = wr_i < rbs_valid;
    const int body_off = kQgHeaderBytes + x_stride;
    const int tile_off = (wr_i * KT + wk_i * TPW) * TB + 16 * lane;  // this lane's first weight vector
    const int sc_off = (wr_i * KT + wk_i * TPW) * TB + WB + g * (KIND == Q4_F16 ? 8 : 16);
    const int x_lane = 2 * (wk_i * TPW * kTileK + 8 * t);            // this lane's k offset in an activation row
    int x_off[NT];                                                // stage-relative; < 0: idle lane (reads zeros)
#pragma unroll
    for (int i = 0; i < NT; ++i) x_off[i] = (8 * i + g < mx) ? x_region + (8 * i + g) * x_stride + x_lane : -1;
    const int zero_off = kQgHeaderBytes + x_lane;
    const bool lane0 = lane == 0;

    int s = 0;
    uint32_t ph = 0;
    int st0 = body_off;  // offset of the current stage
    int kc = wk_i * TPW;
#pragma unroll 1
    for (int it = 0; it < n_iters; ++it, kc += KT) {
      // (looking at the next stage's barrier one stage ahead was measured: 11.9 -> 12.4 us; with four CTAs per SM
      // the other warps already cover the wait)
      if (*failed) break;
      if (!mbar_wait_spin(&full_bar[s], ph)) {
        *failed = 1;
        atomicCAS(p.err, 0, (int)DERR_FULL_WAIT);
        break;
      }
      const int nu = rb_ok ? min(TPW, p.kc_total - kc) : 0;       // tiles of this warp that exist
#pragma unroll 1
      for (int u = 0; u < nu; ++u) {
        const int st = st0 + u * TB;                               // tile u: weights shift by TB, activations by 256 B
        const int xsh = u * (2 * kTileK - TB);
        uint32_t wlo[kIs8 ? 8 : 4], whi[kIs8 ? 8 : 4];
        if constexpr (kIs8) {
          const uint4 a0 = *reinterpret_cast<const uint4*>(smem + st + tile_off);
          const uint4 a1 = *reinterpret_cast<const uint4*>(smem + st + tile_off + 512);
          const uint4 b0 = *reinterpret_cast<const uint4*>(smem + st + tile_off + 1024);
          const uint4 b1 = *reinterpret_cast<const uint4*>(smem + st + tile_off + 1536);
          wlo[0] = a0.x; wlo[1] = a0.y; wlo[2] = a0.z; wlo[3] = a0.w; wlo[4] = a1.x; wlo[5] = a1.y; wlo[6] = a1.z; wlo[7] = a1.w;
          whi[0] = b0.x; whi[1] = b0.y; whi[2] = b0.z; whi[3] = b0.w; whi[4] = b1.x; whi[5] = b1.y; whi[6] = b1.z; whi[7] = b1.w;
        } else {
          const uint4 a = *reinterpret_cast<const uint4*>(smem + st + tile_off);
          const uint4 b = *reinterpret_cast<const uint4*>(smem + st + tile_off + 512);
          wlo[0] = a.x; wlo[1] = a.y; wlo[2] = a.z; wlo[3] = a.w;
          whi[0] = b.x; whi[1] = b.y; whi[2] = b.z; whi[3] = b.w;
        }
        float s_lo[4], s_hi[4];  // scales of rows g and g+8 for the four blocks
        if constexpr (KIND == Q4_F16) {
          const uint2 u0 = *reinterpret_cast<const uint2*>(smem + st + sc_off);
          const uint2 u1 = *reinterpret_cast<const uint2*>(smem + st + sc_off + 64);
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u0.x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u0.y));
          const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&u1.x));
          const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&u1.y));
          s_lo[0] = f0.x; s_lo[1] = f0.y; s_lo[2] = f1.x; s_lo[3] = f1.y;
          s_hi[0] = f2.x; s_hi[1] = f2.y; s_hi[2] = f3.x; s_hi[3] = f3.y;
        } else if constexpr (KIND != I8_ROW) {
          const float4 f0 = *reinterpret_cast<const float4*>(smem + st + sc_off);
          const float4 f1 = *reinterpret_cast<const float4*>(smem + st + sc_off + 128);
          s_lo[0] = f0.x; s_lo[1] = f0.y; s_lo[2] = f0.z; s_lo[3] = f0.w;
          s_hi[0] = f1.x; s_hi[1] = f1.y; s_hi[2] = f1.z; s_hi[3] = f1.w;
        }
        int xo[NT];
#pragma unroll
        for (int i = 0; i < NT; ++i) xo[i] = x_off[i] >= 0 ? st + xsh + x_off[i] : zero_off + u * 2 * kTileK;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a_lo[4], a_hi[4];  // rows g / g+8: (k0,k1) (k2,k3) (k4,k5) (k6,k7) of this lane's 8 k
          if constexpr (kIs8) {
            dequant_i8_words(wlo[2 * j], wlo[2 * j + 1], a_lo);
            dequant_i8_words(whi[2 * j], whi[2 * j + 1], a_hi);
          } else if constexpr (kBiasByMma) {
            dequant_q4_word_biased(wlo[j], a_lo);
            dequant_q4_word_biased(whi[j], a_hi);
          } else {
            dequant_q4_word(wlo[j], a_lo);
            dequant_q4_word(whi[j], a_hi);
          }
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            if (NT > 1 && 8 * i >= mx) break;   // token tiles beyond this launch's (or group's) rows: nothing to do
            const uint4 xv = *reinterpret_cast<const uint4*>(smem + xo[i] + 64 * j);
            float part[4];
            mma_bf16_16816_z(part, a_lo[0], a_hi[0], a_lo[1], a_hi[1], xv.x, xv.y);
            mma_bf16_16816(part, a_lo[2], a_hi[2], a_lo[3], a_hi[3], xv.z, xv.w);
            if constexpr (kBiasByMma) {   // the tensor pipe is far from busy here; the eight bias subtractions were not
              mma_bf16_16816(part, kNeg136x2, kNeg136x2, kNeg136x2, kNeg136x2, xv.x, xv.y);
              mma_bf16_16816(part, kNeg136x2, kNeg136x2, kNeg136x2, kNeg136x2, xv.z, xv.w);
            }
            if constexpr (KIND == I8_ROW) {
              acc[i][0] += part[0];
              acc[i][1] += part[1];
              acc[i][2] += part[2];
              acc[i][3] += part[3];
            } else {
              acc[i][0] = fmaf(s_lo[j], part[0], acc[i][0]);
              acc[i][1] = fmaf(s_lo[j], part[1], acc[i][1]);
              acc[i][2] = fmaf(s_hi[j], part[2], acc[i][2]);
              acc[i][3] = fmaf(s_hi[j], part[3], acc[i][3]);
            }
          }
        }
      }
      __syncwarp();
      mbar_arrive_if(&empty_bar[s], lane0);
      st0 += stage_bytes;
      if (++s == S) {
        s = 0;
        ph ^= 1u;
        st0 = body_off;
      }
    }
    if constexpr (KIND == I8_ROW) {
      const int r_lo = row0 + wr_i * 16 + g;
      const float rs0 = r_lo < p.n_rows ? row_scales[r_lo] : 0.f;
      const float rs1 = r_lo + 8 < p.n_rows ? row_scales[r_lo + 8] : 0.f;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        acc[i][0] *= rs0;
        acc[i][1] *= rs0;
        acc[i][2] *= rs1;
        acc[i][3] *= rs1;
      }
    }
  }

  // ------------------------------------------------------------------ split-K meet + store
  pdl_wait();       // results (and the residual) touch memory the previous kernel may still own
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
  const int rows_valid = min(R, p.n_rows - row0);
  for (int idx = threadIdx.x; idx < m_out * R; idx += blockDim.x) {
    const int r = idx % R, m = idx / R;
    if (r >= rows_valid) continue;
    float v = 0.f;
    for (int c = 0; c < p.combine; ++c) {
      const int col = m * p.combine + c;
      for (int w = 0; w < WK; ++w) v += red[((size_t)w * (8 * NT) + col) * RS + r];
    }
    const size_t o = y_off + (size_t)m * p.ldy + row0 + r;
    if (p.residual) v += p.residual[o];
    if (p.y_bf16)
      reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
    else
      reinterpret_cast<float*>(p.y)[o] = v;
  }
}

}  // namespace tq
