// Persistent dequant-GEMM for a few activation rows (2..8 as launched today; the kernel itself takes up to 16): y[m][n] = sum_k x[m][k] * W[n][k], W quantised (crates/tang-infer/src/quantize.rs:227-289
// repeated per activation row; the reference has no batched form).
//
// The one-row kernel of qgemv_sk.cuh keeps a CTA's whole activation vector in shared memory.  With more rows
// that copy crowds out the weight ring, so here K is cut into slabs of `skc` 128-wide chunks:
//   * the grid is n_slabs groups of `cps` CTAs; a group owns one slab and walks its units (row block, chunk of
//     the slab) in contiguous ranges, exactly as the one-row kernel walks all of K; a CTA keeps only its slab of
//     the activation rows (mx * skc * 256 bytes);
//   * W consumer warps take the tiles of a stage round-robin; a lane dequantises its weights once per 32-block
//     (the same exact 128 + n form, offset taken out by the accumulator input, block scale on the f32 partial)
//     and feeds NT mma.sync m16n8k16 column tiles of eight activation rows each;
//   * partial sums of a row block meet on three levels, always in a fixed order, so results are bit-reproducible:
//     the warps of a CTA through shared memory (epilogue warp, warp order), the CTAs of a slab that share a row
//     block through tagged words in a workspace (CTA order, the lowest CTA adds), and the slabs through a second
//     tagged workspace indexed by (slab, row block): when a CTA's consumer warps are done they add up, slabs in
//     order, the row blocks that their CTA index completes in every slab (each slab's CTA takes every n_slabs-th).
// No CTA waits for one that could be waiting for it: nothing that is parked waits for another CTA, except the lowest
// CTA of a cut row block, which waits for what higher CTAs of its slab park as the first thing they do.  Every wait
// is bounded.
#pragma once

#include "qgemv_sk.cuh"

namespace tq {

// Floats per warp and hand-over buffer, and the shared-memory pieces, for NT column tiles.
__host__ __device__ inline int skw_red_floats(int nt) { return nt * 8 * kSkRedStride; }
// two buffers of per-warp partial sums, then kSkwSums of their sums ([16 rows][nt * 8 columns], column-major)
constexpr int kSkwSums = 8;          // buffers of summed row blocks between the consumer warps and the epilogue warp
constexpr int kSkwHeaderBytes = 384;
__host__ __device__ inline int skw_red_bytes(int w, int nt) { return 2 * w * skw_red_floats(nt) * 4 + kSkwSums * nt * 128 * 4; }
__host__ __device__ inline int skw_x_stride(int skc) { return skc * 256 + 64; }
__host__ __device__ inline int skw_csum_bytes(int kind, int skc, int nt) {
  return (kind == Q4_F32 || kind == Q4_F16) ? skc * 4 * nt * 8 * 4 : 0;
}
__host__ __device__ inline size_t skw_fixed_bytes(int kind, int w, int skc, int mx, int nt) {
  return (size_t)kSkwHeaderBytes + skw_red_bytes(w, nt) + (size_t)mx * skw_x_stride(skc) + skw_csum_bytes(kind, skc, nt);
}

template <int KIND, int W, int TPW, int NT, int MINB = 2, bool SS = false>
__global__ void __launch_bounds__(32 * (W + 2), MINB) qgemm_sk_kernel(const QGemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool kIs8 = (KIND == Q8_F32 || KIND == I8_ROW);
  constexpr int TB = kIs8 ? (KIND == I8_ROW ? 2048 : 2304) : (KIND == Q4_F16 ? 1152 : 1280);
  constexpr int WB = kIs8 ? 2048 : 1024;
  constexpr int G = W * TPW;          // tiles per stage
  constexpr int CSN = NT * 8;         // floats per 32-block in the offset table: one per activation row
  constexpr int NBUF = kSkwSums;     // sums buffers (the per-warp partial buffers alternate by segment parity)
  constexpr int RF = NT * 8 * kSkRedStride;
  constexpr int NV = NT * 4;          // values per lane of a row block's [16 rows][NT * 8 columns]

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kSkMaxStages;
  uint64_t* x_bar = empty_bar + kSkMaxStages;
  uint64_t* red_full = x_bar + 1;     // [NBUF]
  uint64_t* red_empty = red_full + NBUF; // [NBUF]
  volatile int* failed = reinterpret_cast<volatile int*>(red_empty + NBUF);

  const int S = p.stages;
  const int skc = p.skc;
  const int cps = p.cps;
  const int slab = (int)blockIdx.x / cps, j = (int)blockIdx.x - slab * cps;
  const int kxs = skc * 128;          // activations per row in this CTA's slab
  const int x_stride = skw_x_stride(skc);
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t red_off = kSkwHeaderBytes;
  const uint32_t x_off = red_off + skw_red_bytes(W, NT);
  const uint32_t cs_off = x_off + (uint32_t)p.mx * x_stride;
  const uint32_t ring_off = cs_off + skw_csum_bytes(KIND, skc, NT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long U = (long long)p.n_row_blocks * skc;     // units of one slab
  const long long u0 = U * j / cps, u1 = U * (j + 1) / cps;
  SkWalk start;
  start.rb = (int)(u0 / skc);
  start.kc = (int)(u0 - (long long)start.rb * skc);
  start.left = (int)(u1 - u0);

  if (p.x_early && threadIdx.x == 0) pdl_launch_dependents();
  if (threadIdx.x < S) {
    mbar_init(&full_bar[threadIdx.x], 1);
    mbar_init(&empty_bar[threadIdx.x], W);
  } else if (threadIdx.x >= 32 && threadIdx.x < 32 + NBUF) {
    mbar_init(&red_full[threadIdx.x - 32], W);
    mbar_init(&red_empty[threadIdx.x - 32], 1);
  } else if (threadIdx.x == 64) {
    mbar_init(x_bar, 1);
    *failed = 0;
  }
  mbar_init_fence();
  __syncthreads();

  const int n_out = p.m_out * 16;            // (row of the block, output row of x) pairs, <= NT * 128
  auto store = [&](int rb, const float (&vals)[NV]) {
    if (p.swiglu) {
      // rows 0..7 of the block hold gate values, rows 8..15 the up values of the same eight outputs
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        const float up = __shfl_down_sync(0xffffffffu, vals[i], 8);
        const int r8 = idx & 15, m = idx >> 4;
        const int o_col = rb * 8 + r8;
        if (idx < n_out && r8 < 8 && o_col < p.n_rows / 2) {
          const float gt = vals[i];
          const float act = gt * (1.0f / (1.0f + expf(-gt))) * up;   // the formula of swiglu_kernel, term for term
          const size_t o = (size_t)m * p.ldy + o_col;
          if (p.y_bf16)
            reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(act);
          else
            reinterpret_cast<float*>(p.y)[o] = act;
        }
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = lane + 32 * i;
      const int r = rb * 16 + (idx & 15), m = idx >> 4;
      float sq = 0.f;
      if (idx < n_out && r < p.n_rows) {
        const size_t o = (size_t)m * p.ldy + r;
        float v = vals[i];
        if (p.residual) v += p.residual[o];
        if (p.y_bf16)
          reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
        else
          reinterpret_cast<float*>(p.y)[o] = v;
        sq = v * v;
      }
      if constexpr (SS)
        if (p.ss_out) sk_store_sumsq(p.ss_out, sq, lane, m, p.m_out, p.n_row_blocks, rb);
    }
  };
  // One parked partial: NT * 128 words of (value bits | tag << 32), each written with one 64-bit store.  Adds what
  // is parked at `part` to vals and clears it; false: gave up.
  auto take = [&](unsigned long long* part, float (&vals)[NV], int code) -> bool {
    unsigned long long got[NV];
    uint32_t polls = 0;
    for (;;) {
      bool ready = true;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        got[i] = 1ull << 32;
        if (lane + 32 * i < n_out) got[i] = ld_relaxed_u64(part + lane + 32 * i);
        ready = ready && (got[i] >> 32) != 0;
      }
      if (__all_sync(0xffffffffu, ready)) break;
      if (++polls > kMaxPolls || *failed) {
        *failed = 1;
        atomicCAS(p.err, 0, code);
        return false;
      }
      __nanosleep(32);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < n_out) {
        vals[i] += __uint_as_float((uint32_t)got[i]);
        st_relaxed_u64(part + lane + 32 * i, 0ull);
      }
    return true;
  };
  auto park = [&](unsigned long long* part, const float (&vals)[NV]) {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < n_out) st_relaxed_u64(part + lane + 32 * i, (1ull << 32) | __float_as_uint(vals[i]));
  };

  if (warp == W) {
    // ------------------------------------------------------------------ producer (one lane)
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      SkWalk w = start;
      auto issue = [&](int s) {
        const int n = min(G, min(skc - w.kc, w.left));
        const uint32_t bytes = (uint32_t)n * TB;
        const uint8_t* src = p.tiles + ((size_t)w.rb * p.kc_total + (size_t)slab * skc + w.kc) * TB;
        mbar_arrive_expect_tx(&full_bar[s], bytes);
        bulk_g2s(smem + ring_off + (size_t)s * (G * TB), src, bytes, &full_bar[s], pol_w);
        w.left -= n;
        w.kc += n;
        if (w.kc == skc) {
          w.kc = 0;
          ++w.rb;
        }
      };
      auto load_x = [&]() {
        mbar_arrive_expect_tx(x_bar, (uint32_t)p.mx * (uint32_t)kxs * 2u);
        for (int m = 0; m < p.mx; ++m)
          bulk_g2s(smem + x_off + (size_t)m * x_stride, p.x + (size_t)m * p.ldx + (size_t)slab * kxs, (uint32_t)kxs * 2u, x_bar, pol_x);
      };
      int issued = 0;
      if (p.x_tag) {
        // activations staged by the kernel launched just before this one: ring first, then a bounded look at its tag
        while (w.left > 0 && issued < S) issue(issued++);
        uint32_t polls = 0;
        const unsigned want = sk_x_tag_value(p.x_seq, p.x_epoch);
        for (;;) {
          unsigned v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.x_tag) : "memory");
          if (v == want) break;
          if (++polls > kMaxPolls) {
            *failed = 1;
            atomicCAS(p.err, 0, (int)DERR_FULL_WAIT);
            break;
          }
          __nanosleep(32);
        }
        load_x();
      } else if (p.x_early && !p.norm_w) {
        load_x();
      }
      while (w.left > 0 && issued < S) issue(issued++);
      if (!p.x_early && !p.norm_w && !p.x_tag) {   // (a second arrival on x_bar in one phase would overrun its count)
        pdl_wait();
        load_x();
      }
      int s = 0;
      uint32_t ph = 1u;   // only reached with issued == S
      while (w.left > 0) {
        if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, failed, p.err, DERR_EMPTY_WAIT)) break;
        issue(s);
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp < W) {
    // ------------------------------------------------------------------ consumer warps
    const int g = lane >> 2, t = lane & 3;
    bool ok = true;
    if (p.norm_w) {
      // fused rms_norm_residual (device.rs:546-575): the sum of squares runs over the whole row, the normalised
      // values are formed for this CTA's slab only; the first CTA of every slab writes its part of h + delta
      if (p.x_early == 0) pdl_wait();
      float* scratch = reinterpret_cast<float*>(smem + red_off);
      // all rows at once: a group of gsz warps per row (W / gsz >= mx groups), so that the rows' loads overlap
      int gsz = W;
      while (gsz > 1 && W / gsz < p.mx) gsz >>= 1;
      const int m = warp / gsz, sub = warp - m * gsz;
      const bool live = m < p.mx;
      const float* hrow = p.nh + (size_t)(live ? m : 0) * p.ld_h;
      const float* drow = p.ndelta ? p.ndelta + (size_t)(live ? m : 0) * p.ld_h : nullptr;
      float sq = 0.f;
      float total = 0.f;
      const bool have_ss = SS && p.ss_in != nullptr;
      if (have_ss) total = sk_load_sumsq(p.ss_in + (size_t)(live ? m : 0) * p.ss_n, p.ss_n, lane);
      if (live && !have_ss)
        for (int k = 4 * (sub * 32 + lane); k < p.kx; k += 128 * gsz) {
          float4 v = __ldcg(reinterpret_cast<const float4*>(hrow + k));
          if (drow) {
            const float4 d = __ldcg(reinterpret_cast<const float4*>(drow + k));
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
          }
          sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
      if (!have_ss) {
        sq = warp_sum(sq);
        if (lane == 0) scratch[warp] = sq;
        asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
      }
      if (live) {
        if (!have_ss)
          for (int q = 0; q < gsz; ++q) total += scratch[m * gsz + q];
        const float inv = 1.0f / sqrtf(total / (float)p.kx + p.norm_eps);
        uint8_t* xrow_s = smem + x_off + (size_t)m * x_stride;
        const int k0 = slab * kxs;
        for (int kk = 4 * (sub * 32 + lane); kk < kxs; kk += 128 * gsz) {
          const int k = k0 + kk;
          float4 v = __ldcg(reinterpret_cast<const float4*>(hrow + k));
          if (drow) {
            const float4 d = __ldcg(reinterpret_cast<const float4*>(drow + k));
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
          }
          const uint2 gw = *reinterpret_cast<const uint2*>(p.norm_w + k);
          const float g0 = bf16_bits_to_float(gw.x & 0xFFFFu), g1 = bf16_bits_to_float(gw.x >> 16);
          const float g2 = bf16_bits_to_float(gw.y & 0xFFFFu), g3 = bf16_bits_to_float(gw.y >> 16);
          const __nv_bfloat162 a = __floats2bfloat162_rn(v.x * inv * g0, v.y * inv * g1);
          const __nv_bfloat162 b = __floats2bfloat162_rn(v.z * inv * g2, v.w * inv * g3);
          *reinterpret_cast<uint2*>(xrow_s + 2 * kk) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
          if (p.nh_out && j == 0) *reinterpret_cast<float4*>(p.nh_out + (size_t)m * p.ld_h + k) = v;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
    } else {
      ok = mbar_wait_bounded(x_bar, 0u, failed, p.err, DERR_FULL_WAIT);
    }
    if constexpr (!kIs8) {
      // offset table: -136 * (sum of the block's 32 activations), per activation row
      const int nblk = kxs / 32;
      float* cs = reinterpret_cast<float*>(smem + cs_off);
      if (ok) {
        for (int e = threadIdx.x; e < nblk * CSN; e += 32 * W) {
          const int b = e / CSN, m = e - b * CSN;
          float sum = 0.f;
          if (m < p.mx) {
            const uint32_t a = smem0 + x_off + (uint32_t)m * x_stride + (uint32_t)b * 64u;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 v = lds128(a + 16u * q);
              const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) sum += bf16_bits_to_float(wv[i] & 0xFFFFu) + bf16_bits_to_float(wv[i] >> 16);
            }
          }
          cs[e] = -136.0f * sum;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
    }

    uint32_t xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)   // idle columns read a live row
      xrow[nt] = smem0 + x_off + (uint32_t)min(nt * 8 + g, p.mx - 1) * x_stride + 16u * t;
    const uint32_t csl = smem0 + cs_off + 8u * t;
    const uint32_t wl = smem0 + ring_off + 16u * lane;
    const uint32_t scl = smem0 + ring_off + WB + g * (KIND == Q4_F16 ? 8 : 16);

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    SkWalk w = start;
    int s = 0, buf = 0, pbuf = 0;
    uint32_t ph = 0, rph = 0;
    // (a warp that gives up a wait keeps walking the loop without working or waiting, so that the CTA-wide barriers of
    // the hand-over below still see every warp; after the first such barrier all warps know and do the same)
    bool dead = !ok;
    while (w.left > 0) {
      const int n = min(G, min(skc - w.kc, w.left));
      if (!dead && !mbar_wait_spin(&full_bar[s], ph)) {
        *failed = 1;
        atomicCAS(p.err, 0, (int)DERR_FULL_WAIT);
        dead = true;
      }
      const uint32_t st = (uint32_t)s * (G * TB);
#pragma unroll
      for (int jj = 0; jj < TPW; ++jj) {
        const int i = warp + jj * W;
        if (i < n && !dead) {
          const uint32_t to = st + (uint32_t)i * TB;
          const uint32_t kco = (uint32_t)(w.kc + i);
          uint32_t wlo[kIs8 ? 8 : 4], whi[kIs8 ? 8 : 4];
          if constexpr (kIs8) {
            const uint4 a0 = lds128(wl + to), a1 = lds128(wl + to + 512), b0 = lds128(wl + to + 1024), b1 = lds128(wl + to + 1536);
            wlo[0] = a0.x; wlo[1] = a0.y; wlo[2] = a0.z; wlo[3] = a0.w; wlo[4] = a1.x; wlo[5] = a1.y; wlo[6] = a1.z; wlo[7] = a1.w;
            whi[0] = b0.x; whi[1] = b0.y; whi[2] = b0.z; whi[3] = b0.w; whi[4] = b1.x; whi[5] = b1.y; whi[6] = b1.z; whi[7] = b1.w;
          } else {
            const uint4 a = lds128(wl + to), b = lds128(wl + to + 512);
            wlo[0] = a.x; wlo[1] = a.y; wlo[2] = a.z; wlo[3] = a.w;
            whi[0] = b.x; whi[1] = b.y; whi[2] = b.z; whi[3] = b.w;
          }
          float s_lo[4], s_hi[4];
          if constexpr (KIND == Q4_F16) {
            const uint2 v0 = lds64(scl + to), v1 = lds64(scl + to + 64);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v0.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v0.y));
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&v1.x));
            const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&v1.y));
            s_lo[0] = f0.x; s_lo[1] = f0.y; s_lo[2] = f1.x; s_lo[3] = f1.y;
            s_hi[0] = f2.x; s_hi[1] = f2.y; s_hi[2] = f3.x; s_hi[3] = f3.y;
          } else if constexpr (KIND != I8_ROW) {
            const uint4 v0 = lds128(scl + to), v1 = lds128(scl + to + 128);
            s_lo[0] = __uint_as_float(v0.x); s_lo[1] = __uint_as_float(v0.y); s_lo[2] = __uint_as_float(v0.z); s_lo[3] = __uint_as_float(v0.w);
            s_hi[0] = __uint_as_float(v1.x); s_hi[1] = __uint_as_float(v1.y); s_hi[2] = __uint_as_float(v1.z); s_hi[3] = __uint_as_float(v1.w);
          }
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            uint32_t a_lo[4], a_hi[4];
            if constexpr (kIs8) {
              dequant_i8_words(wlo[2 * b], wlo[2 * b + 1], a_lo);
              dequant_i8_words(whi[2 * b], whi[2 * b + 1], a_hi);
            } else {
              dequant_q4_word_offset(wlo[b], a_lo);
              dequant_q4_word_offset(whi[b], a_hi);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint4 xv = lds128(xrow[nt] + kco * 256u + 64u * b);
              float part[4];
              if constexpr (kIs8) {
                part[0] = part[1] = part[2] = part[3] = 0.f;
              } else {
                const uint2 cv = lds64(csl + ((kco * 4u + b) * CSN + nt * 8u) * 4u);
                part[0] = part[2] = __uint_as_float(cv.x);
                part[1] = part[3] = __uint_as_float(cv.y);
              }
              mma_bf16_16816(part, a_lo[0], a_hi[0], a_lo[1], a_hi[1], xv.x, xv.y);
              mma_bf16_16816(part, a_lo[2], a_hi[2], a_lo[3], a_hi[3], xv.z, xv.w);
              if constexpr (KIND == I8_ROW) {
                acc[nt][0] += part[0];
                acc[nt][1] += part[1];
                acc[nt][2] += part[2];
                acc[nt][3] += part[3];
              } else {
                acc[nt][0] = fmaf(s_lo[b], part[0], acc[nt][0]);
                acc[nt][1] = fmaf(s_lo[b], part[1], acc[nt][1]);
                acc[nt][2] = fmaf(s_hi[b], part[2], acc[nt][2]);
                acc[nt][3] = fmaf(s_hi[b], part[3], acc[nt][3]);
              }
            }
          }
        }
      }
      __syncwarp();
      mbar_arrive_if(&empty_bar[s], lane == 0);
      const bool seg_end = (w.kc + n == skc) || (n == w.left);
      if (seg_end) {
        // Hand-over: every warp writes its partial [16][NT * 8], the warps meet, each adds up one W-th of the outputs
        // over the warps (in warp order) and the epilogue warp gets the sums.  The partial buffers alternate and need
        // no barrier of their own: a warp is back at the same buffer only after the next segment's meeting, which
        // every warp reaches after it has read its share of this one.
        if (!dead && !mbar_wait_spin(&red_empty[buf], rph ^ 1u)) {   // (the sums of kSkwSums segments ago have been read)
          *failed = 1;
          atomicCAS(p.err, 0, (int)DERR_EMPTY_WAIT);
          dead = true;
        }
        float rs0 = 1.f, rs1 = 1.f;
        if constexpr (KIND == I8_ROW) {
          const int r_lo = w.rb * 16 + g;
          rs0 = r_lo < p.n_rows ? p.row_scales[r_lo] : 0.f;
          rs1 = r_lo + 8 < p.n_rows ? p.row_scales[r_lo + 8] : 0.f;
        }
        float* part0 = reinterpret_cast<float*>(smem + red_off) + (size_t)pbuf * W * RF;
        pbuf ^= 1;
        float* red = part0 + (size_t)warp * RF;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float* c = red + (nt * 8 + 2 * t) * kSkRedStride + g;
          c[0] = acc[nt][0] * rs0;
          c[8] = acc[nt][2] * rs1;
          c[kSkRedStride] = acc[nt][1] * rs0;
          c[kSkRedStride + 8] = acc[nt][3] * rs1;
          acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
        if (*failed) dead = true;
        if (lane < NT * 16) {
          const int o = warp * (NT * 16) + lane;       // output (column o / 16, row o % 16)
          const float* src = part0 + (o >> 4) * kSkRedStride + (o & 15);
          float v = 0.f;
#pragma unroll
          for (int q = 0; q < W; ++q) v += src[q * RF];
          reinterpret_cast<float*>(smem + red_off)[2 * W * RF + buf * (NT * 128) + o] = v;
        }
        __syncwarp();
        mbar_arrive_if(&red_full[buf], lane == 0 && !dead);
        if (++buf == NBUF) {
          buf = 0;
          rph ^= 1u;
        }
      }
      w.left -= n;
      w.kc += n;
      if (w.kc == skc) {
        w.kc = 0;
        ++w.rb;
      }
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (p.n_slabs > 1 && !dead) {
      // ---- the slabs' sums meet: every slab has the same ranges, so the CTAs with this index complete the same row
      // blocks (those whose first unit they own) at about the same time; slab s adds up the blocks with
      // rb % n_slabs == s, one per warp at a time, slabs in order 0, 1, ..  The parks waited for here never wait
      // for anything themselves.
      pdl_wait();
      const int rb_lo = (int)((u0 + skc - 1) / skc), rb_hi = (int)((u1 + skc - 1) / skc);
      int first = rb_lo + ((slab - rb_lo) % p.n_slabs + p.n_slabs) % p.n_slabs;
      for (int rb = first + warp * p.n_slabs; rb < rb_hi; rb += W * p.n_slabs) {
        float vals[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) vals[i] = 0.f;
        bool good = true;
        for (int sl = 0; sl < p.n_slabs && good; ++sl)
          good = take(p.ws2 + ((size_t)sl * p.n_row_blocks + rb) * (NT * 128), vals, (int)DERR_PEER_WAIT);
        if (!good) break;
        store(rb, vals);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warp
    pdl_wait();    // y, the residual and both workspaces belong to earlier kernels until then
    if (!p.x_early) pdl_launch_dependents();
    // the slab's sum for a row block is complete in vals: stored when K is one slab, else parked for the warps that
    // add the slabs at the end
    auto emit = [&](int rb, float (&vals)[NV]) {
      if (p.n_slabs == 1) store(rb, vals);
      else park(p.ws2 + ((size_t)slab * p.n_row_blocks + rb) * (NT * 128), vals);
    };
    // Within the slab: a row block cut by range boundaries belongs to CTAs c_first..c_last of the slab.  The higher
    // ones park their partial sums (the block is the first thing they work on); the lowest one, for which the
    // block is the LAST segment of its range, adds them in CTA order.
    const long long last_u = u1 - 1;
    const int last_rb = (int)(last_u / skc);
    const long long last_ub = (long long)last_rb * skc;
    const bool last_cut = u1 != last_ub + skc;
    const bool finisher = last_cut && (int)(((last_ub + 1) * cps - 1) / U) == j;
    const int fin_last = finisher ? (int)(((last_ub + skc) * cps - 1) / U) : 0;
    auto peer_slot = [&](int c) {   // c: CTA index inside the slab
      const int c_rb0 = (int)((U * c / cps) / skc);
      return (slab * cps + c) * 2 + (c_rb0 == last_rb ? 0 : 1);
    };
    SkWalk w = start;
    int buf = 0;
    uint32_t rph = 0;
    bool first_seg = true;
    while (w.left > 0) {
      const int seg = min(skc - w.kc, w.left);
      const bool whole = (w.kc == 0 && seg == skc);
      const bool is_last = seg == w.left;
      if (!mbar_wait_bounded(&red_full[buf], rph, failed, p.err, DERR_FULL_WAIT)) break;
      const float* sums = reinterpret_cast<const float*>(smem + red_off) + 2 * W * RF + buf * (NT * 128);
      float vals[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        float v = 0.f;
        if (idx < n_out) {
          const int r = idx & 15, m = idx >> 4;
          for (int c = 0; c < p.combine; ++c) v += sums[(m * p.combine + c) * 16 + r];
        }
        vals[i] = v;
      }
      __syncwarp();
      mbar_arrive_if(&red_empty[buf], lane == 0);
      bool good = true;
      if (whole) {
        emit(w.rb, vals);
      } else if (is_last && finisher) {
        for (int c = j + 1; c <= fin_last && good; ++c)   // own k range first, then the higher ones in CTA order
          good = take(p.ws + (size_t)peer_slot(c) * (NT * 128), vals, (int)DERR_PEER_WAIT);
        if (good) emit(w.rb, vals);
      } else {
        park(p.ws + (size_t)((slab * cps + j) * 2 + (first_seg ? 0 : 1)) * (NT * 128), vals);
      }
      if (!good) break;
      first_seg = false;
      w.left -= seg;
      w.kc += seg;
      if (w.kc == skc) {
        w.kc = 0;
        ++w.rb;
      }
      if (++buf == NBUF) {
        buf = 0;
        rph ^= 1u;
      }
    }
  }
}

}  // namespace tq
