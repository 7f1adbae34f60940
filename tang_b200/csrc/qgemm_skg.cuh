// Grouped dequant-GEMM for a few activation rows per group: one launch over many weights of the same shape stacked
// by rows (a mixture-of-experts layer's experts, the per-head matrices of latent attention), each with its own rows
// of x.  The reference has neither; per group this is crates/tang-infer/src/quantize.rs:227-289 repeated per row.
//
// blockIdx.y picks the group (through the list of groups that have rows, when there is one), blockIdx.z a chunk of
// eight of its activation rows, and the gridDim.x CTAs of such a job walk the weight's (row block, 128-k chunk)
// tiles in contiguous ranges, as the ungrouped kernels of qgemv_sk.cuh / qgemm_sk.cuh do: a ring of bulk copies, W
// consumer warps, exact 128 + n operands with the offset taken out through the accumulator, the block scale on the
// f32 partial sum, the warps' sums added in shared memory.  K is at most 17 chunks here, so a CTA keeps its job's
// whole activation rows (<= 36 KB).
// Which groups have rows is only known on the device, so the grid is sized for the worst case and may exceed what
// the GPU holds at once.  A row block cut by range boundaries is therefore finished by the HIGHEST CTA that holds
// part of it, which waits -- bounded -- only for CTAs with lower indices, and those are never scheduled later; each
// lower one parks its partial sums (tagged 64-bit words) when it reaches the end of its range, and the finisher
// adds them, in CTA order, at the end of its own.  Sums have a fixed order: results are bit-reproducible.
#pragma once

#include "qgemm_sk.cuh"

namespace tq {

struct QGroupParams {
  const uint8_t* tiles;       // [n_groups][n_row_blocks][kc_total][tile bytes]
  const float* row_scales;    // I8_ROW: [n_groups][n_rows]
  const __nv_bfloat16* x;
  void* y;
  long long ldx, ldy;
  int n_rows, n_row_blocks, kc_total;   // per group
  int mx;                     // rows of every group when counts == nullptr
  int y_bf16, stages;
  const int* counts;          // optional: rows of group e are offsets[e] .. + counts[e] of x / y
  const int* offsets;
  const int* active;          // optional: blockIdx.y indexes this list of group ids (-1 = unused entry)
  const int* jobs;            // optional (with counts): blockIdx.y indexes this list of (group | row chunk << 16), -1 = unused entry;
                              // gridDim.z is then 1
  long long x_stride, y_stride;   // without counts: group e's rows start e * stride elements into x / y
  unsigned long long* ws;     // [CTAs of the grid][128] tagged words, all zero between launches
  int* err;
};

// The jobs of a grouped launch whose row counts live on the device: one entry per (group with rows, chunk of eight
// of its rows), groups in list order, then -1s up to `bound`.  One CTA of 256 threads, a group per thread (more
// groups: several rounds), positions from a prefix sum over the CTA.
__global__ void __launch_bounds__(256) skg_jobs_kernel(const int* counts, const int* active, int n_listed, int* jobs, int bound) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ int warp_sums[8];
  __shared__ int base_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  for (int a0 = 0; a0 < n_listed; a0 += 256) {
    const int a = a0 + threadIdx.x;
    int e = -1, chunks = 0;
    if (a < n_listed) {
      e = active ? active[a] : a;
      if (e >= 0) chunks = (counts[e] + 7) / 8;
    }
    int incl = chunks;                        // inclusive prefix sum over the warp, then over the warps
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int before = base_s;
    for (int q = 0; q < warp; ++q) before += warp_sums[q];
    int pos = before + incl - chunks;
    for (int c = 0; c < chunks && pos < bound; ++c, ++pos) jobs[pos] = e | (c << 16);
    __syncthreads();
    if (threadIdx.x == 255) base_s = before + incl;
    __syncthreads();
  }
  for (int i = base_s + threadIdx.x; i < bound; i += 256) jobs[i] = -1;
}

template <int KIND, int W, int TPW>
__global__ void __launch_bounds__(32 * (W + 2), 2) qgemm_skg_kernel(const QGroupParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool kIs8 = (KIND == Q8_F32 || KIND == I8_ROW);
  constexpr int TB = kIs8 ? (KIND == I8_ROW ? 2048 : 2304) : (KIND == Q4_F16 ? 1152 : 1280);
  constexpr int WB = kIs8 ? 2048 : 1024;
  constexpr int G = W * TPW;
  constexpr int CSN = 8;
  constexpr int NBUF = kSkwSums;
  constexpr int RF = 8 * kSkRedStride;
  constexpr int NV = 4;
  static_assert(W == 8, "the hand-over gives each of eight warps sixteen of the 128 outputs");

  // ---- which job: group tables and row offsets come from earlier kernels of the stream
  pdl_wait();
  int e = blockIdx.y;
  int m0 = blockIdx.z * 8;
  if (p.jobs) {
    const int job = p.jobs[blockIdx.y];
    if (job < 0) return;
    e = job & 0xFFFF;
    m0 = (job >> 16) * 8;
  } else if (p.active) {
    e = p.active[blockIdx.y];
    if (e < 0) return;
  }
  int mx;
  size_t row0;   // first row of this job in x / y, in elements of one row's stride
  const __nv_bfloat16* xg = p.x;
  size_t y_off = 0;
  if (p.counts) {
    const int cnt = p.counts[e];
    if (m0 >= cnt) return;
    mx = min(8, cnt - m0);
    row0 = (size_t)p.offsets[e] + m0;
    xg += row0 * p.ldx;
    y_off = row0 * p.ldy;
  } else {
    if (m0 >= p.mx) return;
    mx = min(8, p.mx - m0);
    xg += (size_t)e * p.x_stride + (size_t)m0 * p.ldx;
    y_off = (size_t)e * p.y_stride + (size_t)m0 * p.ldy;
  }
  const int skc = p.kc_total;
  const uint8_t* tiles = p.tiles + (size_t)e * p.n_row_blocks * skc * TB;
  const float* row_scales = p.row_scales ? p.row_scales + (size_t)e * p.n_rows : nullptr;

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kSkMaxStages;
  uint64_t* x_bar = empty_bar + kSkMaxStages;
  uint64_t* red_full = x_bar + 1;
  uint64_t* red_empty = red_full + NBUF;
  volatile int* failed = reinterpret_cast<volatile int*>(red_empty + NBUF);

  const int S = p.stages;
  const int cps = gridDim.x, j = blockIdx.x;
  const int kxs = skc * 128;
  const int x_stride = skw_x_stride(skc);
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t red_off = kSkwHeaderBytes;
  const uint32_t x_off = red_off + skw_red_bytes(W, 1);
  const uint32_t cs_off = x_off + 8u * x_stride;
  const uint32_t ring_off = cs_off + skw_csum_bytes(KIND, skc, 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long U = (long long)p.n_row_blocks * skc;
  const long long u0 = U * j / cps, u1 = U * (j + 1) / cps;
  if (u1 == u0) return;                       // more CTAs than tiles
  SkWalk start;
  start.rb = (int)(u0 / skc);
  start.kc = (int)(u0 - (long long)start.rb * skc);
  start.left = (int)(u1 - u0);

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

  const int n_out = mx * 16;
  const size_t my_slot = ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 128;

  if (warp == W) {
    // ------------------------------------------------------------------ producer (one lane)
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      SkWalk w = start;
      auto issue = [&](int s) {
        const int n = min(G, min(skc - w.kc, w.left));
        const uint32_t bytes = (uint32_t)n * TB;
        mbar_arrive_expect_tx(&full_bar[s], bytes);
        bulk_g2s(smem + ring_off + (size_t)s * (G * TB), tiles + ((size_t)w.rb * skc + w.kc) * TB, bytes, &full_bar[s], pol_w);
        w.left -= n;
        w.kc += n;
        if (w.kc == skc) {
          w.kc = 0;
          ++w.rb;
        }
      };
      mbar_arrive_expect_tx(x_bar, (uint32_t)mx * (uint32_t)kxs * 2u);
      for (int m = 0; m < mx; ++m)
        bulk_g2s(smem + x_off + (size_t)m * x_stride, xg + (size_t)m * p.ldx, (uint32_t)kxs * 2u, x_bar, pol_x);
      int issued = 0;
      while (w.left > 0 && issued < S) issue(issued++);
      int s = 0;
      uint32_t ph = 1u;
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
    bool dead = !mbar_wait_bounded(x_bar, 0u, failed, p.err, DERR_FULL_WAIT);
    if constexpr (!kIs8) {
      const int nblk = kxs / 32;
      float* cs = reinterpret_cast<float*>(smem + cs_off);
      if (!dead) {
        for (int q = threadIdx.x; q < nblk * CSN; q += 32 * W) {
          const int b = q / CSN, m = q - b * CSN;
          float sum = 0.f;
          if (m < mx) {
            const uint32_t a = smem0 + x_off + (uint32_t)m * x_stride + (uint32_t)b * 64u;
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              const uint4 v = lds128(a + 16u * v4);
              const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) sum += bf16_bits_to_float(wv[i] & 0xFFFFu) + bf16_bits_to_float(wv[i] >> 16);
            }
          }
          cs[q] = -136.0f * sum;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
    }
    const uint32_t xrow = smem0 + x_off + (uint32_t)min(g, mx - 1) * x_stride + 16u * t;   // idle columns read a live row
    const uint32_t csl = smem0 + cs_off + 8u * t;
    const uint32_t wl = smem0 + ring_off + 16u * lane;
    const uint32_t scl = smem0 + ring_off + WB + g * (KIND == Q4_F16 ? 8 : 16);

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    SkWalk w = start;
    int s = 0, buf = 0, pbuf = 0;
    uint32_t ph = 0, rph = 0;
    // (a warp that gives up a wait keeps walking the loop without working or waiting, so that the CTA-wide barrier of
    // the hand-over still sees every warp)
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
            const uint4 xv = lds128(xrow + kco * 256u + 64u * b);
            float part[4];
            uint32_t a_lo[4], a_hi[4];
            if constexpr (kIs8) {
              part[0] = part[1] = part[2] = part[3] = 0.f;
              dequant_i8_words(wlo[2 * b], wlo[2 * b + 1], a_lo);
              dequant_i8_words(whi[2 * b], whi[2 * b + 1], a_hi);
            } else {
              const uint2 cv = lds64(csl + (kco * 4u + b) * (CSN * 4u));
              part[0] = part[2] = __uint_as_float(cv.x);
              part[1] = part[3] = __uint_as_float(cv.y);
              dequant_q4_word_offset(wlo[b], a_lo);
              dequant_q4_word_offset(whi[b], a_hi);
            }
            mma_bf16_16816(part, a_lo[0], a_hi[0], a_lo[1], a_hi[1], xv.x, xv.y);
            mma_bf16_16816(part, a_lo[2], a_hi[2], a_lo[3], a_hi[3], xv.z, xv.w);
            if constexpr (KIND == I8_ROW) {
              acc[0] += part[0];
              acc[1] += part[1];
              acc[2] += part[2];
              acc[3] += part[3];
            } else {
              acc[0] = fmaf(s_lo[b], part[0], acc[0]);
              acc[1] = fmaf(s_lo[b], part[1], acc[1]);
              acc[2] = fmaf(s_hi[b], part[2], acc[2]);
              acc[3] = fmaf(s_hi[b], part[3], acc[3]);
            }
          }
        }
      }
      __syncwarp();
      mbar_arrive_if(&empty_bar[s], lane == 0);
      const bool seg_end = (w.kc + n == skc) || (n == w.left);
      if (seg_end) {
        // hand-over: every warp writes its partial [16][8], the warps meet, each adds up one W-th of the outputs over
        // the warps (in warp order) and the epilogue warp gets the sums (see qgemm_sk.cuh)
        if (!dead && !mbar_wait_spin(&red_empty[buf], rph ^ 1u)) {
          *failed = 1;
          atomicCAS(p.err, 0, (int)DERR_EMPTY_WAIT);
          dead = true;
        }
        float rs0 = 1.f, rs1 = 1.f;
        if constexpr (KIND == I8_ROW) {
          const int r_lo = w.rb * 16 + g;
          rs0 = r_lo < p.n_rows ? row_scales[r_lo] : 0.f;
          rs1 = r_lo + 8 < p.n_rows ? row_scales[r_lo + 8] : 0.f;
        }
        float* part0 = reinterpret_cast<float*>(smem + red_off) + (size_t)pbuf * W * RF;
        pbuf ^= 1;
        float* c = part0 + (size_t)warp * RF + (2 * t) * kSkRedStride + g;
        c[0] = acc[0] * rs0;
        c[8] = acc[2] * rs1;
        c[kSkRedStride] = acc[1] * rs0;
        c[kSkRedStride + 8] = acc[3] * rs1;
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
        if (*failed) dead = true;
        if (lane < 16) {
          const int o = warp * 16 + lane;
          const float* src = part0 + (o >> 4) * kSkRedStride + (o & 15);
          float v = 0.f;
#pragma unroll
          for (int q = 0; q < W; ++q) v += src[q * RF];
          reinterpret_cast<float*>(smem + red_off)[2 * W * RF + buf * 128 + o] = v;
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
  } else {
    // ------------------------------------------------------------------ epilogue warp
    pdl_launch_dependents();
    auto store = [&](int rb, const float (&vals)[NV]) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        const int r = rb * 16 + (idx & 15), m = idx >> 4;
        if (idx < n_out && r < p.n_rows) {
          const size_t o = y_off + (size_t)m * p.ldy + r;
          if (p.y_bf16)
            reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(vals[i]);
          else
            reinterpret_cast<float*>(p.y)[o] = vals[i];
        }
      }
    };
    SkWalk w = start;
    int buf = 0;
    uint32_t rph = 0;
    float held[NV] = {0.f, 0.f, 0.f, 0.f};   // the sums of a first segment that ends its row block: finished at the end
    int held_rb = -1;
    bool good = true;
    while (w.left > 0) {
      const int seg = min(skc - w.kc, w.left);
      const bool whole = (w.kc == 0 && seg == skc);
      const bool to_end = w.kc + seg == skc;
      if (!mbar_wait_bounded(&red_full[buf], rph, failed, p.err, DERR_FULL_WAIT)) {
        good = false;
        break;
      }
      const float* sums = reinterpret_cast<const float*>(smem + red_off) + 2 * W * RF + buf * 128;
      float vals[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) vals[i] = lane + 32 * i < n_out ? sums[lane + 32 * i] : 0.f;
      __syncwarp();
      mbar_arrive_if(&red_empty[buf], lane == 0);
      if (whole) {
        store(w.rb, vals);
      } else if (to_end) {
        held_rb = w.rb;                       // (only a range's first segment starts inside a row block and ends it)
#pragma unroll
        for (int i = 0; i < NV; ++i) held[i] = vals[i];
      } else {
        // the row block goes on in the next CTA: this is the last thing this CTA does
#pragma unroll
        for (int i = 0; i < NV; ++i)
          if (lane + 32 * i < n_out) st_relaxed_u64(p.ws + my_slot + lane + 32 * i, (1ull << 32) | __float_as_uint(vals[i]));
      }
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
    if (good && held_rb >= 0) {
      // the CTAs below that hold the rest of the row block have parked their sums by the time they leave
      const int c_first = (int)((((long long)held_rb * skc + 1) * cps - 1) / U);
      for (int c = c_first; c < j && good; ++c) {
        unsigned long long* part = p.ws + my_slot - (size_t)(j - c) * 128;
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
            atomicCAS(p.err, 0, (int)DERR_PEER_WAIT);
            good = false;
            break;
          }
          __nanosleep(64);
        }
        if (!good) break;
#pragma unroll
        for (int i = 0; i < NV; ++i)
          if (lane + 32 * i < n_out) {
            held[i] += __uint_as_float((uint32_t)got[i]);
            st_relaxed_u64(part + lane + 32 * i, 0ull);   // all zero again for the next launch
          }
      }
      if (good) store(held_rb, held);
    }
  }
}

}  // namespace tq
