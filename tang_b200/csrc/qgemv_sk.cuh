// Weight-only quantised linear layer for 1..8 activation rows (single-token decode): the same
//     y[m, n] = sum_k x[m, k] * q[n, k] * scale[n, k/32]
// as qgemm_mma.cuh (crates/tang-infer/src/quantize.rs:227-289, q8_matvec / q4_matvec), arranged as
// a PERSISTENT kernel whose CTAs share the weight stream evenly:
//   * the matrix is a sequence of units (one 16-row x 128-k fragment tile each, qlayout.cuh) in
//     the order they lie in HBM, [row block][k chunk]; CTA c of the grid owns units
//     [c*U/grid, (c+1)*U/grid) — a contiguous byte range, the same size (+-1 tile) on every SM,
//     so no SM carries a tail.  A row block cut by a range boundary is summed across its CTAs
//     through a small workspace: the higher CTAs park their partial sums (each word carries its own
//     "present" tag) at the start of their range, the lowest one adds them in CTA order at the end
//     of its own (a bounded wait on words written microseconds earlier) and stores, so results are
//     bit-reproducible;
//   * one elected lane streams the range through an S-stage mbarrier ring, ONE bulk (TMA) copy of
//     up to G tiles per stage (L2 evict-first); the first ring-full is requested before
//     griddepcontrol.wait, so under programmatic dependent launch the next layer's weights are
//     already in flight while this layer drains (two CTAs fit on an SM for that reason);
//   * the activation rows are copied to shared memory once per CTA, whole — after
//     griddepcontrol.wait, or, when the host knows that the previous kernel of the stream does not
//     write them (x_early), at entry: the kernel then runs alongside its predecessor and only its
//     stores wait for it;
//   * W consumer warps take the tiles of a stage round-robin.  A lane reads its weights for four
//     32-blocks as two 16-byte vectors, turns each 32-bit word (eight 4-bit codes n = q + 8) into
//     bf16 values 128 + n with one lop3 per pair and feeds mma.sync m16n8k16; the offset is taken
//     out again by the accumulator input of the first MMA of the block, -136 * sum(x over the
//     block), a table every CTA builds once from its copy of x.  The block scale multiplies the f32
//     partial sum.  Integer unpack and products are exact; f32 accumulation rounds;
//   * when a row block's last tile has been consumed the warps hand their partial sums to an
//     epilogue warp through a double-buffered shared array (mbarriers, no CTA-wide barrier), which
//     adds them in warp order and stores y (with the optional residual / 3-term f32 combine).
// Every wait is bounded; a wait that gives up records a code in the context's status word.
#pragma once

#include "common.cuh"
#include "qlayout.cuh"

namespace tq {

struct QGemvParams {
  const uint8_t* tiles;     // fragment tiles, [n_row_blocks][kc_total][tile_bytes]
  const float* row_scales;  // I8_ROW only
  const __nv_bfloat16* x;   // [mx][ldx] bf16, rows 16-byte aligned, kx valid (zero-padded) elements
  void* y;                  // [m_out][ldy] f32 or bf16
  const float* residual;    // optional f32 [m_out][ldy]
  long long ldx, ldy;
  long long n_units;        // n_row_blocks * kc_total
  int n_rows, n_row_blocks, kc_total;
  int kx;                   // kc_total * 128
  int mx, m_out, combine, y_bf16;
  int stages;
  int x_early;              // 1: no kernel that may still be running writes x: load it without waiting;
                            // 2: nor does any of them touch y or the residual, or write x: nothing here waits
                            //    (the workspace pointers below are then this launch's own set)
  // Fused prologue (norm_w != nullptr; x is then not read): the activations are rms_norm(h + delta) * norm_w, formed by
  // every CTA from the f32 residual stream (crates/tang-compute/src/device.rs:546-575, rms_norm_residual), and CTA 0
  // writes h + delta to h_out, a buffer other than h.
  const float* nh;              // [mx][ld_h]
  const float* ndelta;          // optional [mx][ld_h]
  const __nv_bfloat16* norm_w;  // [kx]
  float* nh_out;                // optional [mx][ld_h]
  long long ld_h;
  float norm_eps;
  // The row sums of squares, handed from the projection that wrote the residual stream to the one that normalises it
  // (the several-row kernel only): a kernel with ss_out stores, per 16-row block, the sum of the squares of what it
  // wrote to y (y and the residual included), [m_out][n_row_blocks] floats; a fused prologue with ss_in adds the ss_n
  // partial sums of each row of nh instead of reading the whole row first (ndelta is then null).
  float* ss_out;
  const float* ss_in;
  int ss_n;
  // Fused epilogue: rows 0..7 of every 16-row block are gate rows and rows 8..15 the matching up rows; what is stored
  // is silu(gate) * up (crates/tang-compute/src/device.rs:727-736), n_rows / 2 values per activation row.
  int swiglu;
  // x written by a small staging kernel launched just before this one (host vectors): the word *x_tag becomes x_seq
  // once x is complete.  That kernel waits for nothing, so this one may look at the word instead of waiting for it
  // to finish; null otherwise.
  const unsigned* x_tag;
  unsigned x_seq;
  // Inside a captured graph x_seq is frozen, so the tag also carries the replay count, which a one-thread kernel at
  // the head of the graph advances in *x_epoch (null outside a capture): see sk_x_tag_value.
  const unsigned* x_epoch;
  // the several-row kernel (qgemm_sk.cuh): K is cut into n_slabs slabs of skc chunks, cps CTAs per slab; ws2 holds the
  // slabs' parked sums, [n_slabs][n_row_blocks][column tiles * 128] tagged words, all zero between launches
  int skc, n_slabs, cps;
  unsigned long long* ws2;
  unsigned long long* ws;   // [gridDim.x][2][128] (value bits | 1 << 32): partial sums of row blocks cut by a range
                            // boundary; the tag in the upper half says the value is there; all zero between launches
  int* err;
};

// The tag value that says "slot complete": the call's sequence number with the top bit set, or inside a captured
// graph (epoch != null) the replay count over the low 16 bits of the frozen sequence number (top bit clear, never 0:
// the first replay has count 1).
__host__ __device__ inline unsigned sk_x_tag_value(unsigned seq, const unsigned* epoch) {
  return epoch ? (((*epoch) & 0x7FFFu) << 16) | (seq & 0xFFFFu) : (seq | 0x80000000u);
}

// The 16 lanes that hold one activation row's 16 outputs of a row block add their squares (a fixed tree) and the
// first of them stores the sum to ss[m][rb].  Called by whole warps.
__device__ __forceinline__ void sk_store_sumsq(float* ss, float sq, int lane, int m, int m_out, int n_rb, int rb) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if ((lane & 15) == 0 && m < m_out) ss[(size_t)m * n_rb + rb] = sq;
}

// The sum of a row's n partial sums of squares, the same in every lane and every warp that asks.
__device__ __forceinline__ float sk_load_sumsq(const float* ss, int n, int lane) {
  float a = 0.f;
  for (int k = lane; k < n; k += 32) a += __ldcg(ss + k);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
  return a;
}

constexpr int kSkMaxStages = 12;
constexpr int kSkHeaderBytes = 320;
constexpr int kSkRedStride = 20;   // floats per column in the hand-over array (16 rows + 4: conflict-free)

__host__ __device__ inline int sk_tile_bytes(int kind) { return qk_tile_bytes(kind); }
__host__ __device__ inline int sk_x_stride(int kx) { return kx * 2 + 64; }   // 64 (mod 128): rows g, g+1 on different banks
// Hand-over buffers between the consumer warps and the epilogue warp: one activation row needs 16 floats per
// warp and gets four buffers (a kernel that runs alongside its predecessor may not store until that one has
// finished: its warps can work that many row blocks ahead); up to eight rows need 8 x 20 floats, two buffers.
__host__ __device__ inline int sk_red_bufs(bool m1) { return m1 ? 4 : 2; }
__host__ __device__ inline int sk_red_floats(bool m1) { return m1 ? 16 : 8 * kSkRedStride; }   // per warp and buffer
__host__ __device__ inline int sk_red_bytes(int w, bool m1) { return sk_red_bufs(m1) * w * sk_red_floats(m1) * 4; }
__host__ __device__ inline int sk_csum_bytes(int kind, int kx, bool m1) {
  return (kind == Q4_F32 || kind == Q4_F16) ? (kx / 32) * (m1 ? 2 : 8) * 4 : 0;
}
__host__ __device__ inline size_t sk_fixed_bytes(int kind, int w, int kx, int mx, bool m1) {
  return (size_t)kSkHeaderBytes + sk_red_bytes(w, m1) + (size_t)mx * sk_x_stride(kx) + sk_csum_bytes(kind, kx, m1);
}

// Position of a CTA inside its unit range: the next stage starts at tile (rb, kc); `left` tiles remain.
struct SkWalk {
  int rb, kc, left;
};

// 128 + n for the eight codes of a word, as bf16 pairs in the order dequant_q4_word uses.
__device__ __forceinline__ void dequant_q4_word_offset(uint32_t w, uint32_t (&out)[4]) {
  constexpr uint32_t kMask = 0x000F000Fu, kMagic = 0x43004300u;
  out[0] = lop3_and_or(w, kMask, kMagic);
  // (the shifts as upper halves of multiplications, to move them off the half-rate ALU pipe, measured slower:
  // 5.8 -> 7.8 us per launch)
  out[1] = lop3_and_or(w >> 4, kMask, kMagic);
  out[2] = lop3_and_or(w >> 8, kMask, kMagic);
  out[3] = lop3_and_or(w >> 12, kMask, kMagic);
}

__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

template <int KIND, int W, int TPW, bool M1, int MINB = 2>
__global__ void __launch_bounds__(32 * (W + 2), MINB) qgemv_sk_kernel(const QGemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool kIs8 = (KIND == Q8_F32 || KIND == I8_ROW);
  constexpr int TB = kIs8 ? (KIND == I8_ROW ? 2048 : 2304) : (KIND == Q4_F16 ? 1152 : 1280);
  constexpr int WB = kIs8 ? 2048 : 1024;
  constexpr int G = W * TPW;          // tiles per stage
  constexpr int CS = M1 ? 2 : 8;      // floats per block in the offset table

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kSkMaxStages;
  uint64_t* x_bar = empty_bar + kSkMaxStages;
  constexpr int NBUF = M1 ? 4 : 2;    // hand-over buffers (sk_red_bufs)
  constexpr int RF = M1 ? 16 : 8 * kSkRedStride;   // floats per warp and buffer (sk_red_floats)
  uint64_t* red_full = x_bar + 1;     // [NBUF]
  uint64_t* red_empty = red_full + 4; // [NBUF]
  volatile int* failed = reinterpret_cast<volatile int*>(red_empty + 4);

  const int S = p.stages;
  const int x_stride = sk_x_stride(p.kx);
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t red_off = kSkHeaderBytes;
  const uint32_t x_off = red_off + sk_red_bytes(W, M1);
  const uint32_t cs_off = x_off + (uint32_t)p.mx * x_stride;
  const uint32_t ring_off = cs_off + sk_csum_bytes(KIND, p.kx, M1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long U = p.n_units;
  const long long u0 = U * blockIdx.x / gridDim.x, u1 = U * (blockIdx.x + 1) / gridDim.x;
  SkWalk start;
  start.rb = (int)(u0 / p.kc_total);
  start.kc = (int)(u0 - (long long)start.rb * p.kc_total);
  start.left = (int)(u1 - u0);

  // A kernel that does not read what its predecessors write lets the next kernel of the stream be scheduled at
  // once (any number of such kernels then stream their weights side by side); its own stores still wait below.
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

  if (warp == W) {
    // ------------------------------------------------------------------ producer (one lane)
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const uint8_t* src = p.tiles + (size_t)u0 * TB;
      SkWalk w = start;
      auto issue = [&](int s) {
        const int n = min(G, min(p.kc_total - w.kc, w.left));
        const uint32_t bytes = (uint32_t)n * TB;
        mbar_arrive_expect_tx(&full_bar[s], bytes);
        bulk_g2s(smem + ring_off + (size_t)s * (G * TB), src, bytes, &full_bar[s], pol_w);
        src += bytes;
        w.left -= n;
        w.kc += n;
        if (w.kc == p.kc_total) {
          w.kc = 0;
          ++w.rb;
        }
      };
      auto load_x = [&]() {
        mbar_arrive_expect_tx(x_bar, (uint32_t)p.mx * (uint32_t)p.kx * 2u);
        for (int m = 0; m < p.mx; ++m)
          bulk_g2s(smem + x_off + (size_t)m * x_stride, p.x + (size_t)m * p.ldx, (uint32_t)p.kx * 2u, x_bar, pol_x);
      };
      // The weights never depend on the previous kernel of the stream; the activations usually do.
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
      // ---- fused rms_norm_residual: two passes over h (+ delta), both from L2; every CTA forms the same activations
      if (p.x_early == 0) pdl_wait();          // h and delta are the previous kernels' outputs
      float* scratch = reinterpret_cast<float*>(smem + red_off);   // the hand-over buffers are idle until the first flush
      const int nthr = 32 * W;
      for (int m = 0; m < p.mx; ++m) {
        const float* hrow = p.nh + (size_t)m * p.ld_h;
        const float* drow = p.ndelta ? p.ndelta + (size_t)m * p.ld_h : nullptr;
        float sq = 0.f;
        for (int k = 4 * threadIdx.x; k < p.kx; k += 4 * nthr) {
          float4 v = __ldcg(reinterpret_cast<const float4*>(hrow + k));
          if (drow) {
            const float4 d = __ldcg(reinterpret_cast<const float4*>(drow + k));
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
          }
          sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        sq = warp_sum(sq);
        if (lane == 0) scratch[warp] = sq;
        asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
        float total = 0.f;
#pragma unroll
        for (int q = 0; q < W; ++q) total += scratch[q];
        asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");   // (scratch is reused by the next row)
        const float inv = 1.0f / sqrtf(total / (float)p.kx + p.norm_eps);
        uint8_t* xrow_s = smem + x_off + (size_t)m * x_stride;
        for (int k = 4 * threadIdx.x; k < p.kx; k += 4 * nthr) {
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
          *reinterpret_cast<uint2*>(xrow_s + 2 * k) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
          if (p.nh_out && blockIdx.x == 0) *reinterpret_cast<float4*>(p.nh_out + (size_t)m * p.ld_h + k) = v;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
    } else {
      ok = mbar_wait_bounded(x_bar, 0u, failed, p.err, DERR_FULL_WAIT);
    }
    if constexpr (!kIs8) {
      // offset table: -136 * (sum of the block's 32 activations), per activation row
      const int nblk = p.kx / 32;
      float* cs = reinterpret_cast<float*>(smem + cs_off);
      if (ok) {
        for (int e = threadIdx.x; e < nblk * CS; e += 32 * W) {
          const int b = e / CS, m = e - b * CS;
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

    const uint32_t xrow = smem0 + x_off + (uint32_t)min(g, p.mx - 1) * x_stride + 16u * t;  // idle columns read a live row
    const uint32_t csl = smem0 + cs_off + (M1 ? 0u : 8u * t);
    const uint32_t wl = smem0 + ring_off + 16u * lane;
    const uint32_t scl = smem0 + ring_off + WB + g * (KIND == Q4_F16 ? 8 : 16);

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    SkWalk w = start;
    int s = 0, buf = 0;
    uint32_t ph = 0, rph = 0;
    while (ok && w.left > 0) {
      const int n = min(G, min(p.kc_total - w.kc, w.left));
      if (!mbar_wait_spin(&full_bar[s], ph)) {
        *failed = 1;
        atomicCAS(p.err, 0, (int)DERR_FULL_WAIT);
        break;
      }
      const uint32_t st = (uint32_t)s * (G * TB);
#pragma unroll
      for (int j = 0; j < TPW; ++j) {
        const int i = warp + j * W;
        if (i < n) {
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
              const uint2 cv = lds64(csl + (kco * 4u + b) * (CS * 4u));
              part[0] = part[2] = __uint_as_float(cv.x);
              part[1] = part[3] = __uint_as_float(cv.y);
              dequant_q4_word_offset(wlo[b], a_lo);
              dequant_q4_word_offset(whi[b], a_hi);
            }
            mma_bf16_16816(part, a_lo[0], a_hi[0], a_lo[1], a_hi[1], xv.x, xv.y);
            mma_bf16_16816(part, a_lo[2], a_hi[2], a_lo[3], a_hi[3], xv.z, xv.w);
            if constexpr (KIND == I8_ROW) {
              acc[0] += part[0];
              acc[2] += part[2];
              if constexpr (!M1) {
                acc[1] += part[1];
                acc[3] += part[3];
              }
            } else {
              acc[0] = fmaf(s_lo[b], part[0], acc[0]);
              acc[2] = fmaf(s_hi[b], part[2], acc[2]);
              if constexpr (!M1) {
                acc[1] = fmaf(s_lo[b], part[1], acc[1]);
                acc[3] = fmaf(s_hi[b], part[3], acc[3]);
              }
            }
          }
        }
      }
      __syncwarp();
      mbar_arrive_if(&empty_bar[s], lane == 0);
      const bool seg_end = (w.kc + n == p.kc_total) || (n == w.left);
      if (seg_end) {
        // hand this row block's partial sums to the epilogue warp
        if (!mbar_wait_spin(&red_empty[buf], rph ^ 1u)) {
          *failed = 1;
          atomicCAS(p.err, 0, (int)DERR_EMPTY_WAIT);
          break;
        }
        if constexpr (KIND == I8_ROW) {
          const int r_lo = w.rb * 16 + g;
          const float rs0 = r_lo < p.n_rows ? p.row_scales[r_lo] : 0.f;
          const float rs1 = r_lo + 8 < p.n_rows ? p.row_scales[r_lo + 8] : 0.f;
          acc[0] *= rs0;
          acc[1] *= rs0;
          acc[2] *= rs1;
          acc[3] *= rs1;
        }
        float* red = reinterpret_cast<float*>(smem + red_off) + ((size_t)buf * W + warp) * RF;
        if constexpr (M1) {
          if (t == 0) {           // column 0 lives in the lanes with t = 0
            red[g] = acc[0];
            red[g + 8] = acc[2];
          }
        } else {
          red[(2 * t) * kSkRedStride + g] = acc[0];
          red[(2 * t) * kSkRedStride + g + 8] = acc[2];
          red[(2 * t + 1) * kSkRedStride + g] = acc[1];
          red[(2 * t + 1) * kSkRedStride + g + 8] = acc[3];
        }
        __syncwarp();
        mbar_arrive_if(&red_full[buf], lane == 0);
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        if (++buf == NBUF) {
          buf = 0;
          rph ^= 1u;
        }
      }
      w.left -= n;
      w.kc += n;
      if (w.kc == p.kc_total) {
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
    // y, the residual and the workspace belong to earlier kernels until griddepcontrol.wait returns — unless the
    // host has checked that no kernel still running touches them (x_early == 2).  A kernel that had to wait for
    // its activations lets the next one be scheduled only now, so that whatever runs beside a later kernel is
    // either complete or one of the independent kernels the host keeps track of.
    if (p.x_early < 2) pdl_wait();
    if (!p.x_early) pdl_launch_dependents();
    const int n_out = p.m_out * 16;            // (row, output row of x) pairs of a row block, <= 128
    const long long grid = gridDim.x;
    auto store = [&](int rb, const float (&vals)[4]) {
      if (p.swiglu) {
        // rows 0..7 of the block hold gate values, rows 8..15 the up values of the same eight outputs
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = lane + 32 * i;
          const float up = __shfl_down_sync(0xffffffffu, vals[i], 8);    // lane l + 8 holds row (l & 15) + 8 of the same m
          const int r8 = idx & 15, m = idx >> 4;
          const int o_col = rb * 8 + r8;
          if (idx < n_out && r8 < 8 && o_col < p.n_rows / 2) {
            const float g = vals[i];
            const float act = g * (1.0f / (1.0f + expf(-g))) * up;   // the formula of swiglu_kernel, term for term
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
      for (int i = 0; i < 4; ++i) {
        const int idx = lane + 32 * i;
        const int r = rb * 16 + (idx & 15), m = idx >> 4;
        if (idx < n_out && r < p.n_rows) {
          const size_t o = (size_t)m * p.ldy + r;
          float v = vals[i];
          if (p.residual) v += p.residual[o];
          if (p.y_bf16)
            reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
          else
            reinterpret_cast<float*>(p.y)[o] = v;
        }
      }
    };
    // A row block cut by range boundaries belongs to CTAs c_first..c_last.  The higher ones park their partial
    // sums in the workspace (the block is the first thing they work on); the lowest one, for
    // which the block is the LAST segment of its range, finishes it: it fetches the parked partials while its own
    // warps still compute (from three row blocks before the end, without blocking until the very end).
    const long long last_u = u1 - 1;
    const int last_rb = (int)(last_u / p.kc_total);
    const long long last_ub = (long long)last_rb * p.kc_total;
    const bool last_cut = u1 != last_ub + p.kc_total;                      // the range ends inside a row block
    const bool finisher = last_cut && (int)(((last_ub + 1) * grid - 1) / U) == (int)blockIdx.x;
    const int fin_last = finisher ? (int)(((last_ub + p.kc_total) * grid - 1) / U) : 0;
    float others[4] = {0.f, 0.f, 0.f, 0.f};
    bool fetched = !finisher;
    auto peer_slot = [&](int c) {
      const int c_rb0 = (int)((U * c / grid) / p.kc_total);   // first row block of CTA c
      return c * 2 + (c_rb0 == last_rb ? 0 : 1);
    };
    // A parked partial is 128 words of (value bits | tag << 32), each written with one 64-bit store: a word is
    // there when its tag is, so neither side needs a fence or a separate flag, and the reader clears what it took.
    int next_peer = (int)blockIdx.x + 1;
    auto fetch_peers = [&](bool blocking) -> bool {            // false: gave up (only when blocking)
      while (next_peer <= fin_last) {
        unsigned long long* part = p.ws + (size_t)peer_slot(next_peer) * 128;
        unsigned long long got[4];
        uint32_t polls = 0;
        for (;;) {
          bool ready = true;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            got[i] = 1ull << 32;
            if (lane + 32 * i < n_out) got[i] = ld_relaxed_u64(part + lane + 32 * i);
            ready = ready && (got[i] >> 32) != 0;
          }
          if (__all_sync(0xffffffffu, ready)) break;
          if (!blocking) return true;                           // not there yet: try again later
          if (++polls > kMaxPolls || *failed) return false;
          __nanosleep(32);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (lane + 32 * i < n_out) {
            others[i] += __uint_as_float((uint32_t)got[i]);     // higher k ranges in CTA order
            st_relaxed_u64(part + lane + 32 * i, 0ull);         // ready for the next launch that uses this set
          }
        ++next_peer;
      }
      fetched = true;
      return true;
    };
    SkWalk w = start;
    int buf = 0;
    uint32_t rph = 0;
    bool first_seg = true;
    while (w.left > 0) {
      const int seg = min(p.kc_total - w.kc, w.left);
      const bool whole = (w.kc == 0 && seg == p.kc_total);
      const bool is_last = seg == w.left;
      if (!fetched && w.left <= 3 * p.kc_total) {
        if (!fetch_peers(is_last)) {
          *failed = 1;
          atomicCAS(p.err, 0, (int)DERR_PEER_WAIT);
          break;
        }
      }
      if (!mbar_wait_bounded(&red_full[buf], rph, failed, p.err, DERR_FULL_WAIT)) break;
      const float* red = reinterpret_cast<const float*>(smem + red_off) + (size_t)buf * W * RF;
      float vals[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = lane + 32 * i;
        float v = 0.f;
        if (idx < n_out) {
          const int r = idx & 15, m = idx >> 4;
          if constexpr (M1) {
#pragma unroll
            for (int q = 0; q < W; ++q) v += red[q * RF + r];
          } else {
            for (int c = 0; c < p.combine; ++c) {
              const float* col = red + (m * p.combine + c) * kSkRedStride + r;
#pragma unroll
              for (int q = 0; q < W; ++q) v += col[q * RF];
            }
          }
        }
        vals[i] = v;
      }
      __syncwarp();
      mbar_arrive_if(&red_empty[buf], lane == 0);
      if (whole) {
        store(w.rb, vals);
      } else if (is_last && finisher) {
#pragma unroll
        for (int i = 0; i < 4; ++i) vals[i] += others[i];   // own k range first, then the higher ones in CTA order
        store(w.rb, vals);
      } else {
        const int slot = (int)blockIdx.x * 2 + (first_seg ? 0 : 1);
        unsigned long long* mine = p.ws + (size_t)slot * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (lane + 32 * i < n_out) st_relaxed_u64(mine + lane + 32 * i, (1ull << 32) | __float_as_uint(vals[i]));
      }
      first_seg = false;
      w.left -= seg;
      w.kc += seg;
      if (w.kc == p.kc_total) {
        w.kc = 0;
        ++w.rb;
      }
      if (++buf == NBUF) {
        buf = 0;
        rph ^= 1u;
      }
    }
    if (p.x_early == 2) pdl_wait();   // kernels of a stream still complete in launch order
  }
}

}  // namespace tq
