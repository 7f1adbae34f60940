// tcgen05 / tensor-memory dequant-GEMM: kernel and launcher (see qgemm_umma.cuh for the design).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "qgemm_umma.cuh"

namespace tq {

template <int KIND, int TERMS, bool TS = false, bool DUAL = false>
__global__ void __launch_bounds__(kUmmaThreads, 1)
qgemm_umma_kernel(const __grid_constant__ CUtensorMap x_map, const UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int TB = (KIND == I8_ROW) ? 2048 : (KIND == Q8_F32) ? 2304 : (KIND == Q4_F16) ? 1152 : 1280;
  constexpr bool kIs8 = KIND == I8_ROW || KIND == Q8_F32;
  static_assert(KIND != I8_ROW || TERMS == 1, "int8 rows carry no scale into the operand: one exact term");
  // DUAL: the CTA covers two token tiles of p.ntok rows with one conversion of the weights: issuer warp 1 multiplies
  // every stage with the first tile's activations, warp 3 with the second tile's, each into one accumulator
  static_assert(!DUAL || (TS && TERMS == 1), "two token tiles per CTA: single-term weights in tensor memory");
  constexpr int kTokTiles = DUAL ? 2 : 1;
  constexpr int kMaxStages = 6;
  // ---- shared-memory carve-up (operand tiles need 1024-byte alignment for the 128-byte swizzle)
  uint8_t* smem = smem_raw;
  uint64_t* x_full = reinterpret_cast<uint64_t*>(smem);       // [stages] activation box landed
  uint64_t* a_full = x_full + kMaxStages;                      // [stages] A tiles written (one arrival per dequant warp)
  uint64_t* empty = a_full + kMaxStages;                       // [stages] MMAs of the stage retired
  uint64_t* raw_full = empty + kMaxStages;                     // [raw stages] packed tiles landed
  uint64_t* raw_empty = raw_full + kUmmaMaxRawStages;             // [raw stages] packed tiles consumed (one arrival per dequant warp)
  uint64_t* acc_full = raw_empty + kUmmaMaxRawStages;             // accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t base_u32 = smem_u32(smem_raw);
  uint8_t* tiles_s = smem_raw + kUmmaHeader + ((1024 - ((base_u32 + kUmmaHeader) & 1023)) & 1023);  // 1024-aligned
  const size_t stage_bytes = umma_stage_bytes(TERMS, p.ntok, TS ? 1 : 0) * kTokTiles;
  constexpr int kBOff = TS ? 0 : TERMS * kUmmaRows * 128;   // the activation box inside a stage
  uint8_t* raw_s = tiles_s + (size_t)p.stages * stage_bytes;   // [raw stages][8 tiles]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages, RS = p.raw_stages, KT = p.kt;
  const int rb0 = blockIdx.x * (kUmmaRows / kTileRows);        // first 16-row block
  int m0 = blockIdx.y * p.ntok * kTokTiles;                    // first token of this CTA
  int m_end = p.m_total;                                       // rows at or beyond this are not this CTA's to store
  const uint8_t* tile_base = p.tiles;
  const float* row_scales = p.row_scales;   // TQ_I8_ROW: per output row, applied to the accumulator
  if (p.g_counts) {
    // grouped (experts): blockIdx.z picks the group, whose rows are g_offsets[e] .. +g_counts[e] of x and y and
    // whose weights start g_tile_stride bytes further on; token tiles beyond the group's rows leave at once
    pdl_wait();
    int e = blockIdx.z;
    if (p.g_active) {
      e = p.g_active[e];
      if (e < 0) return;
    }
    const int cnt = p.g_counts[e];
    if (m0 >= cnt) return;
    m_end = p.g_offsets[e] + cnt;
    m0 += p.g_offsets[e];
    tile_base += (size_t)e * p.g_tile_stride;
    row_scales += (size_t)e * p.n_rows;
  }
  const int kc_begin = p.g_counts ? 0 : blockIdx.z * p.kc_per_split;   // this CTA's slice of K, in 128-k tiles
  const int kc_len = min(p.kc_per_split, p.kc_total - kc_begin);
  const int n_kb = kc_len * 2;                                 // 64-k steps

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&a_full[s], kUmmaGroupWarps);
      mbar_init(&empty[s], DUAL ? 2 : 1);   // one commit per issuer that reads the stage
    }
    for (int r = 0; r < RS; ++r) {
      mbar_init(&raw_full[r], 1);
      mbar_init(&raw_empty[r], kUmmaDqWarps);          // every group reads some tile of every ring slot
    }
    mbar_init(acc_full, 2);
    *failed = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;

  pdl_wait();
  pdl_launch_dependents();

  auto give_up = [&](int code) {
    *failed = 1;
    atomicCAS(p.err, 0, code);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ packed-weight producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      int r = 0;
      uint32_t rph = 0;
      // one ring slot = KT consecutive k-tiles of the CTA's eight row blocks: eight copies of KT tiles each (the
      // copy engine takes about as long over one tile as over four, so small copies cannot keep up with HBM)
      for (int t0 = 0; t0 < kc_len && !*failed; t0 += KT) {
        const uint32_t kcs = (uint32_t)min(KT, kc_len - t0);
        if (!mbar_wait_spin(&raw_empty[r], rph ^ 1u)) { give_up(DERR_EMPTY_WAIT); break; }
        mbar_arrive_expect_tx(&raw_full[r], 8u * kcs * TB);
        for (int i = 0; i < 8; ++i)
          bulk_g2s(raw_s + ((size_t)(r * 8 + i) * KT) * TB, tile_base + ((size_t)(rb0 + i) * p.kc_total + kc_begin + t0) * TB,
                   kcs * TB, &raw_full[r], pol_w);
        if (++r == RS) {
          r = 0;
          rph ^= 1u;
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ activation producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int kb = 0; kb < n_kb && !*failed; ++kb) {
        if (!mbar_wait_spin(&empty[s], ph ^ 1u)) { give_up(DERR_EMPTY_WAIT); break; }
        mbar_arrive_expect_tx(&x_full[s], (uint32_t)(p.ntok * kTokTiles) * 128u);
        tma_load_2d(tiles_s + (size_t)s * stage_bytes + (size_t)kBOff, &x_map,
                    (kc_begin * 2 + kb) * kUmmaK, m0, &x_full[s]);
        if constexpr (DUAL)     // (rows beyond the matrix read as zeros, a box entirely beyond it too)
          tma_load_2d(tiles_s + (size_t)s * stage_bytes + (size_t)p.ntok * 128, &x_map, (kc_begin * 2 + kb) * kUmmaK,
                      m0 + p.ntok, &x_full[s]);
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------------------------------------------ MMA issuers
    // Two of them: issuing one step's MMAs from a single thread (~55 cycles each, plus the waits and the
    // commit) is what bounds the step time, so warp 1 takes the even steps into the even accumulators and warp 3
    // the odd steps into the odd ones; the epilogue adds them all (a fixed order: reproducible).  With an
    // even ring depth each issuer only ever returns to slots it consumed itself.
    // The whole warp runs the loop (warp-uniform control flow keeps the descriptors in uniform
    // registers); one elected lane issues.  The barriers of the NEXT step are looked at before this
    // step's instructions are issued, so that the answer is there when the loop comes round.
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(p.ntok);
    const uint64_t desc0 = umma_desc_sw128(tiles_s);
    const uint32_t stage_u = (uint32_t)(stage_bytes >> 4), b_off_u = (uint32_t)(kBOff >> 4);
    bool ok = true;
    const int odd = warp == 3;
    // Each issuer rotates over n_acc / 2 accumulators: the tensor core truncates every f32 addition, an error that
    // grows with the number of additions one accumulator sees, so as many short sums as tensor memory holds
    // (512 columns) are kept and the epilogue adds them, in accumulator order.
    const int rot_mask = (p.n_acc >> 1) - 1;
    int j = 0;                                  // this issuer's step count
    constexpr int kStep = DUAL ? 1 : 2;         // (two token tiles: every issuer takes every step)
    int s = DUAL ? 0 : odd;
    uint32_t ph = 0;
    uint32_t tok_x = mbar_test(&x_full[s], 0), tok_a = mbar_test(&a_full[s], 0);
    const uint32_t tile_off_u = DUAL ? (uint32_t)odd * (uint32_t)((p.ntok * 128) >> 4) : 0u;
#pragma unroll 1
    for (int kb = DUAL ? 0 : odd; kb < n_kb; kb += kStep) {
      ok = !*failed && mbar_wait_token(&x_full[s], ph, tok_x) && mbar_wait_token(&a_full[s], ph, tok_a);
      if (!ok) { give_up(DERR_FULL_WAIT); break; }
      tc_fence_after();
      const uint64_t ad = desc0 + (uint64_t)((uint32_t)s * stage_u);
      const int s_cur = s;
      s += kStep;
      if (s >= S) {
        s -= S;
        ph ^= 1u;
      }
      const uint32_t acc = tmem_d + (uint32_t)((DUAL ? odd : odd + 2 * (j & rot_mask)) * p.acc_stride);
      const uint32_t fresh = (DUAL ? j == 0 : j <= rot_mask) ? 0u : 1u;   // the accumulator's first step overwrites it
      ++j;
      if (leader) {
#pragma unroll
        for (int k16 = 0; k16 < kUmmaK / 16; ++k16) {
          const uint64_t bd = ad + b_off_u + tile_off_u + 2 * k16;
          if constexpr (TS) {
            // the stage's weights sit in tensor memory: 32 columns (64 k) of the hi term, then 32 of the lo term
            const uint32_t a_t = tmem_d + (uint32_t)(p.a_col0 + s_cur * (32 * TERMS) + 8 * k16);
            umma_f16_ts(acc, a_t, bd, idesc, fresh | (k16 != 0));
            if (TERMS == 2) umma_f16_ts(acc, a_t + 32u, bd, idesc, 1u);
          } else {
            umma_f16(acc, ad + 2 * k16, bd, idesc, fresh | (k16 != 0));
            if (TERMS == 2) umma_f16(acc, ad + (kUmmaRows * 128 >> 4) + 2 * k16, bd, idesc, 1u);
          }
        }
      }
      if (leader) umma_commit(&empty[s_cur]);   // arrives when the MMAs above have finished reading the stage
      __syncwarp();
      // Look at the next step's barriers only now: the answer takes ~70 cycles, during which an in-order
      // thread issues nothing, and here the tensor core already has this step's work.
      tok_x = mbar_test(&x_full[s], ph);
      tok_a = mbar_test(&a_full[s], ph);
    }
    if (leader) umma_commit(acc_full);           // arrives when every MMA issued so far has completed
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ dequant warps
    // Everything that does not change from step to step (which words of the packed tiles this thread
    // converts, where their scales sit, where the result goes in the swizzled A tile) is computed once.
    // The dequant warps form kUmmaGroups groups; group g produces the stages kb = g, g + G, g + 2G, ...
    // so that G stages are being converted at any time (one stage's chain of waits, loads, arithmetic,
    // stores and fence is long; the groups overlap it).  G is even, so a group always reads the same
    // half (c = g & 1) of its 128-k packed tiles.
    const int group = (warp - kUmmaFirstDqWarp) / kUmmaGroupWarps;
    const int tid = threadIdx.x - 32 * kUmmaFirstDqWarp - group * 32 * kUmmaGroupWarps;
    constexpr int kCombos = 512 / (32 * kUmmaGroupWarps);
    int src_off[kCombos], sc_off[kCombos], dst_off[kCombos][2];
#pragma unroll
    for (int i = 0; i < kCombos; ++i) {
      const int combo = tid + 32 * kUmmaGroupWarps * i;            // (row block, half, lane of the tile layout)
      const int rbi = combo >> 6, h = (combo >> 5) & 1, L = combo & 31;
      const int g = L >> 2, t = L & 3;
      const int row = rbi * 16 + g + 8 * h;
      src_off[i] = rbi * KT * TB + (kIs8 ? h * 1024 : h * 512) + 16 * L;
      sc_off[i] = rbi * KT * TB + (kIs8 ? 2048 : 1024) + (KIND == Q4_F16 ? h * 64 + g * 8 : h * 128 + g * 16);
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) dst_off[i][jj] = row * 128 + (((4 * jj + t) ^ (row & 7)) << 4);
    }
    bool ok = true;
    const int c = group & 1;                                    // which 64-k half of the 128-k tile
    int s = group, r = 0, within = group >> 1;                   // A/B slot; packed-tile slot and the tile inside it
    uint32_t ph = 0, rph = 0;
    while (s >= S) {
      s -= S;
      ph ^= 1u;
    }
    uint32_t tok_raw = mbar_test(&raw_full[r], rph), tok_empty = mbar_test(&empty[s], ph ^ 1u);
#pragma unroll 1
    for (int kb = group; kb < n_kb && ok; kb += kUmmaGroups) {
      // (with two terms in tensor memory the stage is only waited for when the first half of the row is converted:
      // the MMAs that last read it have that long to finish -- decode step at batch 64 8.27 -> 8.11 ms; with one term
      // the conversion is too short for that and the early wait measured 3 % better)
      constexpr bool kLateWait = TS && TERMS == 2;
      ok = !*failed && mbar_wait_token(&raw_full[r], rph, tok_raw) && (kLateWait || mbar_wait_token(&empty[s], ph ^ 1u, tok_empty));
      if (!ok) { give_up(DERR_FULL_WAIT); break; }
      const int s_cur = s, r_cur = r, within_cur = within;
      const uint32_t ph_cur = ph;
      s += kUmmaGroups;
      while (s >= S) {
        s -= S;
        ph ^= 1u;
      }
      within += kUmmaGroups / 2;                  // this group's next tile: two further on
      const bool leaves = within >= KT;           // ... which lies in the next ring slot (KT is 2 or 4)
      if (leaves) {
        within -= KT;
        if (++r == RS) {
          r = 0;
          rph ^= 1u;
        }
      }
      uint8_t* a_hi = tiles_s + (size_t)s_cur * stage_bytes;
      uint8_t* a_lo = a_hi + kUmmaRows * 128;
      const uint8_t* raw = raw_s + ((size_t)r_cur * 8 * KT + within_cur) * TB;
      if constexpr (TS) {
        // ---- weights to tensor memory: this thread owns output row 32 * (warp % 4) + lane, i.e. that lane, and
        // converts the row's 64 k of the stage.  In a fragment tile the row's nibbles are 64 contiguous bytes (its
        // four k quarters of 16 bytes, each holding one word per 32-block), its scales 8 or 16 contiguous bytes.
        if (!kLateWait) tc_fence_after();          // the stage's columns were last read by MMAs whose commit was waited for
        const int q4 = warp & 3;
        const int rbi = 2 * q4 + (lane >> 4), h = (lane >> 3) & 1, g = lane & 7;
        const uint8_t* wrow = raw + rbi * KT * TB + (kIs8 ? h * 1024 + 512 * c : h * 512 + 8 * c) + g * 64;
        const uint32_t a_t = tmem_d + ((uint32_t)(32 * q4) << 16) + (uint32_t)(p.a_col0 + s_cur * (32 * TERMS));
        uint32_t sh = 0, sl = 0;
        if constexpr (KIND != I8_ROW) {
          const uint8_t* srow = raw + rbi * KT * TB + (kIs8 ? 2048 : 1024);
          float2 f;
          if (KIND == Q4_F16) f = __half22float2(*reinterpret_cast<const __half2*>(srow + h * 64 + g * 8 + 4 * c));
          else f = *reinterpret_cast<const float2*>(srow + h * 128 + g * 16 + 8 * c);
          const __nv_bfloat162 shb = __floats2bfloat162_rn(f.x, f.y);
          sh = *reinterpret_cast<const uint32_t*>(&shb);
          const __nv_bfloat162 slb = __floats2bfloat162_rn(f.x - __uint_as_float(sh << 16), f.y - __uint_as_float(sh & 0xFFFF0000u));
          sl = *reinterpret_cast<const uint32_t*>(&slb);
        }
        uint32_t wq[4][4];                         // [k quarter][word]: Q4 uses words 0, 1 (blocks 2c, 2c+1)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          if constexpr (kIs8) {
            const uint4 v = *reinterpret_cast<const uint4*>(wrow + 16 * t);
            wq[t][0] = v.x; wq[t][1] = v.y; wq[t][2] = v.z; wq[t][3] = v.w;
          } else {
            const uint2 v = *reinterpret_cast<const uint2*>(wrow + 16 * t);
            wq[t][0] = v.x; wq[t][1] = v.y; wq[t][2] = 0u; wq[t][3] = 0u;
          }
        }
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          uint32_t hi[16], lo[16];
          const uint32_t s_hi = prmt(sh, sh, jj ? 0x3232u : 0x1010u), s_lo = prmt(sl, sl, jj ? 0x3232u : 0x1010u);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint32_t q[4];                         // (k0,k1) (k2,k3) (k4,k5) (k6,k7) of k quarter t, exact ints
            if constexpr (kIs8) dequant_i8_words(wq[t][2 * jj], wq[t][2 * jj + 1], q);
            else dequant_q4_word(wq[t][jj], q);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if constexpr (KIND == I8_ROW) {
                hi[4 * t + e] = q[e];
              } else {
                const uint32_t tt = bf16x2_mul(q[e], s_lo);
                hi[4 * t + e] = bf16x2_fma(q[e], s_hi, tt);
                if (TERMS == 2) lo[4 * t + e] = bf16x2_add(bf16x2_fma(q[e], s_hi, hi[4 * t + e] ^ 0x80008000u), tt);
              }
            }
          }
          if (kLateWait && jj == 0) {
            // the stage's columns were last read by MMAs whose commit is waited for here
            ok = __all_sync(0xffffffffu, mbar_wait_token(&empty[s_cur], ph_cur ^ 1u, tok_empty));
            tc_fence_after();
          }
          if (ok) {
            tmem_st16(a_t + (uint32_t)(16 * jj), hi);
            if (TERMS == 2) tmem_st16(a_t + (uint32_t)(32 + 16 * jj), lo);
          }
        }
        if (!ok) { give_up(DERR_EMPTY_WAIT); break; }
        tmem_st_wait();
        tc_fence_before();
      } else {
#pragma unroll
      for (int i = 0; i < kCombos; ++i) {
        if constexpr (KIND == I8_ROW) {
          // int8 with one scale per output row: the integers go into the operand as they are (exact in bf16) and the
          // row scale multiplies the accumulator in the epilogue -- an exact product with a single term
          const uint4 w4 = *reinterpret_cast<const uint4*>(raw + src_off[i] + 512 * c);   // [even k | odd k] of blocks 2c, 2c+1
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            uint32_t q[4];
            dequant_i8_words(jj ? w4.z : w4.x, jj ? w4.w : w4.y, q);
            *reinterpret_cast<uint4*>(a_hi + dst_off[i][jj]) = make_uint4(q[0], q[1], q[2], q[3]);
          }
          continue;
        }
        // blocks 2c, 2c+1: eight nibbles per word (Q4), or the [even k | odd k] byte planes of both blocks (Q8)
        uint2 w2 = make_uint2(0u, 0u);
        uint4 w8 = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (KIND == Q8_F32) w8 = *reinterpret_cast<const uint4*>(raw + src_off[i] + 512 * c);
        else w2 = *reinterpret_cast<const uint2*>(raw + src_off[i] + 8 * c);
        // The scale as s_hi + s_lo, two bf16 numbers (exact for an f16 scale: 11 = 8 + 3 significant bits).
        // With t = q*s_lo (7 bits, exact in bf16), hi = fma(q, s_hi, t) is the exact product rounded once;
        // lo = fma(q, s_hi, -hi) + t = q*scale - hi, both steps exact, so hi + lo reproduces the product.
        // (f32 scales keep their first 16 significant bits this way, and with int8 values t itself is rounded to 8
        // bits: hi + lo is then the product to within 2^-15 relative.)
        float2 f;
        if (KIND == Q4_F16) f = __half22float2(*reinterpret_cast<const __half2*>(raw + sc_off[i] + 4 * c));
        else f = *reinterpret_cast<const float2*>(raw + sc_off[i] + 8 * c);
        const __nv_bfloat162 shb = __floats2bfloat162_rn(f.x, f.y);
        const uint32_t sh = *reinterpret_cast<const uint32_t*>(&shb);
        const __nv_bfloat162 slb = __floats2bfloat162_rn(f.x - __uint_as_float(sh << 16), f.y - __uint_as_float(sh & 0xFFFF0000u));
        const uint32_t sl = *reinterpret_cast<const uint32_t*>(&slb);
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const uint32_t s_hi = prmt(sh, sh, jj ? 0x3232u : 0x1010u), s_lo = prmt(sl, sl, jj ? 0x3232u : 0x1010u);
          uint32_t q[4];
          // (k0,k1) (k2,k3) (k4,k5) (k6,k7), exact ints
          if constexpr (KIND == Q8_F32) dequant_i8_words(jj ? w8.z : w8.x, jj ? w8.w : w8.y, q);
          else dequant_q4_word(jj ? w2.y : w2.x, q);
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t t = bf16x2_mul(q[e], s_lo);
            hi[e] = bf16x2_fma(q[e], s_hi, t);
            if (TERMS == 2) lo[e] = bf16x2_add(bf16x2_fma(q[e], s_hi, hi[e] ^ 0x80008000u), t);
          }
          *reinterpret_cast<uint4*>(a_hi + dst_off[i][jj]) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          if (TERMS == 2) *reinterpret_cast<uint4*>(a_lo + dst_off[i][jj]) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
      }
      __syncwarp();
      if (lane == 0) {                                                // one arrival per warp
        mbar_arrive(&a_full[s_cur]);
        if (leaves) mbar_arrive(&raw_empty[r_cur]);   // done with this ring slot (nobody waits for the final ones)
      }
      if (kb + kUmmaGroups < n_kb) {                 // early look at what this group's next stage waits for
        tok_raw = leaves ? mbar_test(&raw_full[r], rph) : 1u;
        tok_empty = mbar_test(&empty[s], ph ^ 1u);
      }
    }
    // ---- epilogue: D[128 features x ntok tokens] -> y[token][feature]
    if (ok && !*failed) ok = mbar_wait_spin(acc_full, 0);
    if (!ok) give_up(DERR_TMEM);
    tc_fence_after();
    if (ok) {
      const int q4 = warp & 3;                                 // tensor-memory lane quarter this warp may read
      const int n = blockIdx.x * kUmmaRows + 32 * q4 + lane;
      // two warps share a lane quarter and alternate over the 16-column chunks
      for (int tile = 0; tile < kTokTiles; ++tile)
      for (int c0 = 16 * ((warp - kUmmaFirstDqWarp) >> 2); c0 < p.ntok; c0 += 16 * (kUmmaDqWarps / 4)) {
        float v[16], v1[16];
        tmem_ld16(tmem_d + ((uint32_t)(32 * q4) << 16) + (uint32_t)(tile * p.acc_stride + c0), v);
        const int mt = m0 + tile * p.ntok;                // first token of the tile
        const int used = DUAL ? 1 : min(p.n_acc, n_kb);   // step kb < n_acc is the first to touch accumulator kb
        for (int a = 1; a < used; ++a) {
          tmem_ld16(tmem_d + ((uint32_t)(32 * q4) << 16) + (uint32_t)(a * p.acc_stride + c0), v1);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] += v1[i];
        }
        if constexpr (KIND == I8_ROW) {
          if (p.splits == 1) {   // (with K split, the scale multiplies the sum of the partials instead)
            const float rs = row_scales[n];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] *= rs;
          }
        }
        if (p.splits > 1) {
          // K is split over gridDim.z CTAs: park the f32 partial; the last CTA of the tile adds them up
          float* part = p.partial + (size_t)blockIdx.z * p.m_total * p.n_rows;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = mt + c0 + i;
            if (m < m_end) __stcg(part + (size_t)m * p.n_rows + n, v[i]);
          }
        } else if (p.swiglu) {
          // lane l holds output row n: gate rows are the lanes with (l & 15) < 8, their up rows sit eight lanes on
          const int o_col = (n >> 4) * 8 + (lane & 7);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float up = __shfl_down_sync(0xffffffffu, v[i], 8);
            const int m = mt + c0 + i;
            if ((lane & 8) == 0 && m < m_end) {
              const float g = v[i];
              const float act = g * (1.0f / (1.0f + expf(-g))) * up;   // the formula of swiglu_kernel, term for term
              if (p.y_bf16) reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)m * p.ldy + o_col] = __float2bfloat16_rn(act);
              else reinterpret_cast<float*>(p.y)[(size_t)m * p.ldy + o_col] = act;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = mt + c0 + i;
            if (m < m_end) {
              if (p.y_bf16) reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)m * p.ldy + n] = __float2bfloat16_rn(v[i]);
              else reinterpret_cast<float*>(p.y)[(size_t)m * p.ldy + n] = v[i];
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, (uint32_t)p.tmem_cols);
  if (p.splits > 1) {
    // Deterministic split-K meet: every CTA of the tile counts in after its partial is visible; the one
    // that counts in last sums the partials in split order (so the result does not depend on which CTA
    // that was), writes y and leaves the counter at zero for the next launch.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    int* counter = p.counters + blockIdx.y * gridDim.x + blockIdx.x;
    if (threadIdx.x == 0) {
      const int seen = atomicAdd(counter, 1);
      is_last = seen == p.splits - 1;
      if (is_last) *counter = 0;
    }
    __syncthreads();
    if (is_last) {
      __threadfence();
      const int m_hi = min(p.ntok, p.m_total - m0);
      const size_t plane = (size_t)p.m_total * p.n_rows;
      for (int idx = threadIdx.x; idx < m_hi * kUmmaRows; idx += blockDim.x) {
        const int m = m0 + idx / kUmmaRows, n = blockIdx.x * kUmmaRows + idx % kUmmaRows;
        const float* src = p.partial + (size_t)m * p.n_rows + n;
        float sum = 0.f;
        for (int z = 0; z < p.splits; ++z) sum += __ldcg(src + z * plane);
        if constexpr (KIND == I8_ROW) sum *= row_scales[n];
        if (p.swiglu) {
          if (n & 8) continue;                                   // up rows are folded into their gate rows
          float up = 0.f;
          for (int z = 0; z < p.splits; ++z) up += __ldcg(src + 8 + z * plane);
          if constexpr (KIND == I8_ROW) up *= row_scales[n + 8];
          const float act = sum * (1.0f / (1.0f + expf(-sum))) * up;
          const size_t o = (size_t)m * p.ldy + (n >> 4) * 8 + (n & 7);
          if (p.y_bf16) reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(act);
          else reinterpret_cast<float*>(p.y)[o] = act;
          continue;
        }
        if (p.y_bf16) reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)m * p.ldy + n] = __float2bfloat16_rn(sum);
        else reinterpret_cast<float*>(p.y)[(size_t)m * p.ldy + n] = sum;
      }
    }
  }
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

bool umma_supported(const tq_qweight* w, size_t m) {
  return (w->kind == TQ_Q4_F16 || w->kind == TQ_Q4_F32 || w->kind == TQ_Q8_F32 || w->kind == TQ_I8_ROW) && w->rows % kUmmaRows == 0 &&
         w->cols % kTileK == 0 && m >= 1;
}

// y[m, rows] = x[m, cols] . W^T through the tcgen05 kernel.  x: bf16, 16-byte aligned rows.
// With `grp`: `grp->n_groups` weight matrices stacked by rows (experts); group e multiplies rows
// offsets[e] .. +counts[e] of x (device arrays) and m is the total row count of x / y.
int launch_qgemm_umma(tq_ctx* ctx, const tq_qweight* w, const void* x_bf16, size_t ldx, size_t m, void* y, int y_dtype,
                      size_t ldy, int terms, const UmmaGroups* grp, bool swiglu) {
  if (w->kind == TQ_I8_ROW) terms = 1;   // exact with one term: the row scale is applied to the accumulator
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(ctx, TQ_EUNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
  TQ_REQUIRE(ctx, umma_supported(w, m), "tcgen05 GEMM: needs rows %% 128 == 0 and cols %% 128 == 0");
  TQ_REQUIRE(ctx, ((uintptr_t)x_bf16 & 15) == 0 && (ldx * 2) % 16 == 0, "tcgen05 GEMM: activation rows must be 16-byte aligned");
  // Ring sizes.  Two rules come from the dequant groups running ahead of one another (a parity wait
  // is only sound when the waiter is at most one phase ahead of the barrier): at least kUmmaGroups
  // A/B stages, and an even number of packed-tile slots whenever slots are reused.  The token tile is
  // the widest that leaves room for four stages and four packed tiles, then evened out over the tiles.
  const size_t kSmemMax = 227 * 1024, raw_tile = 8 * (size_t)qk_tile_bytes(w->kind);
  const size_t budget = kSmemMax - kUmmaHeader - 1024;
  int ntok_max = (int)(((budget - 4 * raw_tile) / kUmmaGroups - (size_t)terms * kUmmaRows * 128) / 128) / 16 * 16;
  if (ntok_max > 256) ntok_max = 256;
  // The dequantised weights in tensor memory instead of shared memory: writing them there and having the tensor core
  // read them back is what fills the shared-memory pipe (32 KB written + 32 KB read per 64-k step with two terms).
  // Four stages of weights take 32 columns per term each; the rest holds the accumulators, two at least (one per
  // issuing warp): token tiles up to 128 with two terms, up to 192 with one.
  // With one term the shared-memory operand allows wider token tiles: it stays where the narrower tiles would mean
  // more of them, i.e. more conversions of the same weights (2048 rows: 9 tiles of 228 against 11 of 192 measured
  // the same; 512 rows, three tiles either way: 95 -> 77 us).
  const size_t m_basis = grp ? (size_t)grp->expected_rows : m;
  const int ts_cap = terms == 2 ? 128 : 192;
  // Many rows, one term: a CTA takes TWO token tiles (each MMA issuer multiplies every stage with its own tile's
  // activations), so the weights are converted once per 2 x <= 192 tokens; the accumulators are 2 x 192 columns, the
  // weights 128.  Only where that still gives about a wave of CTAs (no K split in this form).
  bool dual = false;
  int dual_ntok = 0;
  size_t n_pairs = 0;
  if (terms == 1 && !grp && m > 192) {
    int cap = (int)(((budget - 4 * raw_tile) / kUmmaGroups) / 256) / 16 * 16;   // two activation boxes per stage
    if (cap > 192) cap = 192;
    if (cap >= 64) {
      n_pairs = (m + 2 * (size_t)cap - 1) / (2 * (size_t)cap);
      dual_ntok = (int)(((m + 2 * n_pairs - 1) / (2 * n_pairs) + 15) / 16 * 16);
      dual = (long long)(w->rows / kUmmaRows) * (long long)n_pairs >= (ctx->sm_count * 3) / 4;
    }
  }
  const int ts = (dual || terms == 2 || (m_basis + ts_cap - 1) / ts_cap <= (m_basis + ntok_max - 1) / ntok_max) ? 1 : 0;
  if (ts && (ntok_max > ts_cap || terms == 2)) ntok_max = ts_cap;
  const size_t rows_g = grp ? w->rows / grp->n_groups : w->rows;       // output features per group
  if (grp) TQ_REQUIRE(ctx, grp->n_groups > 0 && w->rows % grp->n_groups == 0 && rows_g % kUmmaRows == 0 && grp->counts && grp->offsets,
                      "tcgen05 GEMM: every group needs a multiple of 128 output features");
  // grouped: the token tile follows the expected rows per group (tiles past a group's rows leave at once)
  const size_t m_tile_basis = grp ? (size_t)grp->expected_rows : m;
  const size_t n_tok_tiles = dual ? n_pairs : grp ? 1 : (m + ntok_max - 1) / ntok_max;   // CTAs along the tokens
  int ntok = (int)(((m_tile_basis + n_tok_tiles - 1) / n_tok_tiles + 15) / 16 * 16);
  if (ntok > ntok_max) ntok = ntok_max;
  if (ntok < 16) ntok = 16;
  if (dual) ntok = dual_ntok;
  const int ntok_stage = dual ? 2 * ntok : ntok;   // activation rows per stage
  // Few output tiles (narrow layers, small batches) leave most SMs idle: split K over gridDim.z.
  const int base_ctas = (int)(w->rows / kUmmaRows) * (int)n_tok_tiles;
  int splits = 1;
  if (!grp && base_ctas < (ctx->sm_count * 3) / 4) {
    splits = ctx->sm_count / base_ctas;
    if (splits > w->n_kc / 4) splits = w->n_kc / 4;      // at least eight 64-k steps per CTA
    if (splits > 16) splits = 16;
    // the f32 partials are written and read once more: keep them below the bytes of the weights themselves
    const size_t wbytes = (size_t)w->n_rb * w->n_kc * qk_tile_bytes(w->kind), pbytes = m * w->rows * 8;
    if ((size_t)splits > wbytes / pbytes) splits = (int)(wbytes / pbytes);
    if (splits < 1) splits = 1;
  }
  const int kc_per_split = (w->n_kc + splits - 1) / splits;
  splits = (w->n_kc + kc_per_split - 1) / kc_per_split;
  int acc_stride = 32;
  while (acc_stride < ntok) acc_stride <<= 1;
  if (ts && ntok > 128) acc_stride = 192;
  const int acc_cols = ts ? 512 - 128 * terms : 512;
  int n_acc = 2;                       // a power of two: 16 accumulators up to 32 tokens, 8 at 64, 4 at 128, 2 at 256 in
  while (!dual && n_acc < 16 && 2 * n_acc * acc_stride <= acc_cols) n_acc <<= 1;   // all of tensor memory, fewer beside the weights
  const int tmem_cols = ts ? 512 : n_acc * acc_stride;
  // Four A/B stages are what the dequant groups need; everything else goes to the packed-tile ring, because
  // the bytes in flight from HBM (ring slots not being read) are what hides its latency.  A ring slot holds
  // KT = 4 k-tiles of the eight row blocks (eight 4.6 KB copies) when three such slots fit, else KT = 2.
  int stages = kUmmaGroups;
  // Two terms and up to 32 tokens: four accumulators take 128 columns, which leaves room for SIX stages of weights, so
  // that a converting group need not wait for the MMAs of its own previous stage (decode step at 20 / 32 rows:
  // 5.16 -> 5.06 ms / 5.82 -> 5.71 ms).
  int a_col0 = acc_cols;
  if (ts && terms == 2 && acc_stride == 32) {
    stages = 6;
    n_acc = 4;
    a_col0 = 128;
  }
  if ((budget - 4 * raw_tile) / umma_stage_bytes(terms, ntok_stage, ts) < (size_t)stages)
    return fail(ctx, TQ_EUNSUPPORTED, "tcgen05 GEMM: token tile of %d does not fit", ntok);
  const size_t avail = budget - (size_t)stages * umma_stage_bytes(terms, ntok_stage, ts);
  int kt = avail / (4 * raw_tile) >= 3 ? 4 : 2;
  int raw_stages = (int)(avail / ((size_t)kt * raw_tile));
  if (raw_stages > kUmmaMaxRawStages) raw_stages = kUmmaMaxRawStages;
  const int slots_needed = (kc_per_split + kt - 1) / kt;
  if (raw_stages > slots_needed) raw_stages = slots_needed;
  if (stages < kUmmaGroups || raw_stages < 1) return fail(ctx, TQ_EUNSUPPORTED, "tcgen05 GEMM: ring sizes %d/%d", stages, raw_stages);
  CUtensorMap map;
  const cuuint64_t gdim[2] = {(cuuint64_t)w->cols, (cuuint64_t)m};
  const cuuint64_t gstride[1] = {(cuuint64_t)ldx * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kUmmaK, (cuuint32_t)ntok};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(ctx, TQ_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)cr);
  UmmaParams p;
  p.tiles = w->tiles;
  p.row_scales = w->row_scales;
  p.y = y;
  p.ldy = (long long)ldy;
  p.m_total = (int)m;
  p.n_rows = (int)rows_g;
  p.g_counts = grp ? grp->counts : nullptr;
  p.g_offsets = grp ? grp->offsets : nullptr;
  p.g_active = grp ? grp->active : nullptr;
  p.g_tile_stride = (long long)(rows_g / kTileRows) * w->n_kc * qk_tile_bytes(w->kind);
  p.kc_total = w->n_kc;
  p.ntok = ntok;
  p.tmem_cols = tmem_cols;
  p.acc_stride = acc_stride;
  p.n_acc = n_acc;
  p.ts = ts;
  p.a_col0 = a_col0;
  p.y_bf16 = y_dtype == TQ_BF16;
  p.swiglu = swiglu ? 1 : 0;
  p.err = ctx->dev_err;
  p.splits = splits;
  p.kc_per_split = kc_per_split;
  p.partial = nullptr;
  p.counters = ctx->dev_err + 1;
  if (splits > 1) {
    if (base_ctas > kTileCounters) return fail(ctx, TQ_EUNSUPPORTED, "tcgen05 GEMM: %d output tiles with split K", base_ctas);
    if (int st = ensure_splitk(ctx, (size_t)splits * m * w->rows * sizeof(float))) return st;
    p.partial = static_cast<float*>(ctx->splitk);
  }
  p.stages = stages;
  p.raw_stages = raw_stages;
  p.kt = kt;
  const size_t smem = umma_smem_bytes(w->kind, terms, ntok_stage, stages, raw_stages * kt, ts);
  if (smem > kSmemMax) return fail(ctx, TQ_EUNSUPPORTED, "tcgen05 GEMM: %zu bytes of shared memory needed", smem);
  dim3 grid((unsigned)(rows_g / kUmmaRows), (unsigned)((m + ntok_stage - 1) / ntok_stage), (unsigned)splits);
  if (grp) {
    grid.y = (unsigned)((grp->max_rows + ntok - 1) / ntok);
    grid.z = (unsigned)((grp->active && grp->max_active < grp->n_groups) ? grp->max_active : grp->n_groups);
  }
  auto go = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return launch_k(ctx, kern, grid, dim3(kUmmaThreads), smem, map, p);
  };
  cudaError_t e;
  if (dual) {
    if (splits != 1) return fail(ctx, TQ_EUNSUPPORTED, "tcgen05 GEMM: two token tiles per CTA with K split");
    if (w->kind == TQ_I8_ROW) e = go(qgemm_umma_kernel<I8_ROW, 1, true, true>);
    else if (w->kind == TQ_Q4_F16) e = go(qgemm_umma_kernel<Q4_F16, 1, true, true>);
    else if (w->kind == TQ_Q8_F32) e = go(qgemm_umma_kernel<Q8_F32, 1, true, true>);
    else e = go(qgemm_umma_kernel<Q4_F32, 1, true, true>);
  } else if (ts) {
    if (w->kind == TQ_I8_ROW) e = go(qgemm_umma_kernel<I8_ROW, 1, true>);
    else if (w->kind == TQ_Q4_F16) e = terms == 2 ? go(qgemm_umma_kernel<Q4_F16, 2, true>) : go(qgemm_umma_kernel<Q4_F16, 1, true>);
    else if (w->kind == TQ_Q8_F32) e = terms == 2 ? go(qgemm_umma_kernel<Q8_F32, 2, true>) : go(qgemm_umma_kernel<Q8_F32, 1, true>);
    else e = terms == 2 ? go(qgemm_umma_kernel<Q4_F32, 2, true>) : go(qgemm_umma_kernel<Q4_F32, 1, true>);
  } else if (w->kind == TQ_I8_ROW) e = go(qgemm_umma_kernel<I8_ROW, 1>);
  else if (w->kind == TQ_Q4_F16) e = terms == 2 ? go(qgemm_umma_kernel<Q4_F16, 2>) : go(qgemm_umma_kernel<Q4_F16, 1>);
  else if (w->kind == TQ_Q8_F32) e = terms == 2 ? go(qgemm_umma_kernel<Q8_F32, 2>) : go(qgemm_umma_kernel<Q8_F32, 1>);
  else e = terms == 2 ? go(qgemm_umma_kernel<Q4_F32, 2>) : go(qgemm_umma_kernel<Q4_F32, 1>);
  TQ_CUDA(ctx, e);
  return TQ_OK;
}

// Grouped entry for the other translation units: experts stacked by rows, rows of x / y grouped by expert.
int launch_qgemm_umma_grouped(tq_ctx* ctx, const tq_qweight* w, int n_groups, const void* x_bf16, size_t ldx, size_t m_total,
                              const int* counts, const int* offsets, const int* active, int max_active, int max_rows,
                              int expected_rows, void* y, int y_dtype, size_t ldy) {
  UmmaGroups g;
  g.n_groups = n_groups;
  g.counts = counts;
  g.offsets = offsets;
  g.active = active;
  g.max_active = max_active;
  g.max_rows = max_rows;
  g.expected_rows = expected_rows;
  return launch_qgemm_umma(ctx, w, x_bf16, ldx, m_total, y, y_dtype, ldy, y_dtype == TQ_F32 ? 2 : 1, &g, false);
}

bool umma_grouped_supported(const tq_qweight* w, int n_groups) {
  return (w->kind == TQ_Q4_F16 || w->kind == TQ_Q4_F32) && n_groups > 0 && w->rows % n_groups == 0 &&
         (w->rows / n_groups) % kUmmaRows == 0 && w->cols % kTileK == 0;
}

}  // namespace tq
