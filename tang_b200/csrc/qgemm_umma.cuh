// Dequant-GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory) for many activation
// rows (prefill, large decode batches, batched experts):
//     y[m, n] = sum_k x[m, k] * q[n, k] * scale[n, k/32]
// restating crates/tang-infer/src/quantize.rs:256-289 (q4_matvec, one call per activation row) as
// one contraction.
//
// Operand roles are swapped so that any token count fits one instruction shape: the 128 output
// features of a CTA are the UMMA M dimension (A operand, the dequantised weights), the tokens are
// the UMMA N dimension (B operand, 16..256), and the f32 accumulator D[128 x tokens] lives in
// tensor memory.  Per 64-k step:
//   * warp 0 streams the packed fragment tiles (1-D bulk copies), warp 2 the activation boxes
//     (cp.async.bulk.tensor, 128-byte swizzle, out-of-range token rows filled with zeros), each as
//     far ahead as its own ring allows;
//   * sixteen dequant warps, in four groups that each take every fourth step, turn nibbles into bf16 A tiles in shared memory in the K-major
//     128-byte-swizzled layout UMMA reads.  The product q*scale (15 significant bits) is split into
//     hi = bf16(q*scale) and lo = bf16(q*scale - hi); hi + lo equals q*scale EXACTLY, so two MMAs
//     per k-step reproduce exact products with f32 accumulation (TERMS = 2).  TERMS = 1 keeps only
//     hi (relative weight error at most 2^-8), for bf16 outputs;
//   * one elected lane of warp 1 (even steps) and of warp 3 (odd steps) issues tcgen05.mma (kind::f16,
//     bf16 x bf16 -> f32), each into an accumulator of its own, and commits each stage back to the
//     producers;
//   * the dequant warps finally read both accumulators with tcgen05.ld, add them and store y.
// Tensor-memory operand (UmmaParams::ts, every launch whose token tile allows it): the A tiles do not go through
// shared memory at all.  A dequant thread owns one output row = one tensor-memory lane (in a fragment tile the row's
// nibbles are 64 contiguous bytes), converts the row's 64 k of the stage and writes them with tcgen05.st (32 columns
// per term and stage); the MMA takes A from tensor memory and only the activation box from shared memory.  Writing
// 32 KB of A tiles per step and reading them back was what bound the step time (14336 x 4096 at 64 rows, f32
// results: the decode step at batch 64 went from 9.55 to 8.26 ms; 4096^2 Q8 blocks at 2048 rows 386 -> 130 us).
// Every mbarrier wait is bounded; on failure the CTA records a code, skips ahead and still frees its
// tensor memory.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "qlayout.cuh"

namespace tq {

constexpr int kUmmaRows = 128;        // output features per CTA
constexpr int kUmmaK = 64;            // k per stage (one 128-byte swizzle span of bf16)
constexpr int kUmmaGroups = 4;        // dequant groups, each converting every fourth 64-k stage (even)
constexpr int kUmmaGroupWarps = 4;    // warps per group
constexpr int kUmmaDqWarps = kUmmaGroups * kUmmaGroupWarps;   // dequant / epilogue warps
constexpr int kUmmaFirstDqWarp = 4;   // warps 0..3: weight producer, MMA issuer (even steps), activation producer, MMA issuer (odd steps)
constexpr int kUmmaThreads = 32 * (kUmmaFirstDqWarp + kUmmaDqWarps);

struct UmmaParams {
  const uint8_t* tiles;   // fragment tiles [n_row_blocks][kc_total][tile_bytes]
  const float* row_scales;   // TQ_I8_ROW: one scale per output row (applied to the accumulator), else unused
  void* y;                // [M][ldy] f32 or bf16
  long long ldy;
  int m_total;            // activation rows
  int n_rows;             // output features (multiple of 128)
  int kc_total;           // K / 128
  int ntok;               // tokens per CTA tile = UMMA N (multiple of 16, <= 256)
  int tmem_cols;          // allocation: n_acc accumulators, power of two
  int acc_stride;         // columns between accumulators
  int ts;                 // 1: the dequantised weights go to tensor memory (columns a_col0 ..: stages x terms x 32), not to
                          //    shared memory, and the MMA reads them from there; a stage in shared memory is then the
                          //    activation box alone
  int a_col0;
  int n_acc;              // accumulators (2, 4, 8 or 16): step kb adds into number (kb & 1) + 2 * ((kb >> 1) % (n_acc / 2))
  int stages;             // A/B ring depth
  int raw_stages;         // packed-tile ring depth (slots of kt tiles of 128 k): what keeps the HBM stream in flight
  int kt;                 // k-tiles per ring slot (2 or 4)
  int y_bf16;
  int swiglu;             // the weight is a gate/up projection in the interleaved row order (rows 0..7 of every 16 gate, rows
                          // 8..15 the matching up rows): y [M][n_rows / 2] = silu(gate) * up, formed from the f32 sums
  int splits;             // CTAs along K per output tile (gridDim.z)
  int kc_per_split;       // 128-k tiles per split
  float* partial;         // [splits][m_total][n_rows] f32, only when splits > 1
  int* counters;          // one per output tile, zero between launches
  const int* g_counts;    // grouped launches (experts stacked by rows): rows of x / y per group, or null
  const int* g_offsets;   // first row of each group
  const int* g_active;    // optional list of group ids with rows (-1 = unused entry); blockIdx.z indexes it
  long long g_tile_stride;   // bytes between the groups' fragment tiles
  int* err;
};

// Host-side description of a grouped launch (device arrays come from the router's bookkeeping kernels).
struct UmmaGroups {
  int n_groups = 1;
  const int* counts = nullptr;
  const int* offsets = nullptr;
  const int* active = nullptr;
  int max_active = 0;      // upper bound of groups with rows (sizes gridDim.z)
  int max_rows = 0;        // upper bound of counts[e] (sizes gridDim.y)
  int expected_rows = 0;   // typical counts[e]: sets the token tile
};

__host__ __device__ inline size_t umma_stage_bytes(int terms, int ntok, int ts = 0) {
  return (ts ? 0 : (size_t)terms * kUmmaRows * 128) + (size_t)ntok * 128;   // A tiles + B tile, all 1024-aligned sizes
}
constexpr int kUmmaMaxRawStages = 16;
constexpr int kUmmaHeader = 1024;
__host__ __device__ inline size_t umma_smem_bytes(int kind, int terms, int ntok, int stages, int raw_tiles, int ts = 0) {
  return kUmmaHeader + 1024 /*alignment slack*/ + (size_t)stages * umma_stage_bytes(terms, ntok, ts) +
         (size_t)raw_tiles * 8 * qk_tile_bytes(kind);
}

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Sixteen 32-bit columns of the calling warp's 32 lanes: thread i writes lane i (registers = consecutive columns).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem descriptor]: the A operand is read from tensor memory (lane = row, each 32-bit
// column holds two consecutive k as bf16, eight columns per 16-k instruction).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_ptr) {
  const uint32_t addr = smem_u32(smem_ptr);
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused with swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                       // 128-byte swizzle
  return d;
}

// Instruction descriptor, kind::f16: D f32, A bf16, B bf16, both K-major, M = 128, N = ntok.
// (A and B must have the same format: an f16 A with a bf16 B is rejected by the hardware as an
// illegal instruction.)
__host__ __device__ inline uint32_t umma_idesc_bf16(int ntok) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ntok >> 3) << 17) | ((uint32_t)(kUmmaRows >> 4) << 24);
}

}  // namespace tq
