// Device-side building blocks shared by every kernel of libtangq: mbarrier + bulk-copy (TMA)
// wrappers with BOUNDED waits, warp-level mma.sync wrappers, and the in-register integer
// dequantisers.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tq {

// Error codes a kernel may leave in the context's device-side status word.
enum DeviceErr : int {
  DERR_NONE = 0,
  DERR_FULL_WAIT = 1,    // consumer gave up waiting for a bulk copy to land
  DERR_EMPTY_WAIT = 2,   // producer gave up waiting for consumers to release a stage
  DERR_SCALE_WAIT = 3,   // gave up waiting for the scale rows
  DERR_PEER_WAIT = 4,    // gave up waiting for a peer rank's flag
  DERR_TMEM = 5,         // tensor-memory allocation / MMA completion wait gave up
  DERR_POSITION = 6,     // a sequence position outside the cache (or the RoPE tables): the access was skipped
};

// Upper bound on polls of one barrier before a kernel records an error and moves on.  Each poll
// is a try_wait (which itself blocks for a hardware-defined slice), so this is seconds, not
// microseconds; it only exists so that a logic error can never hang the GPU.
constexpr uint32_t kMaxPolls = 1u << 19;

// Programmatic dependent launch: wait until every kernel this one depends on has completed and its
// writes are visible (no-op when the kernel was launched without the attribute) / allow the next
// kernel in the stream to begin launching.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async (TMA) proxy.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// One non-blocking look at the phase: 1 when the phase with this parity has completed.  The result can
// be asked for well before it is needed, which takes the barrier unit's latency off the critical path.
__device__ __forceinline__ uint32_t mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}
// Waits for the given phase parity.  Returns false (after recording `code` in *err and raising the
// CTA-wide `failed` flag) if the phase does not complete within kMaxPolls polls, or at once if
// another thread of the CTA has already failed.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* failed, int* err,
                                                  int code) {
  if (mbar_test(bar, parity)) return true;   // a completed phase answers about three times sooner this way
  for (uint32_t i = 0; i < kMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*failed) return false;
  }
  *failed = 1;
  atomicCAS(err, 0, code);
  return false;
}

// Waits for a phase entirely inside one PTX block (no C-level control flow in the hot path).  The first
// look is a test_wait, which answers about three times sooner than try_wait when the phase has already
// completed (measured: ~70 against ~200 cycles); only a phase that is still open falls through to the
// try_wait loop, which may suspend the thread.  Returns false if the phase did not complete within
// kMaxPolls polls.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .u32 n;\n\t"
      "mov.u32 %0, 1;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra TQ_DONE;\n\t"
      "mov.u32 n, 0;\n"
      "TQ_WAIT:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra TQ_DONE;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.lt.u32 p, n, %3;\n\t"
      "@p bra TQ_WAIT;\n\t"
      "mov.u32 %0, 0;\n"
      "TQ_DONE:\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kMaxPolls)
      : "memory");
  return ok != 0;
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Completes a wait whose early look gave `token`: returns at once when the phase was already seen.
__device__ __forceinline__ bool mbar_wait_token(uint64_t* bar, uint32_t parity, uint32_t token) {
  return token ? true : mbar_wait_spin(bar, parity);
}

// Arrives on `bar` from the lanes whose `pred` is set, without a branch.
__device__ __forceinline__ void mbar_arrive_if(uint64_t* bar, bool pred) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(smem_u32(bar)),
      "r"((uint32_t)pred)
      : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

// One-dimensional bulk copy global -> shared, completion reported to `bar` in bytes.  Both
// addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                         uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col).  Fragment ownership for lane = 4*g + t:
//   a0: (row g,   k 2t..2t+1)   a1: (row g+8, k 2t..2t+1)   a2: (row g, k 2t+8..2t+9)   a3: (row g+8, k 2t+8..)
//   b0: (k 2t..2t+1, col g)     b1: (k 2t+8..2t+9, col g)
//   d0,d1: (row g, col 2t,2t+1) d2,d3: (row g+8, col 2t,2t+1)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;  // (a & mask) | orv  -> immLut 0xEA
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_add(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// Unpacks one 32-bit word of tang-infer Q4 payload — eight nibbles n0..n7 for eight consecutive
// k (byte i of a block holds k=2i in its low nibble and k=2i+1 in its high nibble, stored value
// = q+8) — into four bf16x2 registers holding the SIGNED integers q = n-8 exactly:
//   out[0] = (q0, q4)   out[1] = (q1, q5)   out[2] = (q2, q6)   out[3] = (q3, q7)     (low half first)
// 0x4300|n is the bf16 128+n (exact: 7 mantissa bits hold 0..15 at this exponent); subtracting
// 136 = 128+8 is exact as well.
__device__ __forceinline__ void dequant_q4_word(uint32_t w, uint32_t (&out)[4]) {
  constexpr uint32_t kMask = 0x000F000Fu, kMagic = 0x43004300u, kBias = 0x43084308u;  // 0x4308 = 136.0
  out[0] = bf16x2_sub(lop3_and_or(w, kMask, kMagic), kBias);
  out[1] = bf16x2_sub(lop3_and_or(w >> 4, kMask, kMagic), kBias);
  out[2] = bf16x2_sub(lop3_and_or(w >> 8, kMask, kMagic), kBias);
  out[3] = bf16x2_sub(lop3_and_or(w >> 12, kMask, kMagic), kBias);
}

// The same unpacking without the bias removal: out holds 128 + n = 136 + q.  A contraction over these
// is corrected by one more MMA whose A operand is the constant -136 (kNeg136x2 in every register):
// sum (136 + q) x + sum (-136) x = sum q x, with every product still exact in f32.
constexpr uint32_t kNeg136x2 = 0xC308C308u;
__device__ __forceinline__ void dequant_q4_word_biased(uint32_t w, uint32_t (&out)[4]) {
  constexpr uint32_t kMask = 0x000F000Fu, kMagic = 0x43004300u;
  out[0] = lop3_and_or(w, kMask, kMagic);
  out[1] = lop3_and_or(w >> 4, kMask, kMagic);
  out[2] = lop3_and_or(w >> 8, kMask, kMagic);
  out[3] = lop3_and_or(w >> 12, kMask, kMagic);
}

// Converts eight int8 (two words: bytes k0..k3 and k4..k7) to bf16x2 registers in the same
// pairing as dequant_q4_word: out[i] = (q_i, q_{i+4}).  Each byte is biased to unsigned, dropped
// into the mantissa of 2^23 (f32), the bias removed with one exact subtraction, and the pair is
// packed to bf16 (exact: |q| <= 128 needs 8 significant bits).
__device__ __forceinline__ void dequant_i8_words(uint32_t wa, uint32_t wb, uint32_t (&out)[4]) {
  wa ^= 0x80808080u;
  wb ^= 0x80808080u;
  constexpr uint32_t kMagic = 0x4B000000u;
  constexpr float kBias = 8388736.0f;  // 2^23 + 128
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float lo = __uint_as_float(prmt(wa, kMagic, 0x7650u | (uint32_t)i)) - kBias;   // byte i of wa -> mantissa LSB
    float hi = __uint_as_float(prmt(wb, kMagic, 0x7650u | (uint32_t)i)) - kBias;
    __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);  // .x (low half) = lo
    out[i] = *reinterpret_cast<uint32_t*>(&pk);
  }
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace tq
