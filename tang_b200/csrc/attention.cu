// Decode attention over a bf16 KV cache (include/tangq.h: tq_gqa_decode, tq_kv_attention).
//
// tq_gqa_decode is the hot path: one new query token per sequence, grouped-query attention
// (kv_head = head / (n_heads / n_kv_heads), crates/tang-compute/src/cpu.rs:257-315), batched over
// sequences, the cache of each sequence laid out [position, n_kv_heads*head_dim]
// (crates/tang-infer/src/kv_cache.rs:12-24).  It is bound by the HBM read of K and V, so the
// cache is split along positions across CTAs (flash-decoding): grid = (splits, kv heads, batch).
// A CTA streams 64-position K/V tiles through a cp.async double buffer; each of its four warps
// takes 16 positions of a tile, forms S = Q K^T and O += P V with mma.sync m16n8k16 (the group's
// query heads are the 16 MMA rows, of which up to 8 are used; P as a two-term bf16 sum) and keeps a
// running max / sum per
// head (online softmax, f32).  Warps, then splits, are merged with the usual max-rescaled sum.
//
// tq_kv_attention is the reference call itself (ComputeDevice::kv_attention, device.rs:161-180)
// on f32 buffers, any q_len, causal; a plain one-warp-per-(query, head) kernel in f32.
#include <cuda_bf16.h>

#include <cfloat>

#include "common.cuh"
#include "internal.h"

namespace tq {

constexpr int kHD = 128;              // head dimension of the MMA kernel
constexpr int kTileKeys = 64;         // positions per smem tile
constexpr int kRowBytes = kHD * 2 + 16;  // padded smem row: 272 B keeps ldmatrix / 4-byte reads conflict-free
constexpr int kAttnThreads = 128;
constexpr int kMaxSplits = 64;
constexpr float kLog2e = 1.4426950408889634f;

struct GqaParams {
  const __nv_bfloat16* q;        // [B, n_heads, kHD]
  const __nv_bfloat16* k_cache;  // [B][max_seq][n_kv*kHD]
  const __nv_bfloat16* v_cache;
  const int* lens;               // [B] positions to attend (including the newest)
  size_t seq_stride;             // elements between sequences
  int n_heads, n_kv, group;      // group = n_heads / n_kv  (<= 8)
  int n_splits, chunk;           // positions per split (multiple of kTileKeys)
  float scale;                   // 1/sqrt(head_dim)
  void* out;                     // [B, n_heads*kHD] bf16 or f32 (n_splits == 1)
  int out_f32;
  float* part_o;                 // [B, n_heads, n_splits, kHD]
  float* part_ml;                // [B, n_heads, n_splits, 2]
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;  // src-size 0 -> the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kAttnThreads) gqa_decode_kernel(const GqaParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  // smem: K[2][64][272] | V[2][64][272]; reused for the warp merge at the end
  uint8_t* k_s = smem;
  uint8_t* v_s = smem + 2 * kTileKeys * kRowBytes;

  pdl_wait();
  pdl_launch_dependents();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const size_t row_elems = (size_t)p.n_kv * kHD;
  const int len = min(p.lens[b], (int)(p.seq_stride / row_elems));   // never past the sequence's rows
  const int k_begin = split * p.chunk;
  const int k_end = min(len, k_begin + p.chunk);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + kTileKeys - 1) / kTileKeys : 0;
  const __nv_bfloat16* kbase = p.k_cache + (size_t)b * p.seq_stride + (size_t)kvh * kHD;
  const __nv_bfloat16* vbase = p.v_cache + (size_t)b * p.seq_stride + (size_t)kvh * kHD;

  // Q fragments: row g of the MMA = query head (kvh*group + g), zero for g >= group.
  uint32_t qa[8][2];  // [k-step][a0 (d 2t..), a2 (d 2t+8..)]
  {
    const __nv_bfloat16* qrow = p.q + ((size_t)b * p.n_heads + (size_t)kvh * p.group + g) * kHD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = g < p.group ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t) : 0u;
      qa[ks][1] = g < p.group ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t + 8) : 0u;
    }
  }

  auto load_tile = [&](int tile, int buf) {
    const int key0 = k_begin + tile * kTileKeys;
    // 64 rows x 16 chunks of 16 B for K and for V: 2048 chunks / 128 threads
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int c = threadIdx.x + i * kAttnThreads;  // 0..2047
      const int which = c >> 10, rc = c & 1023, row = rc >> 4, ch = rc & 15;
      const int key = key0 + row;
      const bool valid = key < k_end;
      const __nv_bfloat16* src = (which ? vbase : kbase) + (size_t)(valid ? key : k_begin) * row_elems + ch * 8;
      uint8_t* dst = (which ? v_s : k_s) + ((size_t)buf * kTileKeys + row) * kRowBytes + ch * 16;
      cp_async16(dst, src, valid);
    }
    cp_async_commit();
  };

  float o[16][2];  // row g (head), d = 8*dn + 2t, +1
#pragma unroll
  for (int dn = 0; dn < 16; ++dn) o[dn][0] = o[dn][1] = 0.f;
  float m_run = -FLT_MAX, l_run = 0.f;  // l_run: this lane's share of the row sum

  if (n_tiles > 0) load_tile(0, 0);
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) {
      load_tile(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    const int key0 = k_begin + tile * kTileKeys + 16 * warp;  // first of this warp's 16 positions
    if (key0 < k_end) {
      const uint8_t* kt = k_s + ((size_t)buf * kTileKeys + 16 * warp) * kRowBytes;
      const uint8_t* vt = v_s + ((size_t)buf * kTileKeys + 16 * warp) * kRowBytes;
      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const uint8_t* krow = kt + (size_t)(8 * nt + g) * kRowBytes + 4 * t;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + 32 * ks);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + 32 * ks + 16);
          mma_bf16_16816(s[nt], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
        }
      }
      // scores of row g: positions key0 + 8*nt + 2t, +1
      float sc[4];
      float mx = -FLT_MAX;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int key = key0 + 8 * nt + 2 * t + c;
          const float v = key < k_end ? s[nt][c] * p.scale : -FLT_MAX;
          sc[2 * nt + c] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float alpha = exp2f((m_run - m_new) * kLog2e);
      float pr[4];
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pr[i] = sc[i] == -FLT_MAX ? 0.f : exp2f((sc[i] - m_new) * kLog2e);
        psum += pr[i];
      }
      l_run = l_run * alpha + psum;
      m_run = m_new;
#pragma unroll
      for (int dn = 0; dn < 16; ++dn) {
        o[dn][0] *= alpha;
        o[dn][1] *= alpha;
      }
      // P enters the tensor core as bf16; a second, residual term (p - bf16(p)) keeps 16 significant
      // bits so the result does not depend on bf16's 8-bit rounding of the probabilities.
      float ph[4], pl[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ph[i] = __bfloat162float(__float2bfloat16_rn(pr[i]));
        pl[i] = pr[i] - ph[i];
      }
      const uint32_t pa0 = pack_bf16(ph[0], ph[1]);  // row g, positions 2t, 2t+1
      const uint32_t pa2 = pack_bf16(ph[2], ph[3]);  // row g, positions 2t+8, 2t+9
      const uint32_t pb0 = pack_bf16(pl[0], pl[1]);
      const uint32_t pb2 = pack_bf16(pl[2], pl[3]);
      // V fragments, two d-tiles per ldmatrix.x4.trans
      const uint8_t* vrow = vt + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * kRowBytes + 16 * (lane >> 4);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vrow + 32 * dp);
        float acc0[4] = {o[2 * dp][0], o[2 * dp][1], 0.f, 0.f};
        float acc1[4] = {o[2 * dp + 1][0], o[2 * dp + 1][1], 0.f, 0.f};
        mma_bf16_16816(acc0, pa0, 0u, pa2, 0u, vb[0], vb[1]);
        mma_bf16_16816(acc1, pa0, 0u, pa2, 0u, vb[2], vb[3]);
        mma_bf16_16816(acc0, pb0, 0u, pb2, 0u, vb[0], vb[1]);
        mma_bf16_16816(acc1, pb0, 0u, pb2, 0u, vb[2], vb[3]);
        o[2 * dp][0] = acc0[0];
        o[2 * dp][1] = acc0[1];
        o[2 * dp + 1][0] = acc1[0];
        o[2 * dp + 1][1] = acc1[1];
      }
    }
    __syncthreads();  // everyone is done with `buf` before it is refilled
  }

  // ---- merge the four warps (rows g < group only)
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  float* mo = reinterpret_cast<float*>(smem);                   // [4 warps][8 rows][128]
  float* mml = mo + 4 * 8 * kHD;                                // [4 warps][8 rows][2]
#pragma unroll
  for (int dn = 0; dn < 16; ++dn) {
    mo[((size_t)warp * 8 + g) * kHD + 8 * dn + 2 * t] = o[dn][0];
    mo[((size_t)warp * 8 + g) * kHD + 8 * dn + 2 * t + 1] = o[dn][1];
  }
  if (t == 0) {
    mml[(warp * 8 + g) * 2] = m_run;
    mml[(warp * 8 + g) * 2 + 1] = l_run;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.group * kHD; idx += kAttnThreads) {
    const int r = idx / kHD, d = idx % kHD;
    float M = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 8 + r) * 2]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = exp2f((mml[(w * 8 + r) * 2] - M) * kLog2e);
      L += mml[(w * 8 + r) * 2 + 1] * wgt;
      O += mo[((size_t)w * 8 + r) * kHD + d] * wgt;
    }
    const int head = kvh * p.group + r;
    if (p.n_splits == 1) {
      const float v = L > 0.f ? O / L : 0.f;
      const size_t oi = ((size_t)b * p.n_heads + head) * kHD + d;
      if (p.out_f32) reinterpret_cast<float*>(p.out)[oi] = v;
      else reinterpret_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(v);
    } else {
      const size_t pi = ((size_t)b * p.n_heads + head) * p.n_splits + split;
      p.part_o[pi * kHD + d] = O;
      if (d == 0) {
        p.part_ml[pi * 2] = M;
        p.part_ml[pi * 2 + 1] = L;
      }
    }
  }
}

__global__ void __launch_bounds__(kHD) gqa_combine_kernel(const float* part_o, const float* part_ml, int n_splits,
                                                          void* out, int out_f32) {
  pdl_wait();
  pdl_launch_dependents();
  // the splits' merge weights once per CTA (a few numbers), then independent loads over the partial outputs
  __shared__ float wgt_s[kMaxSplits];
  __shared__ float inv_l;
  const size_t bh = blockIdx.x;  // b * n_heads + head
  const int d = threadIdx.x;
  if (threadIdx.x < 32) {
    float M = -FLT_MAX;
    for (int s = threadIdx.x; s < n_splits; s += 32) M = fmaxf(M, part_ml[(bh * n_splits + s) * 2]);
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.f;
    for (int s = threadIdx.x; s < n_splits; s += 32) {
      const float wgt = exp2f((part_ml[(bh * n_splits + s) * 2] - M) * kLog2e);
      wgt_s[s] = wgt;
      L += part_ml[(bh * n_splits + s) * 2 + 1] * wgt;
    }
    // lanes hold disjoint splits: add them in lane order so that the sum does not depend on the shuffle tree
    float Lsum = 0.f;
    for (int l = 0; l < 32; ++l) Lsum += __shfl_sync(0xffffffffu, L, l);
    if (threadIdx.x == 0) inv_l = Lsum > 0.f ? 1.0f / Lsum : 0.f;
  }
  __syncthreads();
  const float* src = part_o + bh * n_splits * kHD + d;
  float O = 0.f;
#pragma unroll 8
  for (int s = 0; s < n_splits; ++s) O += src[(size_t)s * kHD] * wgt_s[s];
  const float v = O * inv_l;
  if (out_f32) reinterpret_cast<float*>(out)[bh * kHD + d] = v;
  else reinterpret_cast<__nv_bfloat16*>(out)[bh * kHD + d] = __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------------------------------------
// Causal GQA attention for a chunk of q_len new positions per sequence (prefill, q_len > 1 of
// ComputeDevice::kv_attention, crates/tang-compute/src/device.rs:161-180; cpu.rs:257-315): query i of sequence b
// attends cache positions 0 .. cache_start[b] + i.  bf16 q / K / V, f32 online softmax, bf16 probabilities into
// the tensor core (mma.sync m16n8k16).  A CTA owns 64 (position, head-of-the-group) rows of one KV head -- so the
// K/V tiles it streams (cp.async, double-buffered, 64 keys each) serve every query head of the group -- and each
// of its four warps 16 of those rows against all 64 keys of a tile.
// ---------------------------------------------------------------------------------------------
struct PrefillParams {
  const __nv_bfloat16* q;        // [B][q_len][n_heads*kHD]
  const __nv_bfloat16* k_cache;  // [B][max_seq][n_kv*kHD], the chunk's own K/V already appended
  const __nv_bfloat16* v_cache;
  const int* cache_start;        // [B] positions in the cache before this chunk
  size_t seq_stride;
  int q_len, n_heads, n_kv, group;
  float scale;
  void* out;                     // [B][q_len][n_heads*kHD]
  int out_f32;
  int* err;                      // the context's status word
};

__global__ void __launch_bounds__(kAttnThreads) gqa_prefill_kernel(const PrefillParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* k_s = smem;
  uint8_t* v_s = smem + 2 * kTileKeys * kRowBytes;
  pdl_wait();
  pdl_launch_dependents();
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int pos_per_cta = 64 / p.group;
  const int pos0 = blockIdx.x * pos_per_cta;                     // first query position of this CTA
  const size_t row_elems = (size_t)p.n_kv * kHD;
  const int start = p.cache_start[b];
  // The chunk must lie inside the sequence's cache rows (cache_start comes from device memory): if not, nothing
  // is read or written for this sequence and the status word says why.
  if (start < 0 || (size_t)start + (size_t)p.q_len > p.seq_stride / row_elems) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && kvh == 0) atomicCAS(p.err, 0, (int)DERR_POSITION);
    return;
  }
  const int last_pos = min(p.q_len, pos0 + pos_per_cta) - 1;     // last live query position
  const int k_end = start + last_pos + 1;                        // keys this CTA needs (causal)
  const int n_tiles = (k_end + kTileKeys - 1) / kTileKeys;
  const __nv_bfloat16* kbase = p.k_cache + (size_t)b * p.seq_stride + (size_t)kvh * kHD;
  const __nv_bfloat16* vbase = p.v_cache + (size_t)b * p.seq_stride + (size_t)kvh * kHD;

  // this lane's two rows: r = 16*warp + g and + 8 -> (position, head)
  int qpos[2];
  bool live[2];
  uint32_t qa[8][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = 16 * warp + g + 8 * h;
    const int pl = r / p.group, head = kvh * p.group + r % p.group;
    qpos[h] = pos0 + pl;
    live[h] = qpos[h] < p.q_len;
    const __nv_bfloat16* qrow = p.q + (((size_t)b * p.q_len + (live[h] ? qpos[h] : 0)) * p.n_heads + head) * kHD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][h] = live[h] ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t) : 0u;          // a0 / a1
      qa[ks][2 + h] = live[h] ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t + 8) : 0u;  // a2 / a3
    }
  }

  auto load_tile = [&](int tile, int buf) {
    const int key0 = tile * kTileKeys;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int c = threadIdx.x + i * kAttnThreads;
      const int which = c >> 10, rc = c & 1023, row = rc >> 4, ch = rc & 15;
      const int key = key0 + row;
      const bool valid = key < k_end;
      const __nv_bfloat16* src = (which ? vbase : kbase) + (size_t)(valid ? key : 0) * row_elems + ch * 8;
      uint8_t* dst = (which ? v_s : k_s) + ((size_t)buf * kTileKeys + row) * kRowBytes + ch * 16;
      cp_async16(dst, src, valid);
    }
    cp_async_commit();
  };

  float o[16][4];   // [d-tile][row g: d 2t, 2t+1 | row g+8: d 2t, 2t+1]
#pragma unroll
  for (int dn = 0; dn < 16; ++dn) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.f;
  float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};

  if (n_tiles > 0) load_tile(0, 0);
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) {
      load_tile(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = tile * kTileKeys;
    const uint8_t* kt = k_s + (size_t)buf * kTileKeys * kRowBytes;
    const uint8_t* vt = v_s + (size_t)buf * kTileKeys * kRowBytes;
    // ---- S = Q K^T for 16 rows x 64 keys
    float sacc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
      const uint8_t* krow = kt + (size_t)(8 * nt + g) * kRowBytes + 4 * t;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + 32 * ks);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + 32 * ks + 16);
        mma_bf16_16816(sacc[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
      }
    }
    // ---- causal mask, online softmax (rows g and g+8; a row's 64 scores live in its four lanes)
    float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int h = c >> 1, key = key0 + 8 * nt + 2 * t + (c & 1);
        const bool ok = live[h] && key <= start + qpos[h];
        const float v = ok ? sacc[nt][c] * p.scale : -FLT_MAX;
        sacc[nt][c] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      alpha[h] = exp2f((m_run[h] - m_new) * kLog2e);
      m_run[h] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int h = c >> 1;
        const float pv = sacc[nt][c] == -FLT_MAX ? 0.f : exp2f((sacc[nt][c] - m_run[h]) * kLog2e);
        sacc[nt][c] = pv;
        psum[h] += pv;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + psum[h];
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) {
      o[dn][0] *= alpha[0];
      o[dn][1] *= alpha[0];
      o[dn][2] *= alpha[1];
      o[dn][3] *= alpha[1];
    }
    // ---- O += P V, 16 keys per k-step; the S accumulator layout is the A fragment layout
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t a0 = pack_bf16(sacc[2 * j][0], sacc[2 * j][1]);
      const uint32_t a1 = pack_bf16(sacc[2 * j][2], sacc[2 * j][3]);
      const uint32_t a2 = pack_bf16(sacc[2 * j + 1][0], sacc[2 * j + 1][1]);
      const uint32_t a3 = pack_bf16(sacc[2 * j + 1][2], sacc[2 * j + 1][3]);
      const uint8_t* vrow = vt + (size_t)(16 * j + (lane & 7) + 8 * ((lane >> 3) & 1)) * kRowBytes + 16 * (lane >> 4);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vrow + 32 * dp);
        mma_bf16_16816(o[2 * dp], a0, a1, a2, a3, vb[0], vb[1]);
        mma_bf16_16816(o[2 * dp + 1], a0, a1, a2, a3, vb[2], vb[3]);
      }
    }
    __syncthreads();
  }
  // ---- normalise and store
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!live[h]) continue;
    const int r = 16 * warp + g + 8 * h;
    const int head = kvh * p.group + r % p.group;
    const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
    const size_t oi = (((size_t)b * p.q_len + qpos[h]) * p.n_heads + head) * kHD;
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) {
      const float v0 = o[dn][2 * h] * inv, v1 = o[dn][2 * h + 1] * inv;
      if (p.out_f32) {
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + oi + 8 * dn + 2 * t) = make_float2(v0, v1);
      } else {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(p.out) + oi + 8 * dn + 2 * t) = pack_bf16(v0, v1);
      }
    }
  }
}

// ComputeDevice::kv_attention on f32 buffers (cpu.rs:257-315): one warp per (query, head); each
// lane owns head_dim/32 output columns; positions are visited in order with the reference's
// running-max update, dot products reduced across the warp.
__global__ void kv_attention_f32_kernel(const float* q, const float* k_cache, const float* v_cache, float* out,
                                        int cache_start, int q_len, int n_heads, int n_kv, int head_dim) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= q_len * n_heads) return;
  const int qi = gw / n_heads, h = gw % n_heads;
  const int kv_h = h / (n_heads / n_kv);
  const int kv_dim = n_kv * head_dim;
  const float scale = 1.0f / sqrtf((float)head_dim);
  const float* qp = q + ((size_t)qi * n_heads + h) * head_dim;
  const int attend = cache_start + qi + 1;
  constexpr int kMaxPer = 8;  // head_dim <= 256
  float acc[kMaxPer];
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) acc[i] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;
  for (int j = 0; j < attend; ++j) {
    const float* kp = k_cache + (size_t)j * kv_dim + (size_t)kv_h * head_dim;
    float dot = 0.f;
    for (int d = lane; d < head_dim; d += 32) dot += qp[d] * kp[d];
    dot = warp_sum(dot);
    const float score = dot * scale;
    const float new_max = fmaxf(run_max, score);
    const float e = expf(score - new_max), rescale = expf(run_max - new_max);
    run_sum = run_sum * rescale + e;
    const float* vp = v_cache + (size_t)j * kv_dim + (size_t)kv_h * head_dim;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) acc[i] = acc[i] * rescale + e * vp[d];
    }
    run_max = new_max;
  }
  const float inv = 1.0f / run_sum;
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) out[((size_t)qi * n_heads + h) * head_dim + d] = acc[i] * inv;
  }
}

int launch_gqa_decode(tq_ctx* ctx, const void* q, const void* k_cache, const void* v_cache, const int* lens, int B,
                      int n_heads, int n_kv, int head_dim, size_t seq_stride, int max_len, void* out, int out_dtype) {
  TQ_REQUIRE(ctx, head_dim == kHD, "tq_gqa_decode: head_dim must be %d", kHD);
  TQ_REQUIRE(ctx, n_kv > 0 && n_heads % n_kv == 0 && n_heads / n_kv <= 8, "tq_gqa_decode: n_heads/n_kv_heads must be 1..8");
  TQ_REQUIRE(ctx, out_dtype == TQ_BF16 || out_dtype == TQ_F32, "tq_gqa_decode: out must be bf16 or f32");
  if (B == 0) return TQ_OK;
  GqaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.lens = lens;
  p.seq_stride = seq_stride;
  p.n_heads = n_heads;
  p.n_kv = n_kv;
  p.group = n_heads / n_kv;
  p.scale = 1.0f / sqrtf((float)head_dim);
  p.out = out;
  p.out_f32 = out_dtype == TQ_F32;
  // enough CTAs for ~4 per SM, at least 128 positions per split
  const int tiles = (max_len + kTileKeys - 1) / kTileKeys;
  int want = (4 * ctx->sm_count + B * n_kv - 1) / (B * n_kv);
  int max_splits = (tiles + 1) / 2;
  if (max_splits < 1) max_splits = 1;
  if (max_splits > kMaxSplits) max_splits = kMaxSplits;   // the merge kernel keeps one weight per split in shared memory
  int n_splits = want < 1 ? 1 : (want > max_splits ? max_splits : want);
  const int tiles_per_split = (tiles + n_splits - 1) / n_splits;
  n_splits = (tiles + tiles_per_split - 1) / tiles_per_split;
  if (n_splits < 1) n_splits = 1;
  p.n_splits = n_splits;
  p.chunk = (tiles_per_split > 0 ? tiles_per_split : 1) * kTileKeys;
  p.part_o = nullptr;
  p.part_ml = nullptr;
  if (n_splits > 1) {
    const size_t n_part = (size_t)B * n_heads * n_splits;
    const size_t bytes = n_part * (kHD + 2) * sizeof(float);
    if (int st = ensure_scratch(ctx, bytes)) return st;
    p.part_o = static_cast<float*>(ctx->scratch);
    p.part_ml = p.part_o + n_part * kHD;
  }
  const size_t smem = 4 * (size_t)kTileKeys * kRowBytes;
  static bool attr_set[64] = {};   // per device: the attribute belongs to the device's copy of the kernel
  if (!attr_set[ctx->device & 63]) {
    TQ_CUDA(ctx, cudaFuncSetAttribute(gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[ctx->device & 63] = true;
  }
  dim3 grid((unsigned)n_splits, (unsigned)n_kv, (unsigned)B);
  TQ_CUDA(ctx, launch_k(ctx, gqa_decode_kernel, grid, dim3(kAttnThreads), smem, p));
  if (n_splits > 1)
    TQ_CUDA(ctx, launch_k(ctx, gqa_combine_kernel, dim3((unsigned)(B * n_heads)), dim3(kHD), 0, (const float*)p.part_o,
                          (const float*)p.part_ml, n_splits, out, p.out_f32));
  return TQ_OK;
}

}  // namespace tq

using namespace tq;

extern "C" {

int tq_gqa_decode(tq_ctx* ctx, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev, const int* lens_dev,
                  size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t seq_stride, size_t max_len,
                  void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;
  if (batch == 0) return TQ_OK;
  TQ_REQUIRE(ctx, q_dev && k_cache_dev && v_cache_dev && lens_dev && out_dev, "tq_gqa_decode: null pointer");
  TQ_REQUIRE(ctx, max_len > 0, "tq_gqa_decode: max_len must bound the sequence lengths");
  return launch_gqa_decode(ctx, q_dev, k_cache_dev, v_cache_dev, lens_dev, (int)batch, (int)n_heads, (int)n_kv_heads,
                           (int)head_dim, seq_stride, (int)max_len, out_dev, out_dtype);
}

int tq_gqa_prefill(tq_ctx* ctx, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev, const int* cache_start_dev,
                   size_t batch, size_t q_len, size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t seq_stride,
                   void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;
  if (batch == 0 || q_len == 0) return TQ_OK;
  TQ_REQUIRE(ctx, q_dev && k_cache_dev && v_cache_dev && cache_start_dev && out_dev, "tq_gqa_prefill: null pointer");
  TQ_REQUIRE(ctx, head_dim == (size_t)kHD, "tq_gqa_prefill: head_dim must be %d", kHD);
  const size_t group = n_kv_heads ? n_heads / n_kv_heads : 0;
  TQ_REQUIRE(ctx, n_kv_heads > 0 && n_heads % n_kv_heads == 0 && (group == 1 || group == 2 || group == 4 || group == 8),
             "tq_gqa_prefill: n_heads/n_kv_heads must be 1, 2, 4 or 8");
  TQ_REQUIRE(ctx, out_dtype == TQ_BF16 || out_dtype == TQ_F32, "tq_gqa_prefill: out must be bf16 or f32");
  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q_dev);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache_dev);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache_dev);
  p.cache_start = cache_start_dev;
  p.seq_stride = seq_stride;
  p.q_len = (int)q_len;
  p.n_heads = (int)n_heads;
  p.n_kv = (int)n_kv_heads;
  p.group = (int)group;
  p.scale = 1.0f / sqrtf((float)head_dim);
  p.out = out_dev;
  p.out_f32 = out_dtype == TQ_F32;
  p.err = ctx->dev_err;
  const size_t smem = 4 * (size_t)kTileKeys * kRowBytes;
  static bool attr_set[64] = {};   // per device, as above
  if (!attr_set[ctx->device & 63]) {
    TQ_CUDA(ctx, cudaFuncSetAttribute(gqa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[ctx->device & 63] = true;
  }
  const size_t pos_per_cta = 64 / group;
  dim3 grid((unsigned)((q_len + pos_per_cta - 1) / pos_per_cta), (unsigned)n_kv_heads, (unsigned)batch);
  TQ_CUDA(ctx, launch_k(ctx, gqa_prefill_kernel, grid, dim3(kAttnThreads), smem, p));
  return TQ_OK;
}

int tq_kv_attention(tq_ctx* ctx, const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                    size_t cache_start, size_t q_len, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                    float* out_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, n_kv_heads > 0 && n_heads % n_kv_heads == 0, "tq_kv_attention: n_heads must be a multiple of n_kv_heads");
  TQ_REQUIRE(ctx, head_dim > 0 && head_dim <= 256, "tq_kv_attention: head_dim must be in 1..256");
  if (q_len == 0 || n_heads == 0) return TQ_OK;
  TQ_REQUIRE(ctx, q_dev && k_cache_dev && v_cache_dev && out_dev, "tq_kv_attention: null pointer");
  const size_t warps = q_len * n_heads;
  kv_attention_f32_kernel<<<(unsigned)((warps * 32 + 127) / 128), 128, 0, ctx->stream>>>(
      q_dev, k_cache_dev, v_cache_dev, out_dev, (int)cache_start, (int)q_len, (int)n_heads, (int)n_kv_heads, (int)head_dim);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}


// ---------------------------------------------------------------------------------------------
// tq_gqa_decode_noalloc: the same split-KV decode attention, for callers that must not allocate.
//
// Who that is: code running where cudaMalloc is off limits — inside a latency-critical serving loop
// that has promised its host not to touch the allocator after start-up, inside a library callback
// that is only handed a stream, or in a process whose memory pool was sized once and is owned by
// someone else.  tq_gqa_decode keeps the per-split partial results in the context's workspace, which
// it grows with cudaFree/cudaMalloc when a call needs more; this variant never does.  Its partials
// live in the fixed array below, which every GPU that loads the library holds until the process
// exits.
//
// The array's name is only a host-side stand-in for the device object: host code cannot pass it to a
// kernel.  The device address is fetched once per device with cudaGetSymbolAddress while that device
// is current (first call on the device), checked, cached, and handed to the kernels.  Because that
// first call also sets the kernel's shared-memory attribute, make it before starting any stream
// capture.
//
// All calls on a device share the one array and it keeps whatever the last call left there.  Nothing
// in it has to start at zero: every (sequence, head, split) slot a call reads is written by that call
// first, including the splits that turn out empty.  Two calls that overlap on the GPU (different
// streams, or a graph replay racing a plain call) would overwrite each other's partials; the caller
// has to keep calls on one device ordered.
// ---------------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = 3u << 20;  // 3 MiB: e.g. 64 sequences x 32 heads x 2 splits = 2.1 MB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
constexpr int kNoAllocMaxDevices = 64;
static void* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};

int tq_gqa_decode_noalloc(tq_ctx* ctx, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev,
                          const int* lens_dev, size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                          size_t seq_stride, size_t max_len, void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;  // makes ctx->device current
  if (batch == 0) return TQ_OK;
  TQ_REQUIRE(ctx, q_dev && k_cache_dev && v_cache_dev && lens_dev && out_dev, "tq_gqa_decode_noalloc: null pointer");
  TQ_REQUIRE(ctx, max_len > 0, "tq_gqa_decode_noalloc: max_len must bound the sequence lengths");
  TQ_REQUIRE(ctx, head_dim == (size_t)kHD, "tq_gqa_decode_noalloc: head_dim must be %d", kHD);
  TQ_REQUIRE(ctx, n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= 8,
             "tq_gqa_decode_noalloc: n_heads/n_kv_heads must be 1..8");
  TQ_REQUIRE(ctx, out_dtype == TQ_BF16 || out_dtype == TQ_F32, "tq_gqa_decode_noalloc: out must be bf16 or f32");
  TQ_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kNoAllocMaxDevices, "tq_gqa_decode_noalloc: device index out of range");
  const size_t smem = 4 * (size_t)kTileKeys * kRowBytes;
  if (g_noalloc_ptr[ctx->device] == nullptr) {  // set-up, once per device, with that device current
    void* ptr = nullptr;
    TQ_CUDA(ctx, cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    TQ_REQUIRE(ctx, ptr != nullptr, "tq_gqa_decode_noalloc: the static scratch array has no device address");
    TQ_CUDA(ctx, cudaFuncSetAttribute(gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    g_noalloc_ptr[ctx->device] = ptr;
  }
  const int B = (int)batch, n_kv = (int)n_kv_heads, nh = (int)n_heads;
  // same split rule as tq_gqa_decode
  const int tiles = ((int)max_len + kTileKeys - 1) / kTileKeys;
  const int want = (4 * ctx->sm_count + B * n_kv - 1) / (B * n_kv);
  int max_splits = (tiles + 1) / 2;
  if (max_splits < 1) max_splits = 1;
  if (max_splits > kMaxSplits) max_splits = kMaxSplits;   // the merge kernel keeps one weight per split in shared memory
  int n_splits = want < 1 ? 1 : (want > max_splits ? max_splits : want);
  const int tiles_per_split = (tiles + n_splits - 1) / n_splits;
  n_splits = (tiles + tiles_per_split - 1) / tiles_per_split;
  if (n_splits < 1) n_splits = 1;
  const size_t n_part = (size_t)B * nh * n_splits;
  const size_t need = n_part * (kHD + 2) * sizeof(float);
  if (n_splits > 1 && need > kNoAllocScratchBytes)
    return fail(ctx, TQ_EINVAL,
                "tq_gqa_decode_noalloc: %zu sequences x %zu heads x %d splits need %zu bytes of partials; the static "
                "scratch holds %zu (use tq_gqa_decode, or a smaller batch)",
                batch, n_heads, n_splits, need, kNoAllocScratchBytes);
  GqaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q_dev);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache_dev);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache_dev);
  p.lens = lens_dev;
  p.seq_stride = seq_stride;
  p.n_heads = nh;
  p.n_kv = n_kv;
  p.group = nh / n_kv;
  p.scale = 1.0f / sqrtf((float)head_dim);
  p.out = out_dev;
  p.out_f32 = out_dtype == TQ_F32;
  p.n_splits = n_splits;
  p.chunk = (tiles_per_split > 0 ? tiles_per_split : 1) * kTileKeys;
  p.part_o = n_splits > 1 ? static_cast<float*>(g_noalloc_ptr[ctx->device]) : nullptr;
  p.part_ml = n_splits > 1 ? p.part_o + n_part * kHD : nullptr;
  dim3 grid((unsigned)n_splits, (unsigned)n_kv, (unsigned)B);
  gqa_decode_kernel<<<grid, kAttnThreads, smem, ctx->stream>>>(p);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  if (n_splits > 1) {
    gqa_combine_kernel<<<(unsigned)(B * nh), kHD, 0, ctx->stream>>>(p.part_o, p.part_ml, n_splits, out_dev, p.out_f32);
    ctx->launches++;
    TQ_CUDA(ctx, cudaGetLastError());
  }
  return TQ_OK;
}

}  // extern "C"
