// Multi-head latent attention, decode step (include/tangq.h, tq_mla_*).  The reference has no MLA;
// this is the absorbed form, composed from the same pieces as tq_gqa_decode:
//     s_j   = (q_lat . c_j + q_rope . r_j) * scale         cache row j = [c_j (kv_lora) | r_j (rope)], bf16
//     o_lat = sum_j softmax(s)_j c_j
// i.e. multi-query attention in which all heads share one 576-wide key and its first 512 columns
// are also the value.  q_lat = W_qk[h] q_nope and o = W_uv[h] o_lat are per-head int8 GEMVs
// (tq_mla_absorb_q / tq_mla_unabsorb, grouped launches of the quantised linear kernel).
//
// Kernel: grid = (splits, heads/(16 HT), batch).  A CTA owns HT = 1 or 2 tiles of 16 heads (one MMA row tile
// each, four warps per tile) and streams 64-position cache tiles, shared by its head tiles, through a cp.async
// double buffer.  Per cache tile, warp w of a head tile scores positions 16w..16w+15 (Q fragments by ldmatrix
// from shared memory, 36 k-steps), the four warps agree on the row maxima through shared memory, write P (two bf16
// terms: with one, a sharply peaked softmax showed errors of 1e-2 of the output rms after the un-absorb GEMV)
// to shared memory, and warp w then accumulates the value columns 128w..128w+127 for all 64 positions.  Two
// head tiles per CTA double the warps that hide the latency of the legacy MMA path and halve the cache bytes
// read through L2.  Splits are merged by mla_combine_kernel with the usual max-rescaled sum.
#include <cuda_bf16.h>

#include <cfloat>

#include "common.cuh"
#include "internal.h"

namespace tq {

int launch_qgemm_grouped(tq_ctx* ctx, const tq_qweight* w, int n_groups, const void* x_bf16, size_t ldx, int mx,
                         const int* counts, const int* offsets, int max_rows, long long x_stride, long long y_stride,
                         void* y, int y_dtype, size_t ldy, const int* active = nullptr,
                         int max_active = 0, size_t total_rows = 0);

constexpr int kC = 512, kR = 64, kRow = kC + kR;         // latent, rope, cache row width
constexpr int kMlaTile = 64;
constexpr int kMlaRowBytes = kRow * 2 + 16;               // 1168: conflict-free ldmatrix rows
constexpr int kPRowBytes = kMlaTile * 2 + 16;             // 144
constexpr int kMlaThreads = 128;                          // per head tile
constexpr float kLog2eM = 1.4426950408889634f;

struct MlaParams {
  const __nv_bfloat16* q;      // [B][H][576]
  const __nv_bfloat16* cache;  // [B][max_seq][576]
  const int* lens;
  size_t seq_stride;
  int n_heads, n_splits, chunk;
  float scale;
  __nv_bfloat16* out;          // [B][H][512] bf16 (n_splits == 1)
  float* part_o;               // [B][H][n_splits][512]
  float* part_ml;              // [B][H][n_splits][2]
};

__device__ __forceinline__ void mla_cp16(void* dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ uint32_t mla_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr size_t kMlaSmemQ = 16 * kMlaRowBytes;
constexpr size_t kMlaSmemKV = 2 * (size_t)kMlaTile * kMlaRowBytes;
constexpr size_t kMlaSmemP = 2 * 16 * kPRowBytes;
constexpr size_t mla_smem(int ht) { return ht * (kMlaSmemQ + kMlaSmemP + 4 * 16 * sizeof(float)) + kMlaSmemKV; }

template <int HT>
__global__ void __launch_bounds__(kMlaThreads * HT) mla_decode_kernel(const MlaParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kThreads = kMlaThreads * HT;
  const int ht = threadIdx.x >> 7;                            // head tile of this warp
  uint8_t* kv_s = smem + HT * kMlaSmemQ;
  uint8_t* q_s = smem + ht * kMlaSmemQ;
  uint8_t* p_s = kv_s + kMlaSmemKV + ht * kMlaSmemP;         // [hi|lo][16 rows][144 B]
  float* mw = reinterpret_cast<float*>(kv_s + kMlaSmemKV + HT * kMlaSmemP) + ht * 64;   // [4 warps][16 rows] tile maxima

  const int split = blockIdx.x, hg = blockIdx.y * HT + ht, b = blockIdx.z;
  const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int len = p.lens[b];
  const int k_begin = split * p.chunk;
  const int k_end = min(len, k_begin + p.chunk);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + kMlaTile - 1) / kMlaTile : 0;
  const __nv_bfloat16* cbase = p.cache + (size_t)b * p.seq_stride;

  // Q of this head tile -> shared memory (16 rows x 72 chunks)
  {
    const __nv_bfloat16* qg = p.q + ((size_t)b * p.n_heads + (size_t)hg * 16) * kRow;
    for (int c = threadIdx.x & 127; c < 16 * 72; c += kMlaThreads) {
      const int row = c / 72, ch = c % 72;
      *reinterpret_cast<uint4*>(q_s + (size_t)row * kMlaRowBytes + ch * 16) =
          *reinterpret_cast<const uint4*>(qg + (size_t)row * kRow + ch * 8);
    }
  }

  auto load_tile = [&](int tile, int buf) {
    const int key0 = k_begin + tile * kMlaTile;
    for (int c = threadIdx.x; c < kMlaTile * 72; c += kThreads) {
      const int row = c / 72, ch = c % 72;
      const int key = key0 + row;
      const bool valid = key < k_end;
      mla_cp16(kv_s + ((size_t)buf * kMlaTile + row) * kMlaRowBytes + ch * 16,
               cbase + (size_t)(valid ? key : k_begin) * kRow + ch * 8, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float o[16][4];  // value columns 128*warp + 8*dn + 2t(+1); rows g (0,1) and g+8 (2,3)
#pragma unroll
  for (int dn = 0; dn < 16; ++dn) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.f;
  float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};

  if (n_tiles > 0) load_tile(0, 0);
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) {
      load_tile(tile + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const uint8_t* kt = kv_s + (size_t)buf * kMlaTile * kMlaRowBytes;
    const int key0 = k_begin + tile * kMlaTile + 16 * warp;

    // ---- scores of this warp's 16 positions for the 16 heads
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    {
      const uint8_t* qrow = q_s + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * kMlaRowBytes + 16 * (lane >> 4);
      // the key fragments of both 8-position halves in one ldmatrix: matrix i = (half i / 2, k 8 (i % 2) .. + 7)
      const uint8_t* krow = kt + (size_t)(16 * warp + 8 * (lane >> 4) + (lane & 7)) * kMlaRowBytes + 16 * ((lane >> 3) & 1);
#pragma unroll 4
      for (int ks = 0; ks < kRow / 16; ++ks) {
        uint32_t a[4], kb[4];
        ldsm_x4(a, qrow + 32 * ks);
        ldsm_x4(kb, krow + 32 * ks);
        mma_bf16_16816(s[0], a[0], a[1], a[2], a[3], kb[0], kb[1]);
        mma_bf16_16816(s[1], a[0], a[1], a[2], a[3], kb[2], kb[3]);
      }
    }
    // scaled, masked; sc[r][i]: row r (g / g+8), position key0 + 8*(i/2) + 2t + (i%2)
    float sc[2][4], mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const bool ok = key0 + 8 * nt + 2 * t + c < k_end;
        sc[0][2 * nt + c] = ok ? s[nt][c] * p.scale : -FLT_MAX;
        sc[1][2 * nt + c] = ok ? s[nt][2 + c] * p.scale : -FLT_MAX;
        mx[0] = fmaxf(mx[0], sc[0][2 * nt + c]);
        mx[1] = fmaxf(mx[1], sc[1][2 * nt + c]);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if (t == 0) {
      mw[warp * 16 + g] = mx[0];
      mw[warp * 16 + g + 8] = mx[1];
    }
    __syncthreads();
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      const float mt = fmaxf(fmaxf(mw[row], mw[16 + row]), fmaxf(mw[32 + row], mw[48 + row]));
      const float m_new = fmaxf(m_run[r], mt);
      alpha[r] = exp2f((m_run[r] - m_new) * kLog2eM);
      float psum = 0.f;
      float ph[4], pl[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pv = sc[r][i] == -FLT_MAX ? 0.f : exp2f((sc[r][i] - m_new) * kLog2eM);
        psum += pv;
        ph[i] = __bfloat162float(__float2bfloat16_rn(pv));
        pl[i] = pv - ph[i];
      }
      l_run[r] = l_run[r] * alpha[r] + psum;
      m_run[r] = m_new;
      // P[row][16*warp + 8*nt + 2t .. +1], two bf16 terms
      uint8_t* prow = p_s + (size_t)row * kPRowBytes + 2 * (16 * warp + 2 * t);
      *reinterpret_cast<uint32_t*>(prow) = mla_pack(ph[0], ph[1]);
      *reinterpret_cast<uint32_t*>(prow + 16) = mla_pack(ph[2], ph[3]);
      *reinterpret_cast<uint32_t*>(prow + 16 * kPRowBytes) = mla_pack(pl[0], pl[1]);
      *reinterpret_cast<uint32_t*>(prow + 16 * kPRowBytes + 16) = mla_pack(pl[2], pl[3]);
    }
    __syncthreads();

    // ---- O[:, 128w .. 128w+127] += P[16 x 64] . V[64 x 128]
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) {
      o[dn][0] *= alpha[0];
      o[dn][1] *= alpha[0];
      o[dn][2] *= alpha[1];
      o[dn][3] *= alpha[1];
    }
    {
      const uint8_t* pa = p_s + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * kPRowBytes + 16 * (lane >> 4);
      const uint8_t* va = kt + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * kMlaRowBytes + 16 * (lane >> 4) + 256 * warp;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t ah[4], al[4];
        ldsm_x4(ah, pa + 32 * ks);
        ldsm_x4(al, pa + 16 * kPRowBytes + 32 * ks);
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          uint32_t vb[4];
          ldsm_x4_t(vb, va + (size_t)16 * ks * kMlaRowBytes + 32 * dp);
          mma_bf16_16816(o[2 * dp], ah[0], ah[1], ah[2], ah[3], vb[0], vb[1]);
          mma_bf16_16816(o[2 * dp + 1], ah[0], ah[1], ah[2], ah[3], vb[2], vb[3]);
          mma_bf16_16816(o[2 * dp], al[0], al[1], al[2], al[3], vb[0], vb[1]);
          mma_bf16_16816(o[2 * dp + 1], al[0], al[1], al[2], al[3], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();  // tile buffer and P may be overwritten
  }

  // ---- row sums: lanes of a quad, then the four warps (all share the same running max)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (t == 0) {
    mw[warp * 16 + g] = l_run[0];
    mw[warp * 16 + g + 8] = l_run[1];
  }
  __syncthreads();
  float L[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    L[r] = mw[row] + mw[16 + row] + mw[32 + row] + mw[48 + row];
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int head = hg * 16 + g + 8 * r;
    const size_t bh = (size_t)b * p.n_heads + head;
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) {
      const int col = 128 * warp + 8 * dn + 2 * t;
      const float v0 = o[dn][2 * r], v1 = o[dn][2 * r + 1];
      if (p.n_splits == 1) {
        const float inv = L[r] > 0.f ? 1.0f / L[r] : 0.f;
        *reinterpret_cast<__nv_bfloat162*>(p.out + bh * kC + col) = __floats2bfloat162_rn(v0 * inv, v1 * inv);
      } else {
        float* po = p.part_o + (bh * p.n_splits + split) * kC + col;
        po[0] = v0;
        po[1] = v1;
      }
    }
    if (p.n_splits > 1 && warp == 0 && t == 0) {
      p.part_ml[(bh * p.n_splits + split) * 2] = m_run[r];
      p.part_ml[(bh * p.n_splits + split) * 2 + 1] = L[r];
    }
  }
}

__global__ void __launch_bounds__(256) mla_combine_kernel(const float* part_o, const float* part_ml, int n_splits,
                                                          __nv_bfloat16* out) {
  const size_t bh = blockIdx.x;
  float M = -FLT_MAX;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(bh * n_splits + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += part_ml[(bh * n_splits + s) * 2 + 1] * exp2f((part_ml[(bh * n_splits + s) * 2] - M) * kLog2eM);
  for (int d = threadIdx.x; d < kC; d += 256) {
    float O = 0.f;
    for (int s = 0; s < n_splits; ++s)
      O += part_o[(bh * n_splits + s) * kC + d] * exp2f((part_ml[(bh * n_splits + s) * 2] - M) * kLog2eM);
    out[bh * kC + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
  }
}

__global__ void mla_place_rope_kernel(const __nv_bfloat16* q_rope, __nv_bfloat16* q_full, size_t n_bh) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_bh * kR) q_full[(i / kR) * kRow + kC + i % kR] = q_rope[i];
}

// q [batch][n_heads][nope + 64] bf16 straight from the q_b projection: rotates each head's 64 rope dimensions
// (interleaved pairs, as ComputeDevice::rope_forward, crates/tang-compute/src/device.rs:582-610) by the table row of
// the query's position lens[b] - 1 and writes them behind the head's latent query in q_full.
__global__ void mla_rope_place_kernel(const __nv_bfloat16* q, int q_head_ld, int nope, const int* lens, const float* cos_t,
                                      const float* sin_t, int max_pos, __nv_bfloat16* q_full, int n_heads, size_t n_bh) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  constexpr int half = kR / 2;
  if (i >= n_bh * half) return;
  const size_t bh = i / half;
  const int pr = (int)(i % half);
  int pos = lens[bh / n_heads] - 1;
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const __nv_bfloat16* src = q + bh * q_head_ld + nope + 2 * pr;
  const float x0 = __bfloat162float(src[0]), x1 = __bfloat162float(src[1]);
  const float c = cos_t[(size_t)pos * half + pr], sn = sin_t[(size_t)pos * half + pr];
  __nv_bfloat16* dst = q_full + bh * kRow + kC + 2 * pr;
  dst[0] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn)));
  dst[1] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c)));
}

}  // namespace tq

struct tq_mla {
  tq_ctx* ctx = nullptr;
  tq_mla_config cfg{};
  const tq_qweight *q_a = nullptr, *q_b = nullptr, *w_qk = nullptr, *w_uv = nullptr, *w_o = nullptr;
  const void* q_norm_gain = nullptr;       // bf16 [q_lora] or null
  const float *cos_t = nullptr, *sin_t = nullptr;
  // workspace for max_batch rows
  float* qc = nullptr;                     // [B][q_lora] f32: q_a's output
  __nv_bfloat16* qc_n = nullptr;           // [B][q_lora]: normalised
  __nv_bfloat16* q = nullptr;              // [B][n_heads][nope + rope]
  __nv_bfloat16* q_full = nullptr;         // [B][n_heads][576]
  __nv_bfloat16* o_lat = nullptr;          // [B][n_heads][512]
  __nv_bfloat16* o = nullptr;              // [B][n_heads][v_dim]
};

using namespace tq;

extern "C" {

int tq_mla_create(tq_ctx* ctx, const tq_mla_config* cfg, const tq_qweight* q_a, const void* q_a_norm_gain_bf16_dev_or_null,
                  const tq_qweight* q_b, const tq_qweight* w_qk_stacked, const tq_qweight* w_uv_stacked, const tq_qweight* w_o,
                  const float* rope_cos_dev, const float* rope_sin_dev, tq_mla** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, cfg && out && q_a && q_b && w_qk_stacked && w_uv_stacked && w_o && rope_cos_dev && rope_sin_dev,
             "tq_mla_create: null argument");
  *out = nullptr;
  const size_t H = cfg->n_heads, qh = (size_t)cfg->nope_dim + cfg->rope_dim;
  TQ_REQUIRE(ctx, cfg->kv_lora == (uint32_t)kC && cfg->rope_dim == (uint32_t)kR, "tq_mla_create: kv_lora must be %d and rope_dim %d", kC, kR);
  TQ_REQUIRE(ctx, H > 0 && H % 16 == 0, "tq_mla_create: heads (per rank) must be a multiple of 16");
  TQ_REQUIRE(ctx, cfg->max_batch >= 1 && cfg->max_batch <= 64 && cfg->max_pos >= 1, "tq_mla_create: max_batch must be 1..64, max_pos >= 1");
  TQ_REQUIRE(ctx, cfg->nope_dim % 8 == 0, "tq_mla_create: nope_dim must be a multiple of 8");
  TQ_REQUIRE(ctx, q_a->rows == cfg->q_lora && q_a->cols == cfg->d_model, "tq_mla_create: q_a must be [%u, %u]", cfg->q_lora, cfg->d_model);
  TQ_REQUIRE(ctx, q_b->rows == H * qh && q_b->cols == cfg->q_lora, "tq_mla_create: q_b must be [%zu * %zu, %u]", H, qh, cfg->q_lora);
  TQ_REQUIRE(ctx, w_qk_stacked->rows == H * kC && w_qk_stacked->cols == cfg->nope_dim, "tq_mla_create: stacked W_qk must be [%zu * %d, %u]", H, kC,
             cfg->nope_dim);
  TQ_REQUIRE(ctx, w_uv_stacked->rows == H * cfg->v_dim && w_uv_stacked->cols == (size_t)kC, "tq_mla_create: stacked W_uv must be [%zu * %u, %d]", H,
             cfg->v_dim, kC);
  TQ_REQUIRE(ctx, w_o->rows == cfg->d_model && w_o->cols == H * cfg->v_dim, "tq_mla_create: W_O must be [%u, %zu * %u]", cfg->d_model, H, cfg->v_dim);
  tq_mla* m = new (std::nothrow) tq_mla();
  if (!m) return fail(ctx, TQ_ENOMEM, "out of host memory");
  m->ctx = ctx;
  m->cfg = *cfg;
  m->q_a = q_a;
  m->q_b = q_b;
  m->w_qk = w_qk_stacked;
  m->w_uv = w_uv_stacked;
  m->w_o = w_o;
  m->q_norm_gain = q_a_norm_gain_bf16_dev_or_null;
  m->cos_t = rope_cos_dev;
  m->sin_t = rope_sin_dev;
  const size_t B = cfg->max_batch;
  cudaError_t e = cudaMalloc(&m->qc, B * cfg->q_lora * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&m->qc_n, B * cfg->q_lora * 2);
  if (e == cudaSuccess) e = cudaMalloc(&m->q, B * H * qh * 2);
  if (e == cudaSuccess) e = cudaMalloc(&m->q_full, B * H * kRow * 2);
  if (e == cudaSuccess) e = cudaMalloc(&m->o_lat, B * H * kC * 2);
  if (e == cudaSuccess) e = cudaMalloc(&m->o, B * H * cfg->v_dim * 2);
  if (e != cudaSuccess) {
    cudaGetLastError();
    tq_mla_destroy(m);
    return fail(ctx, TQ_ENOMEM, "tq_mla_create: workspace allocation failed");
  }
  *out = m;
  return TQ_OK;
}

int tq_mla_destroy(tq_mla* m) {
  if (!m) return TQ_OK;
  if (m->ctx) cudaSetDevice(m->ctx->device);
  for (void* p : {(void*)m->qc, (void*)m->qc_n, (void*)m->q, (void*)m->q_full, (void*)m->o_lat, (void*)m->o})
    if (p) cudaFree(p);
  delete m;
  return TQ_OK;
}

int tq_mla_layer_decode(tq_mla* m, const void* h_bf16_dev, const void* cache_bf16_dev, const int* lens_dev, size_t batch,
                        size_t seq_stride, size_t max_len, tq_comm* comm_or_null, float* out_dev) {
  if (!m || !m->ctx) return TQ_EINVAL;
  tq_ctx* ctx = m->ctx;
  if (int st = bind(ctx)) return st;
  if (batch == 0) return TQ_OK;
  const tq_mla_config& c = m->cfg;
  TQ_REQUIRE(ctx, h_bf16_dev && cache_bf16_dev && lens_dev && out_dev, "tq_mla_layer_decode: null pointer");
  TQ_REQUIRE(ctx, batch <= c.max_batch, "tq_mla_layer_decode: batch %zu exceeds the layer's max_batch %u", batch, c.max_batch);
  const size_t H = c.n_heads, qh = (size_t)c.nope_dim + c.rope_dim;
  // hidden -> compressed query (f32) -> RMSNorm (when the layer has a gain) -> per-head [nope | rope] queries
  if (m->q_norm_gain) {
    if (int st = tq_qlinear(ctx, m->q_a, h_bf16_dev, TQ_BF16, c.d_model, batch, m->qc, TQ_F32, c.q_lora, nullptr)) return st;
    QlinearNorm norm;
    norm.h = m->qc;
    norm.gain_bf16 = m->q_norm_gain;
    norm.eps = c.norm_eps;
    norm.xn_tmp = m->qc_n;
    if (int st = qlinear_fused(ctx, m->q_b, nullptr, &norm, batch, m->q, TQ_BF16, H * qh, false, nullptr)) return st;
  } else {
    if (int st = tq_qlinear(ctx, m->q_a, h_bf16_dev, TQ_BF16, c.d_model, batch, m->qc_n, TQ_BF16, c.q_lora, nullptr)) return st;
    if (int st = tq_qlinear(ctx, m->q_b, m->qc_n, TQ_BF16, c.q_lora, batch, m->q, TQ_BF16, H * qh, nullptr)) return st;
  }
  // absorb W_UK: the nope part of each head is read in place (row stride H * qh, head stride qh)
  if (int st = launch_qgemm_grouped(ctx, m->w_qk, (int)H, m->q, H * qh, (int)batch, nullptr, nullptr, 0, (long long)qh, (long long)kRow,
                                    m->q_full, TQ_BF16, H * kRow))
    return st;
  const size_t n = batch * H * (kR / 2);
  mla_rope_place_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(m->q, (int)qh, (int)c.nope_dim, lens_dev, m->cos_t, m->sin_t,
                                                                              (int)c.max_pos, m->q_full, (int)H, batch * H);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  if (int st = tq_mla_decode(ctx, m->q_full, cache_bf16_dev, lens_dev, batch, H, kC, kR, seq_stride, max_len,
                             1.0f / sqrtf((float)qh), m->o_lat))
    return st;
  if (int st = tq_mla_unabsorb(ctx, m->w_uv, m->o_lat, batch, H, c.v_dim, m->o, TQ_BF16)) return st;
  // row-parallel output projection over this rank's heads, then the sum over the ranks
  if (int st = tq_qlinear(ctx, m->w_o, m->o, TQ_BF16, H * c.v_dim, batch, out_dev, TQ_F32, c.d_model, nullptr)) return st;
  if (comm_or_null && tq_comm_world(comm_or_null) > 1) return tq_all_reduce_f32(ctx, comm_or_null, out_dev, batch * c.d_model);
  return TQ_OK;
}

int tq_mla_absorb_q(tq_ctx* ctx, const tq_qweight* w_qk_stacked, const void* q_nope_bf16_dev, const void* q_rope_bf16_dev,
                    size_t batch, size_t n_heads, size_t nope_dim, void* q_full_bf16_dev) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, w_qk_stacked && q_nope_bf16_dev && q_rope_bf16_dev && q_full_bf16_dev, "tq_mla_absorb_q: null pointer");
  TQ_REQUIRE(ctx, batch > 0 && batch <= 64, "tq_mla_absorb_q: batch must be 1..64");
  TQ_REQUIRE(ctx, w_qk_stacked->rows == n_heads * kC && w_qk_stacked->cols == nope_dim,
             "tq_mla_absorb_q: stacked W_qk must be [%zu * %d, %zu]", n_heads, kC, nope_dim);
  if (int st = launch_qgemm_grouped(ctx, w_qk_stacked, (int)n_heads, q_nope_bf16_dev, n_heads * nope_dim, (int)batch, nullptr,
                                    nullptr, 0, (long long)nope_dim, (long long)kRow, q_full_bf16_dev, TQ_BF16, n_heads * kRow))
    return st;
  const size_t n = batch * n_heads * kR;
  mla_place_rope_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
      static_cast<const __nv_bfloat16*>(q_rope_bf16_dev), static_cast<__nv_bfloat16*>(q_full_bf16_dev), batch * n_heads);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

int tq_mla_unabsorb(tq_ctx* ctx, const tq_qweight* w_uv_stacked, const void* o_lat_bf16_dev, size_t batch, size_t n_heads,
                    size_t v_dim, void* out_dev, int out_dtype) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, w_uv_stacked && o_lat_bf16_dev && out_dev, "tq_mla_unabsorb: null pointer");
  TQ_REQUIRE(ctx, batch > 0 && batch <= 64, "tq_mla_unabsorb: batch must be 1..64");
  TQ_REQUIRE(ctx, w_uv_stacked->rows == n_heads * v_dim && w_uv_stacked->cols == (size_t)kC,
             "tq_mla_unabsorb: stacked W_uv must be [%zu * %zu, %d]", n_heads, v_dim, kC);
  TQ_REQUIRE(ctx, out_dtype == TQ_F32 || out_dtype == TQ_BF16, "tq_mla_unabsorb: out must be f32 or bf16");
  return launch_qgemm_grouped(ctx, w_uv_stacked, (int)n_heads, o_lat_bf16_dev, n_heads * kC, (int)batch, nullptr, nullptr, 0,
                              (long long)kC, (long long)v_dim, out_dev, out_dtype, n_heads * v_dim);
}

int tq_mla_decode(tq_ctx* ctx, const void* q_full_bf16_dev, const void* cache_bf16_dev, const int* lens_dev, size_t batch,
                  size_t n_heads, size_t kv_lora, size_t rope_dim, size_t seq_stride, size_t max_len, float softmax_scale,
                  void* o_lat_bf16_dev) {
  if (int st = bind(ctx)) return st;
  if (batch == 0) return TQ_OK;
  TQ_REQUIRE(ctx, q_full_bf16_dev && cache_bf16_dev && lens_dev && o_lat_bf16_dev, "tq_mla_decode: null pointer");
  TQ_REQUIRE(ctx, kv_lora == (size_t)kC && rope_dim == (size_t)kR, "tq_mla_decode: kv_lora must be %d and rope_dim %d", kC, kR);
  TQ_REQUIRE(ctx, n_heads > 0 && n_heads % 16 == 0, "tq_mla_decode: heads (per rank) must be a multiple of 16");
  TQ_REQUIRE(ctx, max_len > 0, "tq_mla_decode: max_len must bound the sequence lengths");
  const int HT = n_heads % 32 == 0 ? 2 : 1;   // head tiles per CTA
  const int B = (int)batch, HG = (int)(n_heads / (16 * HT));
  const int tiles = ((int)max_len + kMlaTile - 1) / kMlaTile;
  int want = (2 * ctx->sm_count + B * HG - 1) / (B * HG);
  int max_splits = (tiles + 1) / 2;
  if (max_splits < 1) max_splits = 1;
  int n_splits = want < 1 ? 1 : (want > max_splits ? max_splits : want);
  const int tps = (tiles + n_splits - 1) / n_splits;
  n_splits = (tiles + tps - 1) / tps;
  if (n_splits < 1) n_splits = 1;
  MlaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q_full_bf16_dev);
  p.cache = static_cast<const __nv_bfloat16*>(cache_bf16_dev);
  p.lens = lens_dev;
  p.seq_stride = seq_stride;
  p.n_heads = (int)n_heads;
  p.n_splits = n_splits;
  p.chunk = (tps > 0 ? tps : 1) * kMlaTile;
  p.scale = softmax_scale;
  p.out = static_cast<__nv_bfloat16*>(o_lat_bf16_dev);
  p.part_o = nullptr;
  p.part_ml = nullptr;
  if (n_splits > 1) {
    const size_t n_part = batch * n_heads * n_splits;
    if (int st = ensure_scratch(ctx, n_part * (kC + 2) * sizeof(float))) return st;
    p.part_o = static_cast<float*>(ctx->scratch);
    p.part_ml = p.part_o + n_part * kC;
  }
  static thread_local int attr_dev = -1;   // the attribute is per device
  if (attr_dev != ctx->device) {
    TQ_CUDA(ctx, cudaFuncSetAttribute(mla_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mla_smem(1)));
    TQ_CUDA(ctx, cudaFuncSetAttribute(mla_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mla_smem(2)));
    attr_dev = ctx->device;
  }
  dim3 grid((unsigned)n_splits, (unsigned)HG, (unsigned)B);
  if (HT == 2) mla_decode_kernel<2><<<grid, 2 * kMlaThreads, mla_smem(2), ctx->stream>>>(p);
  else mla_decode_kernel<1><<<grid, kMlaThreads, mla_smem(1), ctx->stream>>>(p);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  if (n_splits > 1) {
    mla_combine_kernel<<<(unsigned)(batch * n_heads), 256, 0, ctx->stream>>>(p.part_o, p.part_ml, n_splits, p.out);
    ctx->launches++;
    TQ_CUDA(ctx, cudaGetLastError());
  }
  return TQ_OK;
}

}  // extern "C"
