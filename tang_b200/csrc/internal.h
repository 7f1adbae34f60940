// Host-side internals shared by the translation units of libtangq.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/tangq.h"

constexpr int kTileCounters = 1024;
constexpr int kGemvSets = 6, kGemvMaxGrid = 512;
constexpr int kSkgJobs = 4096;
constexpr int kHostXSlots = 64;
constexpr size_t kHostXSlotBytes = 64 * 1024;

struct tq_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  int* dev_err = nullptr;        // device status word written by kernels that give up a bounded wait,
                                 // followed by kTileCounters zeroed tile counters (split-K meets of the tcgen05
                                 // GEMM and the MoE router) and kTileCounters more for the persistent GEMV
  int* skg_jobs = nullptr;                 // [kSkgJobs] job list of a grouped persistent launch (rebuilt by every such launch)
  unsigned long long* gemm_ws2 = nullptr;  // the several-row persistent kernel's per-(slab, row block) parked sums (zero between launches)
  size_t gemm_ws2_bytes = 0;
  unsigned long long* gemv_ws = nullptr;   // [kGemvSets][kGemvMaxGrid][2][128] tagged f32 words: the persistent GEMV's
                                 // partial row blocks, all zero whenever no GEMV is running;
                                 // consecutive launches rotate through the sets (at most three kernels ever have
                                 // resident CTAs at a time: a CTA slot only frees when an older kernel's CTA exits)
  unsigned gemv_seq = 0;
  int* host_err = nullptr;       // pinned [2]: the device's status word and the number of the last tq_sync whose signal kernel ran
  int* host_err_dev = nullptr;   // ... as the device sees it
  unsigned sync_seq = 0;
  void* xprep = nullptr;         // activation staging for tq_qlinear (bf16 copy / 3-way f32 split)
  size_t xprep_bytes = 0;
  void* scratch = nullptr;       // general workspace (attention partials, host-call staging, ...)
  size_t scratch_bytes = 0;
  void* splitk = nullptr;        // f32 partials of split-K GEMMs; separate because callers that carve
  size_t splitk_bytes = 0;       // their own buffers out of `scratch` run linear layers in between
  int sm_count = 148;
  // Kernels that may still be running when the next kernel launched with the programmatic-launch attribute
  // starts: either exactly the previous one, with unknown outputs (`inflight_unknown`; every kernel but the
  // persistent GEMV waits for its predecessor before it lets its successor be scheduled), or a run of
  // persistent GEMVs whose inputs and outputs are the byte ranges listed here.  A GEMV whose activations
  // overlap none of the outputs reads them without waiting and lets its own successor be scheduled at once; if
  // its output and residual are clear of everything listed as well, it does not wait at all.
  bool inflight_unknown = true;
  // Set around one tq_qlinear call by a caller that wants the row sums of squares of the f32 output (residual
  // included), [m][row blocks of the weight]: the persistent GEMV kernels store them and set ss_written; every other
  // path leaves both alone.
  float* ss_req = nullptr;
  bool ss_written = false;
  int n_inflight = 0;
  struct Range { uintptr_t lo, hi; bool written; } inflight[96];
  // Host-vector matvecs (tq_q_matvec_host*) with pinned vectors: a one-CTA kernel copies x from the pinned host
  // vector into the next slot of this ring and tags it; the GEMV looks at the tag.  kHostXSlots exceeds the
  // longest run of kernels that wait for nothing (the in-flight list holds 32), so a slot is never rewritten
  // while a kernel that reads it can still be running.
  uint8_t* hostx_ring = nullptr;     // [kHostXSlots][kHostXSlotBytes]
  unsigned* hostx_tags = nullptr;    // [kHostXSlots]
  unsigned hostx_seq = 0;
  unsigned* hostx_epoch = nullptr;   // device word: replays of captured graphs that stage host vectors (bumped by the graph's first such call)
  bool hostx_epoch_pending = false;  // a capture is open and has not bumped the word yet
  unsigned long long ws_generation = 0;        // bumped whenever a workspace is freed and reallocated: graphs recorded
                                               // before that hold the old addresses and refuse to launch
  unsigned long long launches = 0;             // kernels launched through this context
  bool pdl = true;                             // programmatic dependent launch for the decode-path kernels
  bool capturing = false;                      // between tq_graph_begin and tq_graph_end
  unsigned long long launches_at_capture = 0;
  std::string last_error = "";
};

struct tq_qweight {
  int kind = 0;
  size_t rows = 0, cols = 0;
  size_t kpad = 0;             // cols rounded up to a multiple of 32
  int n_rb = 0, n_kc = 0;      // 16-row blocks, 128-k chunks
  uint8_t* tiles = nullptr;    // fragment tiles (csrc/qlayout.cuh), owned
  size_t tile_bytes = 0;
  float* row_scales = nullptr; // TQ_I8_ROW only, owned
  bool gate_up_interleaved = false;  // rows 16b..16b+7 are gate rows 8b..8b+7, rows 16b+8..16b+15 the matching up rows
};

namespace tq {

inline int fail(tq_ctx* ctx, int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->last_error = buf;
  return status;
}

#define TQ_CUDA(ctx, expr)                                                                         \
  do {                                                                                             \
    cudaError_t e__ = (expr);                                                                      \
    if (e__ != cudaSuccess)                                                                        \
      return ::tq::fail((ctx), TQ_ECUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
  } while (0)

#define TQ_REQUIRE(ctx, cond, ...)                                \
  do {                                                            \
    if (!(cond)) return ::tq::fail((ctx), TQ_EINVAL, __VA_ARGS__); \
  } while (0)

// Makes the device of `ctx` current for the calling thread.
inline int bind(tq_ctx* ctx) {
  if (!ctx) return TQ_EINVAL;
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  return TQ_OK;
}

// The decode step's fused forms of the quantised linear layer (qlinear.cu).  `norm`: the activations are
// rms_norm(h + delta) * gain instead of x, and h + delta goes to h_out (another buffer than h).  `swiglu`: the weight
// is a gate/up matrix in the interleaved row order and y receives silu(gate) * up, rows / 2 values per activation row.
// Up to eight rows run as one kernel; larger batches fall back to the separate operators (xn_tmp / gu_tmp).
struct QlinearNorm {
  const float* h = nullptr;
  const float* delta = nullptr;
  const void* gain_bf16 = nullptr;
  float* h_out = nullptr;
  float eps = 0.f;
  void* xn_tmp = nullptr;      // bf16 [m][cols]: the normalised rows, when the fused kernel does not apply
  // n_sumsq partial sums of squares per row of h, [m][n_sumsq], left by the projection that wrote h (tq_ctx::ss_req);
  // delta is then null.  Only a shortcut: the separate operators ignore it.
  const float* sumsq = nullptr;
  int n_sumsq = 0;
};
int qlinear_fused(tq_ctx* ctx, const tq_qweight* w, const void* x_bf16, const QlinearNorm* norm, size_t m, void* y, int y_dtype,
                  size_t ldy, bool swiglu, float* gu_tmp);

// silu(gate) * up over the f32 output of a gate/up projection in the interleaved row order: gu [rows][2n] -> out [rows][n].
int launch_swiglu_interleaved(tq_ctx* ctx, const float* gu, size_t rows, size_t n, void* out, int out_dtype);

int ensure_xprep(tq_ctx* ctx, size_t bytes);
int ensure_gemm_ws2(tq_ctx* ctx, size_t bytes);
int ensure_scratch(tq_ctx* ctx, size_t bytes);
int ensure_splitk(tq_ctx* ctx, size_t bytes);

// Launches `kern` on the context's stream.  With programmatic dependent launch enabled (default;
// TQ_PDL=0 turns it off) the launch carries the programmatic-stream-serialization attribute, so the
// kernel may start while its predecessor drains; every kernel launched this way executes
// `griddepcontrol.wait` before it touches memory another kernel wrote or still reads.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(tq_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  ctx->launches++;
  ctx->inflight_unknown = true;
  ctx->n_inflight = 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// The same launch for a kernel that neither reads nor writes anything a kernel in flight touches and that waits for
// nothing before its last instruction (the host-vector staging kernel): what the context knows about the kernels
// in flight stays valid.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k_independent(tq_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  const bool unknown = ctx->inflight_unknown;
  const int n = ctx->n_inflight;
  cudaError_t e = launch_k(ctx, kern, grid, block, smem, args...);
  ctx->inflight_unknown = unknown;
  ctx->n_inflight = n;
  return e;
}

inline size_t dtype_size(int dt) {
  switch (dt) {
    case TQ_F32: case TQ_I32: return 4;
    case TQ_BF16: case TQ_F16: return 2;
    case TQ_I8: case TQ_U8: return 1;
    case TQ_F64: return 8;
    default: return 0;
  }
}

}  // namespace tq
