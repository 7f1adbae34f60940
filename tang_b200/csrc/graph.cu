// CUDA-graph capture of a sequence of library calls (include/tangq.h, tq_graph_*), standing in
// for CudaComputeDevice::begin_capture / end_capture (crates/tang-compute/src/cuda.rs:344-356).
#include <new>

#include "internal.h"

struct tq_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  unsigned long long kernels = 0;  // kernels recorded between begin and end
  unsigned long long ws_generation = 0;  // the context's workspace generation when the graph was recorded
};

using namespace tq;

extern "C" {

int tq_graph_begin(tq_ctx* ctx) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, !ctx->capturing, "tq_graph_begin: a capture is already open");
  TQ_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->capturing = true;
  ctx->hostx_epoch_pending = true;
  ctx->launches_at_capture = ctx->launches;
  ctx->inflight_unknown = true;   // a graph starts after everything before it: its first kernel assumes nothing
  ctx->n_inflight = 0;
  return TQ_OK;
}

int tq_graph_end(tq_ctx* ctx, tq_graph** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, out != nullptr, "tq_graph_end: null output");
  *out = nullptr;
  TQ_REQUIRE(ctx, ctx->capturing, "tq_graph_end: no capture is open");
  ctx->capturing = false;
  ctx->inflight_unknown = true;   // what was recorded has not run: later launches assume nothing about it
  ctx->n_inflight = 0;
  tq_graph* g = new (std::nothrow) tq_graph();
  if (!g) return fail(ctx, TQ_ENOMEM, "out of host memory");
  g->kernels = ctx->launches - ctx->launches_at_capture;
  g->ws_generation = ctx->ws_generation;
  ctx->launches = ctx->launches_at_capture;  // nothing ran yet; replays are counted by tq_graph_launch
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
  if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  if (e != cudaSuccess) {
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    cudaGetLastError();
    return fail(ctx, TQ_ECUDA, "tq_graph_end: %s", cudaGetErrorString(e));
  }
  *out = g;
  return TQ_OK;
}

int tq_graph_launch(tq_ctx* ctx, tq_graph* g) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, g && g->exec, "tq_graph_launch: null graph");
  // The recorded kernels hold the addresses of the context's workspaces (attention partials, staged activations,
  // split-K partials).  A later call that needed a larger workspace freed the old one: replaying would write there.
  TQ_REQUIRE(ctx, g->ws_generation == ctx->ws_generation,
             "tq_graph_launch: a workspace of this context was reallocated after the graph was recorded; record it again");
  TQ_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->kernels;
  ctx->inflight_unknown = true;
  ctx->n_inflight = 0;
  return TQ_OK;
}

int tq_graph_free(tq_ctx* ctx, tq_graph* g) {
  if (!g) return TQ_OK;
  if (int st = bind(ctx)) return st;
  cudaStreamSynchronize(ctx->stream);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return TQ_OK;
}

unsigned long long tq_launch_count(const tq_ctx* ctx) { return ctx ? ctx->launches : 0; }

}  // extern "C"
