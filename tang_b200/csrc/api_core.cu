// Context, raw buffers and dtype conversion of the C ABI (include/tangq.h).
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>
#include <new>

#include "internal.h"

namespace tq {

int ensure_xprep(tq_ctx* ctx, size_t bytes) {
  if (ctx->xprep_bytes >= bytes) return TQ_OK;
  if (ctx->capturing)   // growing means a stream wait and an allocation, neither of which a capture allows
    return fail(ctx, TQ_EINVAL, "a workspace has to grow (%zu bytes) during graph capture: run the same calls once before tq_graph_begin", bytes);
  if (ctx->xprep) {
    TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    TQ_CUDA(ctx, cudaFree(ctx->xprep));
    ctx->xprep = nullptr;
    ctx->xprep_bytes = 0;
    ctx->ws_generation++;
  }
  size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
  TQ_CUDA(ctx, cudaMalloc(&ctx->xprep, want));
  ctx->xprep_bytes = want;
  return TQ_OK;
}

int ensure_scratch(tq_ctx* ctx, size_t bytes) {
  if (ctx->scratch_bytes >= bytes) return TQ_OK;
  if (ctx->capturing)   // growing means a stream wait and an allocation, neither of which a capture allows
    return fail(ctx, TQ_EINVAL, "a workspace has to grow (%zu bytes) during graph capture: run the same calls once before tq_graph_begin", bytes);
  if (ctx->scratch) {
    TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    TQ_CUDA(ctx, cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    ctx->ws_generation++;
  }
  size_t want = bytes < (4u << 20) ? (4u << 20) : bytes;
  TQ_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
  ctx->scratch_bytes = want;
  return TQ_OK;
}

int ensure_splitk(tq_ctx* ctx, size_t bytes) {
  if (ctx->splitk_bytes >= bytes) return TQ_OK;
  if (ctx->capturing)   // growing means a stream wait and an allocation, neither of which a capture allows
    return fail(ctx, TQ_EINVAL, "a workspace has to grow (%zu bytes) during graph capture: run the same calls once before tq_graph_begin", bytes);
  if (ctx->splitk) {
    TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    TQ_CUDA(ctx, cudaFree(ctx->splitk));
    ctx->splitk = nullptr;
    ctx->splitk_bytes = 0;
    ctx->ws_generation++;
  }
  size_t want = bytes < (8u << 20) ? (8u << 20) : bytes;
  TQ_CUDA(ctx, cudaMalloc(&ctx->splitk, want));
  ctx->splitk_bytes = want;
  return TQ_OK;
}

int ensure_gemm_ws2(tq_ctx* ctx, size_t bytes) {
  if (ctx->gemm_ws2_bytes >= bytes) return TQ_OK;
  if (ctx->capturing)
    return fail(ctx, TQ_EINVAL, "a workspace has to grow (%zu bytes) during graph capture: run the same calls once before tq_graph_begin", bytes);
  if (ctx->gemm_ws2) {
    TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    TQ_CUDA(ctx, cudaFree(ctx->gemm_ws2));
    ctx->gemm_ws2 = nullptr;
    ctx->gemm_ws2_bytes = 0;
    ctx->ws_generation++;
  }
  size_t want = bytes < (8u << 20) ? (8u << 20) : bytes;
  TQ_CUDA(ctx, cudaMalloc(&ctx->gemm_ws2, want));
  ctx->gemm_ws2_bytes = want;
  TQ_CUDA(ctx, cudaMemsetAsync(ctx->gemm_ws2, 0, want, ctx->stream));   // tags: nothing parked
  return TQ_OK;
}

__global__ void convert_kernel(const void* src, int sdt, void* dst, int ddt, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v;
    if (sdt == TQ_F32) v = reinterpret_cast<const float*>(src)[i];
    else if (sdt == TQ_BF16) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i]);
    else v = (float)reinterpret_cast<const double*>(src)[i];
    if (ddt == TQ_F32) reinterpret_cast<float*>(dst)[i] = v;
    else if (ddt == TQ_BF16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<double*>(dst)[i] = (double)v;
  }
}

}  // namespace tq

using namespace tq;

extern "C" {

int tq_version(void) { return 100; }

int tq_ctx_create(int device, void* stream, tq_ctx** out) {
  if (!out) return TQ_EINVAL;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0 || device < 0 || device >= n) return TQ_ECUDA;
  tq_ctx* ctx = new (std::nothrow) tq_ctx();
  if (!ctx) return TQ_ENOMEM;
  ctx->device = device;
  auto bail = [&](int st) {
    delete ctx;
    return st;
  };
  if (cudaSetDevice(device) != cudaSuccess) return bail(TQ_ECUDA);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return bail(TQ_ECUDA);
  if (prop.major != 10) return bail(TQ_EUNSUPPORTED);  // kernels are built for sm_100a only
  ctx->sm_count = prop.multiProcessorCount;
  if (const char* e = std::getenv("TQ_PDL")) ctx->pdl = std::atoi(e) != 0;
  if (stream) {
    ctx->stream = reinterpret_cast<cudaStream_t>(stream);
  } else {
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) return bail(TQ_ECUDA);
    ctx->owns_stream = true;
  }
  if (cudaMalloc(&ctx->dev_err, (1 + kTileCounters) * sizeof(int)) != cudaSuccess) return bail(TQ_ECUDA);
  if (cudaMemsetAsync(ctx->dev_err, 0, (1 + kTileCounters) * sizeof(int), ctx->stream) != cudaSuccess) return bail(TQ_ECUDA);
  const size_t ws_bytes = (size_t)kGemvSets * kGemvMaxGrid * 2 * 128 * sizeof(unsigned long long);
  if (cudaMalloc(&ctx->gemv_ws, ws_bytes) != cudaSuccess) return bail(TQ_ECUDA);
  if (cudaMemsetAsync(ctx->gemv_ws, 0, ws_bytes, ctx->stream) != cudaSuccess) return bail(TQ_ECUDA);
  if (cudaMalloc(&ctx->skg_jobs, kSkgJobs * sizeof(int)) != cudaSuccess) return bail(TQ_ECUDA);
  if (cudaHostAlloc(reinterpret_cast<void**>(&ctx->host_err), 2 * sizeof(int), cudaHostAllocMapped) != cudaSuccess) return bail(TQ_ECUDA);
  ctx->host_err[0] = ctx->host_err[1] = 0;
  if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->host_err_dev), ctx->host_err, 0) != cudaSuccess) return bail(TQ_ECUDA);
  if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return bail(TQ_ECUDA);
  *out = ctx;
  return TQ_OK;
}

int tq_ctx_destroy(tq_ctx* ctx) {
  if (!ctx) return TQ_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->xprep) cudaFree(ctx->xprep);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->splitk) cudaFree(ctx->splitk);
  if (ctx->dev_err) cudaFree(ctx->dev_err);
  if (ctx->gemv_ws) cudaFree(ctx->gemv_ws);
  if (ctx->skg_jobs) cudaFree(ctx->skg_jobs);
  if (ctx->gemm_ws2) cudaFree(ctx->gemm_ws2);
  if (ctx->hostx_ring) cudaFree(ctx->hostx_ring);
  if (ctx->hostx_tags) cudaFree(ctx->hostx_tags);   // (the epoch word sits behind the tags)
  if (ctx->host_err) cudaFreeHost(ctx->host_err);
  if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return TQ_OK;
}

const char* tq_last_error(const tq_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

void* tq_ctx_stream(tq_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

// Last kernel before a wait: copies the status word into pinned host memory and, after a system-wide fence, the wait's
// number behind it.  It waits for everything before it on the stream, so a host that sees the number has the results.
__global__ void sync_signal_kernel(const int* dev_err, volatile int* host_words, unsigned seq) {
  asm volatile("griddepcontrol.wait;" ::: "memory");   // (launched with programmatic stream serialization)
  host_words[0] = *dev_err;
  __threadfence_system();
  host_words[1] = (int)seq;
}

int tq_sync(tq_ctx* ctx) {
  if (int st = bind(ctx)) return st;
  // A short wait costs less as a look at pinned memory than as a driver call (the wake-up of cudaStreamSynchronize is
  // ~10 us): the signal kernel rides behind the work on the same stream, the host polls its word for up to ~100 us and
  // only then blocks in the driver.  Either way the status word arrives with the same round trip.
  TQ_REQUIRE(ctx, !ctx->capturing, "tq_sync: a graph capture is open (a capture cannot wait for the stream)");
  const unsigned seq = ++ctx->sync_seq;
  volatile int* hw = ctx->host_err;
  TQ_CUDA(ctx, launch_k(ctx, sync_signal_kernel, dim3(1), dim3(1), 0, (const int*)ctx->dev_err, (volatile int*)ctx->host_err_dev, seq));
  bool seen = false;
  for (int spin = 0; spin < 40000 && !seen; ++spin) seen = (unsigned)hw[1] == seq;
  if (!seen) TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->inflight_unknown = false;   // the stream has drained: nothing is in flight
  ctx->n_inflight = 0;
  const int code = *ctx->host_err;
  if (code != 0) {
    cudaMemset(ctx->dev_err, 0, (1 + kTileCounters) * sizeof(int));   // a kernel that gave up may have left tile counters half counted
    cudaMemset(ctx->gemv_ws, 0, (size_t)kGemvSets * kGemvMaxGrid * 2 * 128 * sizeof(unsigned long long));
    if (ctx->gemm_ws2) cudaMemset(ctx->gemm_ws2, 0, ctx->gemm_ws2_bytes);   // ... or parked partial sums
    if (code == 6)   // DERR_POSITION
      return fail(ctx, TQ_EINVAL, "a sequence position outside the KV cache reached a kernel (the access was skipped): positions must stay below max_seq");
    return fail(ctx, TQ_ETIMEOUT, "a kernel gave up a bounded wait (device code %d)", code);
  }
  return TQ_OK;
}

int tq_buf_alloc(tq_ctx* ctx, size_t bytes, void** dev_out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, dev_out != nullptr, "tq_buf_alloc: null output");
  *dev_out = nullptr;
  if (bytes == 0) bytes = 16;
  cudaError_t e = cudaMalloc(dev_out, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return fail(ctx, TQ_ENOMEM, "tq_buf_alloc: out of device memory (%zu bytes)", bytes);
  }
  TQ_CUDA(ctx, e);
  return TQ_OK;
}

int tq_buf_free(tq_ctx* ctx, void* dev) {
  if (int st = bind(ctx)) return st;
  if (!dev) return TQ_OK;
  TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  TQ_CUDA(ctx, cudaFree(dev));
  return TQ_OK;
}

int tq_upload(tq_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
  if (int st = bind(ctx)) return st;
  if (bytes == 0) return TQ_OK;
  TQ_REQUIRE(ctx, dst_dev && src_host, "tq_upload: null pointer");
  TQ_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return TQ_OK;
}

int tq_download(tq_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
  if (int st = bind(ctx)) return st;
  if (bytes == 0) return TQ_OK;
  TQ_REQUIRE(ctx, dst_host && src_dev, "tq_download: null pointer");
  TQ_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  TQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return TQ_OK;
}

int tq_memset(tq_ctx* ctx, void* dst_dev, int byte, size_t bytes) {
  if (int st = bind(ctx)) return st;
  if (bytes == 0) return TQ_OK;
  TQ_REQUIRE(ctx, dst_dev != nullptr, "tq_memset: null pointer");
  TQ_CUDA(ctx, cudaMemsetAsync(dst_dev, byte, bytes, ctx->stream));
  return TQ_OK;
}

int tq_convert(tq_ctx* ctx, const void* src_dev, int src_dtype, void* dst_dev, int dst_dtype, size_t n) {
  if (int st = bind(ctx)) return st;
  auto okdt = [](int d) { return d == TQ_F32 || d == TQ_BF16 || d == TQ_F64; };
  TQ_REQUIRE(ctx, okdt(src_dtype) && okdt(dst_dtype), "tq_convert: dtypes must be f32, bf16 or f64");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(ctx, src_dev && dst_dev, "tq_convert: null pointer");
  int blocks = (int)((n + 255) / 256);
  if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  convert_kernel<<<blocks, 256, 0, ctx->stream>>>(src_dev, src_dtype, dst_dev, dst_dtype, n);
  ctx->launches++;
  TQ_CUDA(ctx, cudaGetLastError());
  return TQ_OK;
}

}  // extern "C"
