/* tangq.h — C ABI of libtangq, the sm_100a implementation of tang-infer's quantised decode path.
 *
 * Every entry point takes plain pointers and sizes, returns a tq_status, never unwinds, and is
 * what a Rust `extern "C"` block in tang-compute / tang-infer would bind.  Each declaration names
 * the reference interface it stands in for (paths relative to the ecto/tang repository root).
 *
 * Conventions
 *   - "dev" pointers are CUDA device pointers valid on the context's GPU; "host" pointers are
 *     ordinary host memory.  Matrices are row-major.
 *   - All work is issued on the context's stream and is asynchronous unless the name ends in
 *     _host or the comment says it synchronises.
 *   - The library has no CPU fallback: without a usable CUDA device tq_ctx_create fails.
 */
#ifndef TANGQ_H_
#define TANGQ_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TQ_API __attribute__((visibility("default")))
#else
#define TQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tq_ctx tq_ctx;         /* one per (host thread, GPU): stream, workspace, error state */
typedef struct tq_qweight tq_qweight; /* a quantised weight matrix resident in HBM */

typedef enum tq_status {
  TQ_OK = 0,
  TQ_EINVAL = 1,       /* bad argument (the reference panics via assert!, e.g. quantize.rs:228-231) */
  TQ_ECUDA = 2,        /* a CUDA runtime call failed; see tq_last_error */
  TQ_ENCCL = 3,        /* a NCCL call failed */
  TQ_ETIMEOUT = 4,     /* a kernel gave up a bounded wait and recorded a device error code */
  TQ_ENOMEM = 5,
  TQ_EUNSUPPORTED = 6
} tq_status;

typedef enum tq_dtype { TQ_F32 = 0, TQ_BF16 = 1, TQ_F16 = 2, TQ_I8 = 3, TQ_U8 = 4, TQ_I32 = 5, TQ_F64 = 6 } tq_dtype;

/* Weight formats.  Q4/Q8 blocks are tang-infer's: 32 weights along K share one scale; a Q4 byte
 * holds k=2i in its low nibble and k=2i+1 in its high nibble, each stored as q+8
 * (crates/tang-infer/src/quantize.rs:11-31,110-111). */
typedef enum tq_qkind {
  TQ_Q4_F32 = 0, /* Q4Block: f32 scale per block (quantize.rs:25-31) */
  TQ_Q4_F16 = 1, /* same blocks, scale narrowed to IEEE half */
  TQ_Q8_F32 = 2, /* Q8Block: f32 scale + 32 x i8 (quantize.rs:15-20) */
  TQ_I8_ROW = 3  /* int8 [rows, cols] with one f32 scale per output row */
} tq_qkind;

/* ---- context --------------------------------------------------------------------------------
 * Stands in for CudaComputeDevice::new (crates/tang-compute/src/cuda.rs:151-179): one device,
 * one stream.  `stream` is a cudaStream_t to adopt, or NULL to create a private non-blocking one. */
TQ_API int tq_ctx_create(int device, void* stream, tq_ctx** out);
TQ_API int tq_ctx_destroy(tq_ctx* ctx);
/* Text of the last failure on this context (never NULL). */
TQ_API const char* tq_last_error(const tq_ctx* ctx);
/* ComputeDevice::sync (crates/tang-compute/src/device.rs:367): waits for the stream, then reports
 * any error code a kernel recorded (TQ_ETIMEOUT) and clears it. */
TQ_API int tq_sync(tq_ctx* ctx);
TQ_API void* tq_ctx_stream(tq_ctx* ctx);
TQ_API int tq_version(void);

/* ---- raw buffers ----------------------------------------------------------------------------
 * ComputeDevice::alloc / upload / download (device.rs:33-60; cuda.rs:1078-1133).  upload and
 * download synchronise, like the reference's. */
TQ_API int tq_buf_alloc(tq_ctx* ctx, size_t bytes, void** dev_out);
TQ_API int tq_buf_free(tq_ctx* ctx, void* dev);
TQ_API int tq_upload(tq_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
TQ_API int tq_download(tq_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
TQ_API int tq_memset(tq_ctx* ctx, void* dst_dev, int byte, size_t bytes);
/* dtype conversion on device: f32 <-> bf16 with the reference's round-to-nearest-even
 * (crates/tang-compute/src/kernels/util_cuda.rs:7-40; cuda.rs:22-31). */
TQ_API int tq_convert(tq_ctx* ctx, const void* src_dev, int src_dtype, void* dst_dev, int dst_dtype, size_t n);

/* ---- quantised weights ----------------------------------------------------------------------
 * Upload of a QuantizedQ4 / QuantizedQ8 (quantize.rs:34-44), shape [rows, cols], blocks in
 * row-major order, ceil(cols/32) per row (quantize.rs:193-220).
 *
 * tq_qweight_from_blocks takes the array-of-structs wire form: per block a little-endian f32
 * scale followed by the 16 (Q4) or 32 (Q8) payload bytes — 20 / 36 bytes per block, no padding.
 * kind must be TQ_Q4_F32 or TQ_Q8_F32. */
TQ_API int tq_qweight_from_blocks(tq_ctx* ctx, int kind, const void* blocks_host, size_t rows, size_t cols,
                           tq_qweight** out);
/* Structure-of-arrays host form: payload [rows][ceil(cols/32)*16] (Q4) or [rows][ceil(cols/32)*32]
 * (Q8) or [rows][cols] (TQ_I8_ROW); scales [rows][ceil(cols/32)] as f32 or f16 bits, or [rows]
 * f32 for TQ_I8_ROW. */
TQ_API int tq_qweight_from_arrays(tq_ctx* ctx, int kind, const void* payload_host, const void* scales_host, size_t rows,
                           size_t cols, tq_qweight** out);
/* The same structure-of-arrays form, but already in HBM (payload 8-byte, scales 4-byte aligned).
 * The arrays are read once and can be freed after the next tq_sync.
 *
 * All three constructors regroup the numbers into the library's device layout (16-row x 128-k
 * fragment tiles, see csrc/qlayout.cuh); integer codes and scale bits are copied unchanged. */
TQ_API int tq_qweight_from_device_arrays(tq_ctx* ctx, int kind, const void* payload_dev, const void* scales_dev,
                                         size_t rows, size_t cols, tq_qweight** out);
TQ_API int tq_qweight_free(tq_ctx* ctx, tq_qweight* w);
TQ_API int tq_qweight_shape(const tq_qweight* w, size_t* rows, size_t* cols, int* kind);
TQ_API size_t tq_qweight_bytes(const tq_qweight* w); /* payload + scale bytes one matvec has to stream */

/* dequantize_q4 / dequantize_q8 (quantize.rs:73-81,121-132): out_dev f32 [rows, cols] =
 * (integer as f32) * scale.  With ints_dev != NULL also writes the signed integers (i8
 * [rows, cols]) so the unpack can be checked bit for bit. */
TQ_API int tq_dequantize(tq_ctx* ctx, const tq_qweight* w, float* out_dev, int8_t* ints_dev);

/* ---- quantised linear -----------------------------------------------------------------------
 * y[m, rows] = x[m, cols] . W^T for m activation rows.  This is q4_matvec / q8_matvec
 * (quantize.rs:227-289) at m = 1 and Linear::forward_2d -> matmul_b_transposed (crates/
 * tang-compute/src/modules.rs:56-70, device.rs:407-419) for a quantised W at m > 1.
 *   x_dtype: TQ_BF16 or TQ_F32 (f32 activations are used exactly, as three bf16 terms).
 *   y_dtype: TQ_F32 or TQ_BF16.   ldx / ldy: row strides in elements (0 = dense).
 *   residual_dev: optional f32 [m, rows] (stride ldy) added to the result; may equal y_dev when
 *   y is f32.  Products are exact; accumulation is f32. */
TQ_API int tq_qlinear(tq_ctx* ctx, const tq_qweight* w, const void* x_dev, int x_dtype, size_t ldx, size_t m, void* y_dev,
               int y_dtype, size_t ldy, const float* residual_dev);

/* The reference call itself: q4_matvec(&QuantizedQ4, &[f64]) -> Vec<f64> (quantize.rs:256) and
 * q8_matvec (quantize.rs:227), with HOST vectors.  x_host [m, cols], y_host [m, rows]; dtype is
 * TQ_F64 (the reference's), TQ_F32 or TQ_BF16 (bit patterns) for both.  f64 input is narrowed to
 * f32 (on the device, after upload).  Synchronises. */
TQ_API int tq_q_matvec_host(tq_ctx* ctx, const tq_qweight* w, const void* x_host, void* y_host, int dtype, size_t m);

/* Launch-shape override for tq_qlinear, for tuning runs: rows-per-CTA = 16*wr, K slices = wk,
 * ring depth = stages, 128-k tiles per warp and stage = tiles_per_warp.  wr = 0 restores the
 * built-in choice. */
TQ_API int tq_qlinear_set_config(tq_ctx* ctx, int wr, int wk, int stages, int tiles_per_warp);

/* ---- CUDA graphs ------------------------------------------------------------------------------
 * CudaComputeDevice::begin_capture / end_capture (crates/tang-compute/src/cuda.rs:344-356): every
 * asynchronous call made on the context between begin and end is recorded instead of run, and
 * replayed by tq_graph_launch.  Calls that allocate or synchronise (uploads, downloads, _host
 * calls, the first tq_qlinear that needs a larger staging buffer) must not be made while
 * capturing: run the sequence once eagerly first. */
typedef struct tq_graph tq_graph;
TQ_API int tq_graph_begin(tq_ctx* ctx);
TQ_API int tq_graph_end(tq_ctx* ctx, tq_graph** out);
TQ_API int tq_graph_launch(tq_ctx* ctx, tq_graph* graph);
TQ_API int tq_graph_free(tq_ctx* ctx, tq_graph* graph);
/* Kernels launched through this context so far (graph replays count their recorded kernels). */
TQ_API unsigned long long tq_launch_count(const tq_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* TANGQ_H_ */
