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
/* quantize_matrix_q4 / quantize_matrix_q8 (crates/tang-infer/src/quantize.rs:193-220, with quantize_q4/q8 :47-118)
 * on the device: `src` is the [rows, cols] matrix as it comes out of a checkpoint (f32, bf16 or f16, widened to
 * f32 exactly, crates/tang-safetensors/src/lib.rs:262-297; ld = row stride in elements, 0 = dense), `kind` is
 * TQ_Q4_F32 or TQ_Q8_F32.  Scales and integer codes are the reference's bit for bit (scale = amax/7 or amax/127,
 * 1.0 for a zero block, round half away from zero, clamp, ragged tail padded with zeros). */
TQ_API int tq_quantize_matrix(tq_ctx* ctx, const void* src_dev, int src_dtype, size_t ld, size_t rows, size_t cols, int kind,
                              tq_qweight** out);
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

/* The same call without the final wait, for a caller with several matvecs to run (a list of layers, a batch of
 * independent requests): the upload, the kernel and the read-back are queued on the context's stream in call
 * order, and ONE tq_sync after the last call makes every y_host valid (and reports a device-side failure).  Both
 * vectors must stay alive and untouched until that tq_sync; pageable vectors make the copies themselves block, so
 * pinned ones (cudaHostAlloc / cudaHostRegister) are what this form is for -- a pinned y_host is written by the
 * kernel directly, and pinned bf16 / f32 x_host of up to eight rows are read by a small staging kernel through their
 * device alias instead of being copied.  The reference has no asynchronous form: this replaces a loop of
 * quantize.rs:256 calls.
 * With pinned vectors the call may be recorded between tq_graph_begin and tq_graph_end (after one eager call has set
 * the staging ring up): every tq_graph_launch then reads the vectors' current contents and writes the results again,
 * so a step of many matvecs costs the host one launch and one tq_sync. */
TQ_API int tq_q_matvec_host_async(tq_ctx* ctx, const tq_qweight* w, const void* x_host, void* y_host, int dtype, size_t m);

/* Row-wise concatenation of weights already on the device (same kind and column count; every part
 * but the last with a multiple of 16 rows): builds the fused [q;k;v] and [gate;up] projections
 * from the reference's separate matrices (weight order [wq, wk, wv, wo, gate, up, down],
 * crates/tang-mesh/src/inference.rs:1306-1413). */
TQ_API int tq_qweight_concat_rows(tq_ctx* ctx, const tq_qweight* const* parts, size_t n_parts, tq_qweight** out);

/* A fused [gate; up] projection (gate rows, then the same number of up rows) regrouped so that every 16-row block
 * holds eight gate rows and the eight up rows of the same outputs.  In that order the decode step applies
 * swiglu_fused_buf (crates/tang-compute/src/device.rs:727-736) inside the projection kernel and the 2 x ffn f32
 * intermediate never reaches HBM; tq_llama_set_layer accepts either order.  tq_qlinear on the result yields the
 * outputs in the regrouped order.  Integer codes and scale bits are copied unchanged; the source can be freed
 * after the next tq_sync. */
TQ_API int tq_qweight_interleave_gate_up(tq_ctx* ctx, const tq_qweight* w_gate_up, tq_qweight** out);

/* ---- small operators of the decode step ------------------------------------------------------
 * dtypes are TQ_F32 or TQ_BF16 throughout. */

/* ComputeDevice::rms_norm (crates/tang-compute/src/device.rs:121-128; cpu.rs:126-149) and, with
 * residual_dev != NULL, rms_norm_residual (device.rs:546-575): v = x + residual,
 * out = v / sqrt(mean(v^2) + eps) * weight, and v itself to sum_out_dev (f32, may alias
 * residual_dev) when that is non-NULL.  dim <= 8192. */
TQ_API int tq_rms_norm(tq_ctx* ctx, const void* x_dev, int x_dtype, const float* residual_dev, const void* weight_dev,
                       int w_dtype, size_t n_groups, size_t dim, float eps, void* out_dev, int out_dtype,
                       float* sum_out_dev);
/* InterleavedRoPE::new (crates/tang-compute/src/modules.rs:495-510): cos/sin tables
 * [max_seq_len, head_dim/2], computed in f64 on the host and stored as f32 on the device. */
TQ_API int tq_rope_tables(tq_ctx* ctx, size_t head_dim, size_t max_seq_len, double base, float* cos_dev, float* sin_dev);
/* ComputeDevice::rope_forward (device.rs:582-610): x [seq_len, n_heads, head_dim], pairs (2i, 2i+1)
 * rotated by the table row of position start_pos + s — or positions_dev[s] when that is non-NULL
 * (one decode token per sequence, each at its own position). */
TQ_API int tq_rope_forward(tq_ctx* ctx, const void* x_dev, int x_dtype, const float* cos_dev, const float* sin_dev,
                           const int* positions_dev, size_t seq_len, size_t n_heads, size_t head_dim, size_t start_pos,
                           void* out_dev, int out_dtype);
/* ComputeDevice::swiglu_fused_buf (device.rs:727-736): out[r, i] = silu(gate[r*ld + i]) * up[r*ld + i]
 * (ld = 0: dense).  gate and up may be the two halves of one fused projection. */
TQ_API int tq_swiglu(tq_ctx* ctx, const void* gate_dev, const void* up_dev, int in_dtype, size_t ld, size_t rows, size_t n,
                     void* out_dev, int out_dtype);
/* ComputeDevice::embedding (device.rs:131-138; cpu.rs:151-167): out[i, :] = weight[ids[i], :];
 * ids are int32 (the reference smuggles u32 bit patterns through an f32 buffer, cpu.rs:51-56). */
TQ_API int tq_embedding(tq_ctx* ctx, const void* weight_dev, int w_dtype, const int* ids_dev, size_t seq_len, size_t dim,
                        size_t vocab, void* out_dev, int out_dtype);
/* The greedy branch of Sampler::sample (crates/tang-infer/src/sampling.rs:108-111,183-194): the index of the
 * FIRST maximum of each row (strict '>' scan; NaN is never chosen).  x is f32 [slices][rows][cols] -- a
 * vocabulary gathered rank-major from `slices` tensor-parallel ranks, slices = 1 for a plain matrix -- and the
 * index written is slice * cols + column. */
TQ_API int tq_argmax_rows(tq_ctx* ctx, const float* x_dev, size_t slices, size_t rows, size_t cols, int* idx_out_dev);
/* Sampler::sample (crates/tang-infer/src/sampling.rs:86-158) for `rows` sequences at once, on the device:
 * repetition penalty (once per occurrence in the sequence's past tokens: positive logits divided, the others
 * multiplied), temperature (0 = greedy: first maximum), exp(l - max), top-k (entries equal to the k-th largest
 * survive; 0 = off), normalisation, top-p (descending probability, equal probabilities in index order, cut after
 * the first rank whose running sum reaches p; 1 = off), re-normalisation, and one step of the reference's LCG
 * (sampling.rs:72-79) per sequence for the categorical draw.  logits f32 [slices][rows][cols] as for
 * tq_argmax_rows.  rng_states [rows] are read and advanced (unused when temperature = 0).  past_tokens
 * [rows][past_ld] / past_lens [rows] may be null (no penalty).  While at most 1024 probabilities survive the
 * top-k filter, every sum whose order matters is formed in the reference's order. */
typedef struct tq_sampler_config {
  double temperature;
  uint64_t top_k;
  double top_p;
  double repetition_penalty;
} tq_sampler_config;
TQ_API int tq_sample(tq_ctx* ctx, const float* logits_dev, size_t slices, size_t rows, size_t cols, const tq_sampler_config* cfg,
                     unsigned long long* rng_states_dev, const int* past_tokens_dev_or_null, const int* past_lens_dev_or_null,
                     size_t past_ld, int* tokens_out_dev);
/* The bookkeeping of `generate` (sampling.rs:229-256) between two decode steps, on the device: stores the chosen
 * tokens in out_tokens[row][*step], makes them the next step's input, adds one to every position, to *step and
 * (when given) to every entry of lens_io -- the per-sequence count of past tokens that tq_sample's repetition
 * penalty reads when out_tokens is the sequences' whole history and *step starts at the prompt length.
 * With the decode step and tq_argmax_rows / tq_sample in front of it, one captured graph generates a token per
 * replay and no logits leave the device.  rows <= 1024. */
TQ_API int tq_generate_advance(tq_ctx* ctx, const int* chosen_dev, size_t rows, int* tokens_io_dev, int* positions_io_dev,
                               int* out_tokens_dev, size_t out_ld, int* step_io_dev, int* lens_io_dev_or_null);

/* ---- attention -------------------------------------------------------------------------------
 * ComputeDevice::kv_attention (device.rs:161-180; cpu.rs:257-315) on f32 buffers, exactly the
 * reference's signature: q [q_len, n_heads*head_dim], caches [cache_start + q_len, n_kv_heads*
 * head_dim], query i attends positions 0..cache_start+i.  Any q_len; head_dim <= 256. */
TQ_API int tq_kv_attention(tq_ctx* ctx, const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                           size_t cache_start, size_t q_len, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                           float* out_dev);
/* The decode hot path: the same attention for ONE new token of each of `batch` sequences, bf16
 * q [batch, n_heads*128] and bf16 caches [batch][position][n_kv_heads*128] (sequence b starts at
 * element b*seq_stride; tang-infer's KVCache layout, crates/tang-infer/src/kv_cache.rs:12-24).
 * Sequence b attends positions 0..lens_dev[b]-1; max_len >= every length.  head_dim = 128,
 * n_heads/n_kv_heads <= 8.  out [batch, n_heads*128] bf16 or f32. */
TQ_API int tq_gqa_decode(tq_ctx* ctx, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev,
                         const int* lens_dev, size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                         size_t seq_stride, size_t max_len, void* out_dev, int out_dtype);

/* No counterpart in the reference.  tq_gqa_decode for callers that may not allocate device memory
 * (a serving loop that froze its allocator after start-up, a callback that only owns a stream):
 * same arguments and results, but the per-split partial results live in a fixed 3 MiB array inside
 * the library instead of the context's growable workspace, and the call never reaches cudaMalloc
 * or cudaFree.  It fails with TQ_EINVAL when batch x heads x splits needs more than that.  The
 * first call on a device looks the array's address up and sets a kernel attribute: make it before
 * any stream capture.  All calls on a device share the array — keep them ordered; two that overlap
 * on the GPU corrupt each other's partials. */
TQ_API int tq_gqa_decode_noalloc(tq_ctx* ctx, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev,
                                 const int* lens_dev, size_t batch, size_t n_heads, size_t n_kv_heads,
                                 size_t head_dim, size_t seq_stride, size_t max_len, void* out_dev, int out_dtype);
/* The same attention for a chunk of q_len new positions per sequence (prefill; kv_attention with q_len > 1,
 * device.rs:161-180): q bf16 [batch][q_len][n_heads*128]; query i of sequence b attends cache positions
 * 0 .. cache_start[b] + i, the chunk's own K/V rows being in the cache already; out [batch][q_len][n_heads*128]
 * bf16 or f32.  Probabilities enter the tensor core as bf16 (results to the bf16 bar).  n_heads/n_kv_heads in
 * {1, 2, 4, 8}. */
TQ_API int tq_gqa_prefill(tq_ctx* ctx, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev,
                          const int* cache_start_dev, size_t batch, size_t q_len, size_t n_heads, size_t n_kv_heads,
                          size_t head_dim, size_t seq_stride, void* out_dev, int out_dtype);

/* ---- collectives -----------------------------------------------------------------------------
 * NCCL over NVLink at the shard boundaries (the reference's only collective is a star sum over
 * QUIC, crates/tang-mesh/src/allreduce.rs:43-70).  One communicator per context; calls are
 * issued on the context's stream.  tq_comm_unique_id fills 128 bytes that rank 0 shares with the
 * other ranks by any host-side means. */
typedef struct tq_comm tq_comm;
TQ_API int tq_comm_unique_id(void* id_out128);
TQ_API int tq_comm_create(tq_ctx* ctx, const void* id128, int rank, int world, tq_comm** out);
TQ_API int tq_comm_destroy(tq_ctx* ctx, tq_comm* comm);
/* Tears the communicator down from the host without waiting for peers (ncclCommAbort); later
 * collective calls on it fail with TQ_EINVAL. */
TQ_API int tq_comm_abort(tq_comm* comm);
TQ_API int tq_comm_rank(const tq_comm* comm);
TQ_API int tq_comm_world(const tq_comm* comm);
/* Sum of buf_dev [n] f32 over the ranks, in place (the coordinator's sum of crates/tang-mesh/src/allreduce.rs:43-70,
 * with every rank ending up with the result).  NCCL, unless the communicator has the peer-memory path below and
 * n fits it: then one kernel per rank stores its partial into every rank's buffer, waits (bounded) for the others'
 * flags and adds the partials in rank order -- every rank gets the same bits.  A peer that never arrives turns
 * into TQ_ETIMEOUT at the next tq_sync, with buf_dev left as this rank's own partial. */
TQ_API int tq_all_reduce_f32(tq_ctx* ctx, tq_comm* comm, float* buf_dev, size_t n);
/* Gives the communicator the peer-memory path for sums of up to max_elems floats (a multiple of 4): allocates
 * this rank's buffer, exchanges CUDA IPC handles through the communicator and maps every peer's buffer.  Collective:
 * every rank calls it with the same max_elems.  Ranks must be separate processes on GPUs with peer access (NVLink).
 * With world = 1 or more than 8 ranks it does nothing.  No reference counterpart (tang-mesh sums over QUIC). */
TQ_API int tq_comm_enable_peer(tq_ctx* ctx, tq_comm* comm, size_t max_elems);
/* The same path over buffers the caller has already made visible to this GPU (its own symmetric-memory
 * allocator, or a test): peer_bufs_dev[r] is rank r's buffer as addressed from this device, each of
 * tq_comm_peer_bytes(world, max_elems) bytes, zeroed before the first sum.  The communicator only supports
 * tq_all_reduce_f32 of at most max_elems floats. */
TQ_API int tq_comm_peer_local(tq_ctx* ctx, int rank, int world, void* const* peer_bufs_dev, size_t max_elems, tq_comm** out);
TQ_API size_t tq_comm_peer_bytes(int world, size_t max_elems);
/* How many times the peer path looks at a peer's flag before it gives up (default 4 Mi looks, a few seconds). */
TQ_API int tq_comm_set_wait_limit(tq_comm* comm, unsigned polls);
TQ_API int tq_all_gather(tq_ctx* ctx, tq_comm* comm, const void* send_dev, void* recv_dev, size_t bytes_per_rank);
TQ_API int tq_all_to_all(tq_ctx* ctx, tq_comm* comm, const void* send_dev, void* recv_dev, size_t bytes_per_peer);

/* ---- Llama-shaped decode step ----------------------------------------------------------------
 * The reference's decode loop (crates/tang-train/examples/smollm.rs:215-296) for `batch`
 * sequences at once, one new token each, KV cache resident in HBM.  Dimensions in the config are
 * the WHOLE model's; with a communicator of size n each rank holds n_heads/n, n_kv_heads/n,
 * ffn/n and vocab/n and is given weights of those shard shapes:
 *   wqkv [ (n_heads + 2 n_kv_heads)/n * head_dim, d_model ]   rows = this rank's q heads, k heads, v heads
 *   wo   [ d_model, n_heads/n * head_dim ]                    columns = this rank's heads
 *   wgate_up [ 2 ffn/n, d_model ] (gate rows then up rows)    wdown [ d_model, ffn/n ]
 *   lm_head [ vocab/n, d_model ]
 * Norm gains and the embedding table are bf16 and replicated.  Weight handles are borrowed. */
typedef struct tq_llama tq_llama;
typedef struct tq_llama_config {
  uint32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn, vocab;
  uint32_t max_seq;   /* cache positions per sequence */
  uint32_t max_batch; /* sequences (<= 64) */
  float eps;          /* RMSNorm epsilon (1e-5 in smollm.rs:29) */
  double rope_base;   /* RoPE theta */
} tq_llama_config;
TQ_API int tq_llama_create(tq_ctx* ctx, const tq_llama_config* cfg, tq_comm* comm_or_null, tq_llama** out);
TQ_API int tq_llama_destroy(tq_llama* model);
TQ_API int tq_llama_set_layer(tq_llama* model, size_t layer, const tq_qweight* wqkv, const tq_qweight* wo,
                              const tq_qweight* wgate_up, const tq_qweight* wdown, const void* attn_norm_bf16_dev,
                              const void* ffn_norm_bf16_dev);
TQ_API int tq_llama_set_head(tq_llama* model, const void* embed_bf16_dev, const void* final_norm_bf16_dev,
                             const tq_qweight* lm_head);
/* This rank's bf16 caches of one layer, [max_batch][max_seq][n_kv_heads/n * head_dim], so a caller
 * can prefill them; seq_stride_elems = elements between sequences. */
TQ_API int tq_llama_kv_cache(tq_llama* model, size_t layer, void** k_cache_dev, void** v_cache_dev,
                             size_t* seq_stride_elems);
/* KVCache::trim_to (crates/tang-infer/src/kv_cache.rs:138-149), for every layer and for each of `batch` sequences
 * at once: seq_lens_io_dev[b] is the number of positions sequence b holds (its next position); a sequence that
 * holds more than `keep` drops its OLDEST positions -- rows [len - keep, len) of its K and V caches move to
 * [0, keep) -- and its length becomes `keep`; shorter sequences are untouched.  The K rows keep the rotation of
 * the positions they were appended at, exactly as the reference's trimmed cache does.  Asynchronous. */
TQ_API int tq_llama_kv_trim(tq_llama* model, int* seq_lens_io_dev, size_t batch, size_t keep);
/* The f32 residual stream [max_batch, d_model] after the last tq_llama_decode (the input of the final norm). */
TQ_API int tq_llama_hidden(tq_llama* model, float** hidden_dev);
/* One decode step: sequence b consumes token_ids_dev[b] at position positions_dev[b] (its k, v are
 * appended there) and attends positions 0..positions_dev[b].  max_len > every position.
 * logits_dev: f32 [batch, vocab] for one rank; with n ranks [n][batch][vocab/n] (rank-major
 * vocabulary slices).  Asynchronous; capturable once run eagerly. */
TQ_API int tq_llama_decode(tq_llama* model, const int* token_ids_dev, const int* positions_dev, size_t batch,
                           size_t max_len, float* logits_dev);
/* The same step for caches that have been trimmed (tq_llama_kv_trim): sequence b's K/V are appended at cache row
 * positions_dev[b] and positions 0..positions_dev[b] are attended, but the rotation of its q and k uses
 * rope_positions_dev[b], the caller's running position count (model.forward(&[tok], cache, pos) with a cache whose
 * seq_len is no longer pos, smollm.rs:535 + kv_cache.rs:138-149).  Both stay below max_seq.  NULL rope positions =
 * tq_llama_decode. */
TQ_API int tq_llama_decode_at(tq_llama* model, const int* token_ids_dev, const int* positions_dev, const int* rope_positions_dev,
                              size_t batch, size_t max_len, float* logits_dev);
/* The same step for a chunk of q_len new tokens per sequence (prompt processing): token_ids [batch][q_len],
 * sequence b's chunk starts at position cache_start[b] (its earlier positions are in the cache already).
 * Appends the chunk's K/V rows, runs causal attention over cache + chunk (tq_gqa_prefill) and the linear layers
 * on all batch*q_len rows at once; logits [batch, vocab] (gathered as for tq_llama_decode) are those of each
 * sequence's LAST chunk position.  Workspaces grow on first use: not inside a graph capture. */
TQ_API int tq_llama_prefill(tq_llama* model, const int* token_ids_dev, const int* cache_start_dev, size_t batch, size_t q_len,
                            float* logits_dev);

/* ---- mixture-of-experts FFN -------------------------------------------------------------------
 * No counterpart in the reference (it has no MoE); composed from its primitives.  Router: logits =
 * h . Wg^T in f64 (ascending k), top_k experts by (logit descending, index ascending), weights =
 * softmax over ALL experts (optionally renormalised over the chosen ones).  Expert: down(bf16(
 * silu(gate h) * (up h))) with int4/int8 block weights.  out = sum_chosen w_e expert_e(h) + sum
 * shared experts. */
TQ_API int tq_moe_router(tq_ctx* ctx, const void* h_bf16_dev, const void* wg_bf16_dev, size_t n_tokens, size_t d_model,
                         size_t n_experts, size_t top_k, int renormalize, int* idx_out_dev, float* weight_out_dev,
                         double* logits_out_dev);
typedef struct tq_moe tq_moe;
typedef struct tq_moe_config {
  uint32_t d_model, ffn, n_experts, top_k, n_shared;
  uint32_t renormalize;      /* 1: divide the chosen weights by their sum */
  uint32_t ep_rank, ep_size; /* this rank holds experts [ep_rank, ep_rank+1) * n_experts / ep_size */
} tq_moe_config;
/* Stacked weights: this rank's experts concatenated by rows (tq_qweight_concat_rows): gate|up
 * [n_local * 2*ffn, d_model] (per expert: gate rows then up rows) and down [n_local * d_model, ffn].
 * Shared experts: n_shared pairs of fused gate|up [2*ffn, d_model] and down [d_model, ffn],
 * replicated.  Handles are borrowed. */
TQ_API int tq_moe_create(tq_ctx* ctx, const tq_moe_config* cfg, const void* wg_bf16_dev, const tq_qweight* w_gate_up_stacked,
                         const tq_qweight* w_down_stacked, const tq_qweight* const* shared_gate_up,
                         const tq_qweight* const* shared_down, tq_moe** out);
TQ_API int tq_moe_destroy(tq_moe* moe);
/* h bf16 [n_tokens, d_model] (the same on every rank) -> out f32 [n_tokens, d_model].  With a
 * communicator each rank adds its own experts' terms (and the shared experts for its slice of the
 * tokens) and the result is all-reduced.  idx_out / weight_out (optional): the router's choices,
 * [n_tokens, top_k]. */
TQ_API int tq_moe_ffn(tq_moe* moe, const void* h_bf16_dev, size_t n_tokens, float* out_dev, tq_comm* comm_or_null,
                      int* idx_out_dev, float* weight_out_dev);
/* The same layer with the tokens SHARDED over the expert-parallel ranks: every rank passes its own n_tokens
 * (>= 1, the SAME count on every rank: pad the shorter shards) rows and gets their outputs.  Each (token, choice) row travels to the rank that owns the expert
 * (all-to-all dispatch, padded to the worst case of n_tokens*top_k rows per peer so that the exchange has a
 * fixed size and can be captured in a graph), the owners run their experts on what arrived, and a second
 * all-to-all brings the f32 results back to be weighted and summed where the token lives; shared experts run
 * locally.  The communicator must have the layer's ep_size and ep_rank.  No reference counterpart.
 * From 256 (token, choice) rows per rank on, and when no graph capture is open (on ALL ranks alike), the ranks
 * exchange their per-peer row counts first and the call waits once for the stream to read them; rows, expert ids
 * and results then travel with their true sizes.  Results do not depend on which form ran. */
TQ_API int tq_moe_ffn_dispatch(tq_moe* moe, const void* h_bf16_dev, size_t n_tokens, float* out_dev, tq_comm* comm_or_null,
                               int* idx_out_dev_or_null, float* weight_out_dev_or_null);

/* ---- multi-head latent attention, decode ------------------------------------------------------
 * No counterpart in the reference (it has no MLA).  Absorbed form: the bf16 cache row of position j
 * is [c_j (kv_lora = 512) | r_j (rope = 64)], sequence b starting at element b*seq_stride;
 *   s_j = (q_lat . c_j + q_rope . r_j) * softmax_scale,   o_lat = sum_j softmax(s)_j c_j.
 * q_full [batch, n_heads, 576] bf16 holds q_lat | q_rope per head; o_lat [batch, n_heads, 512] bf16.
 * n_heads (per rank, when heads are sharded) must be a multiple of 16. */
TQ_API int tq_mla_decode(tq_ctx* ctx, const void* q_full_bf16_dev, const void* cache_bf16_dev, const int* lens_dev,
                         size_t batch, size_t n_heads, size_t kv_lora, size_t rope_dim, size_t seq_stride, size_t max_len,
                         float softmax_scale, void* o_lat_bf16_dev);
/* q_lat = W_qk[h] q_nope[h] for every head (int8 per-row weights stacked by rows,
 * [n_heads*512, nope_dim]) written as bf16 into q_full, with q_rope copied behind it.
 * q_nope [batch, n_heads, nope_dim], q_rope [batch, n_heads, 64] bf16; batch <= 64. */
TQ_API int tq_mla_absorb_q(tq_ctx* ctx, const tq_qweight* w_qk_stacked, const void* q_nope_bf16_dev,
                           const void* q_rope_bf16_dev, size_t batch, size_t n_heads, size_t nope_dim,
                           void* q_full_bf16_dev);
/* o[h] = W_uv[h] o_lat[h] (stacked [n_heads*v_dim, 512]); out [batch, n_heads, v_dim] f32 or bf16. */
TQ_API int tq_mla_unabsorb(tq_ctx* ctx, const tq_qweight* w_uv_stacked, const void* o_lat_bf16_dev, size_t batch,
                           size_t n_heads, size_t v_dim, void* out_dev, int out_dtype);

/* One MLA attention layer of a decode step, composed from the calls above (no reference counterpart):
 *   c_q = q_a h                      [q_lora]            (h bf16 [batch, d_model])
 *   c_q = rms_norm(c_q) * gain       when the layer has a gain (eps = norm_eps)
 *   q[h] = q_b[h] c_q                [nope_dim | 64] per head, the 64 rope dimensions rotated (interleaved pairs,
 *                                    device.rs:582-610) by the table row of the query's position lens[b] - 1
 *   o_lat = tq_mla_decode(absorb(q)) over the latent cache (which already holds the current token's row)
 *   out = W_O concat_h(W_uv[h] o_lat[h])  f32 [batch, d_model], summed over the ranks when heads are sharded.
 * All five weights are int8 with one f32 scale per row (any kind tq_qlinear takes works).  n_heads is THIS rank's
 * head count: q_b, W_qk and W_uv hold its heads' rows, W_O [d_model, n_heads * v_dim] its heads' columns; the
 * cache is replicated.  rope tables: tq_rope_tables(head_dim = 64, max_pos, ...).  The layer owns a workspace
 * for max_batch <= 64 rows, so tq_mla_layer_decode allocates nothing and can be captured in a graph. */
typedef struct tq_mla tq_mla;
typedef struct tq_mla_config {
  uint32_t d_model, n_heads, q_lora, kv_lora, nope_dim, rope_dim, v_dim, max_batch, max_pos;
  float norm_eps;
} tq_mla_config;
TQ_API int tq_mla_create(tq_ctx* ctx, const tq_mla_config* cfg, const tq_qweight* q_a, const void* q_a_norm_gain_bf16_dev_or_null,
                         const tq_qweight* q_b, const tq_qweight* w_qk_stacked, const tq_qweight* w_uv_stacked,
                         const tq_qweight* w_o, const float* rope_cos_dev, const float* rope_sin_dev, tq_mla** out);
TQ_API int tq_mla_destroy(tq_mla* layer);
TQ_API int tq_mla_layer_decode(tq_mla* layer, const void* h_bf16_dev, const void* cache_bf16_dev, const int* lens_dev, size_t batch,
                               size_t seq_stride, size_t max_len, tq_comm* comm_or_null, float* out_dev);

/* ---- CUDA graphs ------------------------------------------------------------------------------
 * CudaComputeDevice::begin_capture / end_capture (crates/tang-compute/src/cuda.rs:344-356): every
 * asynchronous call made on the context between begin and end is recorded instead of run, and
 * replayed by tq_graph_launch.  Calls that allocate or synchronise (uploads, downloads, _host
 * calls, the first tq_qlinear that needs a larger staging buffer) must not be made while
 * capturing: run the sequence once eagerly first.  The recorded kernels hold the addresses of the
 * context's workspaces; when a later call makes one of them grow (it is freed and reallocated),
 * tq_graph_launch of a graph recorded before that fails with TQ_EINVAL: record the graph again. */
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
