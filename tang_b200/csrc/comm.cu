// Collectives at the shard boundaries of tensor-/expert-/head-parallel decode (include/tangq.h,
// tq_comm_*).  The reference has no intra-node collective (its tang-mesh crate averages over QUIC,
// crates/tang-mesh/src/allreduce.rs:43-70), so these stand in for the sums a sharded
// Linear::forward_2d needs.  NCCL is resolved at run time with dlopen: a single-GPU process never
// needs it, and a process that already loaded a NCCL (e.g. through torch) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <new>

#include "common.cuh"
#include "internal.h"

// ---------------------------------------------------------------------------------------------
// One-shot all-reduce over peer memory, for the small sums of tensor-parallel decode (a [batch, d_model] f32
// partial per row-parallel layer: 16 KB to 1 MB).  At these sizes a library all-reduce is bound by its launch and
// protocol latency, not by NVLink.  Here every rank owns a buffer that all ranks have mapped (CUDA IPC):
//   [2 parities][world ranks][max_elems] f32  +  [2][world] flag words.
// One kernel per rank: it stores its partial into slot (parity, own rank) of EVERY rank's buffer with plain stores
// (through NVLink for the peers), raises its flag in every buffer with a system-scope release once all of its
// CTAs have finished storing, waits — bounded — until every rank's flag in its OWN buffer carries the current
// sequence number, and adds the world partials it now holds locally in rank order (every rank forms the same sum,
// bit for bit).  No loads cross NVLink, no multicast, no TMA.  The parity alternates per call, which is enough:
// a rank can only be two calls ahead of a peer once that peer has raised its flag for the call in between, i.e.
// after the peer finished reading the buffer of the call before.  The sequence number lives in device memory and
// is advanced by the kernel, so a recorded graph replays correctly.
// A peer that never arrives makes the wait run out: the kernel records DERR_PEER_WAIT, leaves the output as it
// was, and the next tq_sync reports TQ_ETIMEOUT.
// ---------------------------------------------------------------------------------------------
constexpr int kPeerMaxWorld = 8;

struct PeerGroup {
  int world = 1, rank = 0;
  size_t max_elems = 0;
  float* bufs[kPeerMaxWorld] = {};     // every rank's buffer as mapped in this process (bufs[rank] is the local one)
  bool opened[kPeerMaxWorld] = {};     // mapped with cudaIpcOpenMemHandle (to be closed)
  bool owns_local = false;
  unsigned* state = nullptr;           // device: [0] sequence number, [1] CTAs done storing, [2] CTAs done reading
  unsigned poll_limit = 1u << 22;      // polls of one flag before giving up (each a system-scope load)
};

struct tq_comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  PeerGroup* peer = nullptr;
};

namespace tq {

struct PeerArParams {
  float* bufs[kPeerMaxWorld];
  int world, rank;
  size_t max_elems, n;
  float* io;
  unsigned* state;
  int* err;
  unsigned poll_limit;
};

__host__ __device__ inline size_t peer_data_floats(int world, size_t max_elems) { return (size_t)2 * world * max_elems; }

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const PeerArParams p) {
  pdl_wait();                 // io is the previous kernel's output
  pdl_launch_dependents();
  __shared__ int s_fail;
  const unsigned seq = p.state[0] + 1u;          // (advanced only after every CTA has read it, below)
  const unsigned parity = seq & 1u;
  const size_t n4 = p.n / 4;                     // n is a multiple of 4
  const size_t slot = ((size_t)parity * p.world + p.rank) * p.max_elems;
  if (threadIdx.x == 0) s_fail = 0;
  // ---- store this rank's partial into every rank's buffer
  const float4* src = reinterpret_cast<const float4*>(p.io);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = src[i];
    for (int r = 0; r < p.world; ++r) reinterpret_cast<float4*>(p.bufs[r] + slot)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned arrived = atomicAdd(&p.state[1], 1u);
    if (arrived == gridDim.x - 1) {              // every CTA of this rank has stored and fenced
      p.state[1] = 0;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r) {
        int* flag = reinterpret_cast<int*>(p.bufs[r] + peer_data_floats(p.world, p.max_elems)) + parity * p.world + p.rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"((int)seq) : "memory");
      }
    }
  }
  // ---- wait for every rank's flag in the local buffer
  if (threadIdx.x < p.world) {
    const int* flag = reinterpret_cast<const int*>(p.bufs[p.rank] + peer_data_floats(p.world, p.max_elems)) + parity * p.world + threadIdx.x;
    unsigned polls = 0;
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v == (int)seq) break;
      if (++polls > p.poll_limit) {
        s_fail = 1;
        atomicCAS(p.err, 0, (int)DERR_PEER_WAIT);
        break;
      }
    }
  }
  __syncthreads();
  // ---- add the partials in rank order (skipped when a peer never arrived: io keeps this rank's partial)
  if (!s_fail) {
    const float* base = p.bufs[p.rank] + (size_t)parity * p.world * p.max_elems;
    float4* dst = reinterpret_cast<float4*>(p.io);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
      float4 acc = __ldcg(reinterpret_cast<const float4*>(base) + i);
      for (int r = 1; r < p.world; ++r) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (size_t)r * p.max_elems) + i);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      dst[i] = acc;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned finished = atomicAdd(&p.state[2], 1u);
    if (finished == gridDim.x - 1) {             // every CTA has read the sequence number and its flags
      p.state[2] = 0;
      p.state[0] = seq;
    }
  }
}

}  // namespace tq

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  bool ok = false;
};

NcclApi& api() {
  static NcclApi a;
  static bool tried = false;
  if (tried) return a;
  tried = true;
  a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!a.handle) return a;
#define TQ_SYM(field, name)                                         \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.handle, name)); \
  if (!a.field) return a;
  TQ_SYM(GetUniqueId, "ncclGetUniqueId")
  TQ_SYM(CommInitRank, "ncclCommInitRank")
  TQ_SYM(CommDestroy, "ncclCommDestroy")
  TQ_SYM(CommAbort, "ncclCommAbort")
  TQ_SYM(GetErrorString, "ncclGetErrorString")
  TQ_SYM(AllReduce, "ncclAllReduce")
  TQ_SYM(AllGather, "ncclAllGather")
  TQ_SYM(Send, "ncclSend")
  TQ_SYM(Recv, "ncclRecv")
  TQ_SYM(GroupStart, "ncclGroupStart")
  TQ_SYM(GroupEnd, "ncclGroupEnd")
#undef TQ_SYM
  a.ok = true;
  return a;
}

int nccl_fail(tq_ctx* ctx, const char* what, ncclResult_t r) {
  return tq::fail(ctx, TQ_ENCCL, "%s failed: %s", what, api().GetErrorString ? api().GetErrorString(r) : "?");
}

#define TQ_NCCL(ctx, expr)                                   \
  do {                                                       \
    ncclResult_t r__ = (expr);                               \
    if (r__ != ncclSuccess) return nccl_fail((ctx), #expr, r__); \
  } while (0)

}  // namespace

using namespace tq;

static void peer_free(tq_comm* comm) {
  PeerGroup* g = comm ? comm->peer : nullptr;
  if (!g) return;
  for (int r = 0; r < g->world; ++r)
    if (g->opened[r] && g->bufs[r]) cudaIpcCloseMemHandle(g->bufs[r]);
  if (g->owns_local && g->bufs[g->rank]) cudaFree(g->bufs[g->rank]);
  if (g->state) cudaFree(g->state);
  delete g;
  comm->peer = nullptr;
}

static int peer_setup_state(tq_ctx* ctx, PeerGroup* g) {
  TQ_CUDA(ctx, cudaMalloc(&g->state, 4 * sizeof(unsigned)));
  TQ_CUDA(ctx, cudaMemset(g->state, 0, 4 * sizeof(unsigned)));
  return TQ_OK;
}

extern "C" {

size_t tq_comm_peer_bytes(int world, size_t max_elems) {
  if (world < 1 || world > kPeerMaxWorld) return 0;
  return (peer_data_floats(world, max_elems) + 2 * (size_t)world) * sizeof(float);
}

int tq_comm_peer_local(tq_ctx* ctx, int rank, int world, void* const* peer_bufs_dev, size_t max_elems, tq_comm** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, out != nullptr, "tq_comm_peer_local: null output");
  *out = nullptr;
  TQ_REQUIRE(ctx, world >= 1 && world <= kPeerMaxWorld && rank >= 0 && rank < world, "tq_comm_peer_local: world must be 1..%d", kPeerMaxWorld);
  TQ_REQUIRE(ctx, peer_bufs_dev && max_elems > 0 && max_elems % 4 == 0, "tq_comm_peer_local: null buffers, or max_elems not a multiple of 4");
  for (int r = 0; r < world; ++r)
    TQ_REQUIRE(ctx, peer_bufs_dev[r] != nullptr && ((uintptr_t)peer_bufs_dev[r] & 15) == 0, "tq_comm_peer_local: buffer %d is null or not 16-byte aligned", r);
  tq_comm* c = new (std::nothrow) tq_comm();
  PeerGroup* g = new (std::nothrow) PeerGroup();
  if (!c || !g) {
    delete c;
    delete g;
    return fail(ctx, TQ_ENOMEM, "out of host memory");
  }
  c->rank = rank;
  c->world = world;
  c->peer = g;
  g->world = world;
  g->rank = rank;
  g->max_elems = max_elems;
  for (int r = 0; r < world; ++r) g->bufs[r] = static_cast<float*>(peer_bufs_dev[r]);
  if (int st = peer_setup_state(ctx, g)) {
    peer_free(c);
    delete c;
    return st;
  }
  *out = c;
  return TQ_OK;
}

int tq_comm_enable_peer(tq_ctx* ctx, tq_comm* comm, size_t max_elems) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, comm != nullptr && comm->comm != nullptr, "tq_comm_enable_peer: needs a live NCCL communicator (it carries the handle exchange)");
  TQ_REQUIRE(ctx, max_elems > 0 && max_elems % 4 == 0, "tq_comm_enable_peer: max_elems must be a positive multiple of 4");
  if (comm->world == 1 || comm->world > kPeerMaxWorld) return TQ_OK;   // nothing to exchange / left to NCCL
  if (comm->peer) peer_free(comm);
  PeerGroup* g = new (std::nothrow) PeerGroup();
  if (!g) return fail(ctx, TQ_ENOMEM, "out of host memory");
  g->world = comm->world;
  g->rank = comm->rank;
  g->max_elems = max_elems;
  comm->peer = g;
  auto bail = [&](int st) {
    peer_free(comm);
    return st;
  };
  const size_t bytes = tq_comm_peer_bytes(g->world, max_elems);
  float* local = nullptr;
  if (cudaMalloc(&local, bytes) != cudaSuccess) {
    cudaGetLastError();
    return bail(fail(ctx, TQ_ENOMEM, "tq_comm_enable_peer: %zu bytes of peer buffer", bytes));
  }
  g->bufs[g->rank] = local;
  g->owns_local = true;
  if (cudaMemset(local, 0, bytes) != cudaSuccess) return bail(fail(ctx, TQ_ECUDA, "tq_comm_enable_peer: memset failed"));
  if (int st = peer_setup_state(ctx, g)) return bail(st);
  // every rank's IPC handle to every rank, carried by the communicator's all-gather
  cudaIpcMemHandle_t mine;
  if (cudaIpcGetMemHandle(&mine, local) != cudaSuccess) {
    cudaGetLastError();
    return bail(fail(ctx, TQ_EUNSUPPORTED, "tq_comm_enable_peer: cudaIpcGetMemHandle failed"));
  }
  unsigned char* stage = nullptr;
  const size_t hb = sizeof(cudaIpcMemHandle_t);
  if (cudaMalloc(&stage, hb * (g->world + 1)) != cudaSuccess) return bail(fail(ctx, TQ_ENOMEM, "tq_comm_enable_peer: staging"));
  cudaMemcpy(stage, &mine, hb, cudaMemcpyHostToDevice);
  ncclResult_t nr = api().AllGather(stage, stage + hb, hb, ncclInt8, comm->comm, ctx->stream);
  cudaError_t ce = cudaStreamSynchronize(ctx->stream);
  cudaIpcMemHandle_t all[kPeerMaxWorld];
  if (nr == ncclSuccess && ce == cudaSuccess) ce = cudaMemcpy(all, stage + hb, hb * g->world, cudaMemcpyDeviceToHost);
  cudaFree(stage);
  if (nr != ncclSuccess || ce != cudaSuccess) return bail(fail(ctx, TQ_ENCCL, "tq_comm_enable_peer: handle exchange failed"));
  for (int r = 0; r < g->world; ++r) {
    if (r == g->rank) continue;
    void* ptr = nullptr;
    if (cudaIpcOpenMemHandle(&ptr, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      return bail(fail(ctx, TQ_EUNSUPPORTED, "tq_comm_enable_peer: rank %d's buffer cannot be mapped (no peer access?)", r));
    }
    g->bufs[r] = static_cast<float*>(ptr);
    g->opened[r] = true;
  }
  // nobody may start storing into a peer's buffer before that peer has zeroed it: one more exchange as a barrier
  if (cudaMalloc(&stage, (size_t)g->world + 1) != cudaSuccess) return bail(fail(ctx, TQ_ENOMEM, "tq_comm_enable_peer: staging"));
  nr = api().AllGather(stage, stage + 1, 1, ncclInt8, comm->comm, ctx->stream);
  ce = cudaStreamSynchronize(ctx->stream);
  cudaFree(stage);
  if (nr != ncclSuccess || ce != cudaSuccess) return bail(fail(ctx, TQ_ENCCL, "tq_comm_enable_peer: barrier failed"));
  return TQ_OK;
}

int tq_comm_set_wait_limit(tq_comm* comm, unsigned polls) {
  if (!comm || !comm->peer || polls == 0) return TQ_EINVAL;
  comm->peer->poll_limit = polls;
  return TQ_OK;
}

int tq_comm_unique_id(void* id_out128) {
  if (!id_out128) return TQ_EINVAL;
  if (!api().ok) return TQ_ENCCL;
  ncclUniqueId id;
  if (api().GetUniqueId(&id) != ncclSuccess) return TQ_ENCCL;
  memcpy(id_out128, &id, sizeof id);
  return TQ_OK;
}

int tq_comm_create(tq_ctx* ctx, const void* id128, int rank, int world, tq_comm** out) {
  if (int st = bind(ctx)) return st;
  TQ_REQUIRE(ctx, out != nullptr, "tq_comm_create: null output");
  *out = nullptr;
  TQ_REQUIRE(ctx, id128 != nullptr && world >= 1 && rank >= 0 && rank < world, "tq_comm_create: bad rank/world");
  if (!api().ok) return fail(ctx, TQ_ENCCL, "NCCL could not be loaded (libnccl.so.2)");
  tq_comm* c = new (std::nothrow) tq_comm();
  if (!c) return fail(ctx, TQ_ENOMEM, "out of host memory");
  c->rank = rank;
  c->world = world;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof id);
  ncclResult_t r = api().CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) {
    delete c;
    return nccl_fail(ctx, "ncclCommInitRank", r);
  }
  *out = c;
  return TQ_OK;
}

int tq_comm_destroy(tq_ctx* ctx, tq_comm* comm) {
  if (!comm) return TQ_OK;
  if (ctx) {
    bind(ctx);
    cudaStreamSynchronize(ctx->stream);
  }
  peer_free(comm);
  if (comm->comm && api().ok) api().CommDestroy(comm->comm);
  delete comm;
  return TQ_OK;
}

int tq_comm_abort(tq_comm* comm) {
  if (!comm) return TQ_OK;
  if (comm->comm && api().ok) api().CommAbort(comm->comm);
  comm->comm = nullptr;
  return TQ_OK;
}

int tq_comm_rank(const tq_comm* comm) { return comm ? comm->rank : 0; }
int tq_comm_world(const tq_comm* comm) { return comm ? comm->world : 1; }

int tq_all_reduce_f32(tq_ctx* ctx, tq_comm* comm, float* buf_dev, size_t n) {
  if (int st = bind(ctx)) return st;
  ctx->inflight_unknown = true;   // a library kernel follows: later launches assume nothing about what runs
  ctx->n_inflight = 0;
  if (!comm || comm->world == 1 || n == 0) return TQ_OK;
  TQ_REQUIRE(ctx, buf_dev != nullptr, "tq_all_reduce_f32: null buffer");
  if (comm->peer && n <= comm->peer->max_elems && n % 4 == 0 && ((uintptr_t)buf_dev & 15) == 0) {
    const PeerGroup* g = comm->peer;
    PeerArParams p;
    for (int r = 0; r < kPeerMaxWorld; ++r) p.bufs[r] = g->bufs[r];
    p.world = g->world;
    p.rank = g->rank;
    p.max_elems = g->max_elems;
    p.n = n;
    p.io = buf_dev;
    p.state = g->state;
    p.err = ctx->dev_err;
    p.poll_limit = g->poll_limit;
    size_t ctas = (n / 4 + 255) / 256;
    if (ctas > 64) ctas = 64;
    TQ_CUDA(ctx, launch_k(ctx, peer_allreduce_kernel, dim3((unsigned)ctas), dim3(256), 0, p));
    return TQ_OK;
  }
  TQ_REQUIRE(ctx, comm->comm != nullptr, "tq_all_reduce_f32: aborted communicator");
  TQ_NCCL(ctx, api().AllReduce(buf_dev, buf_dev, n, ncclFloat, ncclSum, comm->comm, ctx->stream));
  return TQ_OK;
}

int tq_all_gather(tq_ctx* ctx, tq_comm* comm, const void* send_dev, void* recv_dev, size_t bytes_per_rank) {
  if (int st = bind(ctx)) return st;
  ctx->inflight_unknown = true;   // a library kernel follows: later launches assume nothing about what runs
  ctx->n_inflight = 0;
  if (bytes_per_rank == 0) return TQ_OK;
  TQ_REQUIRE(ctx, send_dev && recv_dev, "tq_all_gather: null buffer");
  if (!comm || comm->world == 1) {
    if (send_dev != recv_dev)
      TQ_CUDA(ctx, cudaMemcpyAsync(recv_dev, send_dev, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
    return TQ_OK;
  }
  TQ_REQUIRE(ctx, comm->comm != nullptr, "tq_all_gather: aborted communicator");
  TQ_NCCL(ctx, api().AllGather(send_dev, recv_dev, bytes_per_rank, ncclInt8, comm->comm, ctx->stream));
  return TQ_OK;
}

int tq_all_to_all(tq_ctx* ctx, tq_comm* comm, const void* send_dev, void* recv_dev, size_t bytes_per_peer) {
  if (int st = bind(ctx)) return st;
  ctx->inflight_unknown = true;   // a library kernel follows: later launches assume nothing about what runs
  ctx->n_inflight = 0;
  if (bytes_per_peer == 0) return TQ_OK;
  TQ_REQUIRE(ctx, send_dev && recv_dev, "tq_all_to_all: null buffer");
  if (!comm || comm->world == 1) {
    if (send_dev != recv_dev)
      TQ_CUDA(ctx, cudaMemcpyAsync(recv_dev, send_dev, bytes_per_peer, cudaMemcpyDeviceToDevice, ctx->stream));
    return TQ_OK;
  }
  TQ_REQUIRE(ctx, comm->comm != nullptr, "tq_all_to_all: aborted communicator");
  TQ_NCCL(ctx, api().GroupStart());
  for (int peer = 0; peer < comm->world; ++peer) {
    const char* s = static_cast<const char*>(send_dev) + (size_t)peer * bytes_per_peer;
    char* r = static_cast<char*>(recv_dev) + (size_t)peer * bytes_per_peer;
    TQ_NCCL(ctx, api().Send(s, bytes_per_peer, ncclInt8, peer, comm->comm, ctx->stream));
    TQ_NCCL(ctx, api().Recv(r, bytes_per_peer, ncclInt8, peer, comm->comm, ctx->stream));
  }
  TQ_NCCL(ctx, api().GroupEnd());
  return TQ_OK;
}

}  // extern "C"

namespace tq {
// All-to-all with a different amount per peer (sizes known on the host): rank p's send_bytes[p'] bytes at
// send_off[p'] go to rank p', which receives them at its recv_off[p].  One grouped NCCL call.
int all_to_all_v(tq_ctx* ctx, tq_comm* comm, const void* send_dev, const size_t* send_off, const size_t* send_bytes, void* recv_dev,
                 const size_t* recv_off, const size_t* recv_bytes) {
  if (int st = bind(ctx)) return st;
  ctx->inflight_unknown = true;
  ctx->n_inflight = 0;
  TQ_REQUIRE(ctx, comm && comm->world > 1 && comm->comm != nullptr, "all_to_all_v: needs a live communicator of several ranks");
  TQ_NCCL(ctx, api().GroupStart());
  for (int peer = 0; peer < comm->world; ++peer) {
    if (send_bytes[peer])
      TQ_NCCL(ctx, api().Send(static_cast<const char*>(send_dev) + send_off[peer], send_bytes[peer], ncclInt8, peer, comm->comm, ctx->stream));
    if (recv_bytes[peer])
      TQ_NCCL(ctx, api().Recv(static_cast<char*>(recv_dev) + recv_off[peer], recv_bytes[peer], ncclInt8, peer, comm->comm, ctx->stream));
  }
  TQ_NCCL(ctx, api().GroupEnd());
  return TQ_OK;
}
}  // namespace tq

