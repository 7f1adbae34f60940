// Collectives at the shard boundaries of tensor-/expert-/head-parallel decode (include/tangq.h,
// tq_comm_*).  The reference has no intra-node collective (its tang-mesh crate averages over QUIC,
// crates/tang-mesh/src/allreduce.rs:43-70), so these stand in for the sums a sharded
// Linear::forward_2d needs.  NCCL is resolved at run time with dlopen: a single-GPU process never
// needs it, and a process that already loaded a NCCL (e.g. through torch) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <new>

#include "internal.h"

struct tq_comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
};

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

extern "C" {

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
  TQ_REQUIRE(ctx, buf_dev != nullptr && comm->comm != nullptr, "tq_all_reduce_f32: null buffer or aborted communicator");
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
