// The group of contexts a sharded index is searched by: one rank per GPU (one process per GPU, or one host thread
// per GPU of a single process), NCCL over NVLink / NVSwitch for the one exchange step of a search (the per-shard
// candidate lists, and for IVF-PQ the probed cells of the query slices).  The reference is a single process and
// has no counterpart; the row-sharded layout needs it.
//
// NCCL is bound at run time (dlopen of libnccl.so.2): a host that never shards does not need the library, and a
// process that has NCCL loaded already (a PyTorch host, for instance) shares that copy.
#include <dlfcn.h>

#include <mutex>

#include "internal.h"

namespace fv {
namespace {

// the part of NCCL's C interface this file uses (nccl.h: ncclResult_t is an enum with ncclSuccess = 0,
// ncclUniqueId is 128 opaque bytes, ncclChar = 0 in ncclDataType_t)
struct NcclId {
  char internal[128];
};
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(void** comm, int nranks, NcclId id, int rank);
typedef int (*CommDestroyFn)(void* comm);
typedef int (*AllGatherFn)(const void* send, void* recv, size_t count, int dtype, void* comm, cudaStream_t stream);
typedef const char* (*GetErrorStringFn)(int);

struct Nccl {
  void* handle = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  AllGatherFn all_gather = nullptr;
  GetErrorStringFn error_string = nullptr;
  std::string why;  // why it could not be loaded
};

Nccl* nccl() {
  static Nccl lib;
  static std::once_flag once;
  std::call_once(once, [] {
    lib.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib.handle) lib.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib.handle) {
      const char* e = dlerror();
      lib.why = std::string("NCCL is not available: ") + (e ? e : "libnccl.so.2 not found");
      return;
    }
    lib.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(lib.handle, "ncclGetUniqueId"));
    lib.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(lib.handle, "ncclCommInitRank"));
    lib.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(lib.handle, "ncclCommDestroy"));
    lib.all_gather = reinterpret_cast<AllGatherFn>(dlsym(lib.handle, "ncclAllGather"));
    lib.error_string = reinterpret_cast<GetErrorStringFn>(dlsym(lib.handle, "ncclGetErrorString"));
    if (!lib.get_unique_id || !lib.comm_init_rank || !lib.comm_destroy || !lib.all_gather) {
      lib.why = "NCCL is not available: libnccl.so.2 lacks an entry point this library needs";
      lib.handle = nullptr;
    }
  });
  return &lib;
}

int nccl_fail(Nccl* n, const char* what, int rc) {
  return fail(FV_ERR_COMM, std::string(what) + ": " + (n->error_string ? n->error_string(rc) : "NCCL error") + " (" +
                               std::to_string(rc) + ")");
}

}  // namespace

int comm_all_gather(fv_ctx* ctx, const void* d_send, void* d_recv, size_t bytes) {
  if (!ctx->comm) return fail(FV_ERR_ARG, "the context belongs to no group (fv_ctx_comm_init)");
  Nccl* n = nccl();
  if (!n->handle) return fail(FV_ERR_COMM, n->why);
  const int rc = n->all_gather(d_send, d_recv, bytes, /* ncclChar */ 0, ctx->comm, ctx->stream);
  if (rc != 0) return nccl_fail(n, "ncclAllGather", rc);
  return FV_OK;
}

void comm_destroy(fv_ctx* ctx) {
  if (!ctx->comm) return;
  Nccl* n = nccl();
  if (n->handle) n->comm_destroy(ctx->comm);
  ctx->comm = nullptr;
  ctx->comm_rank = 0;
  ctx->comm_size = 1;
}

}  // namespace fv

extern "C" {

int fv_comm_unique_id(uint8_t* id128) {
  if (!id128) return fv::fail(FV_ERR_ARG, "fv_comm_unique_id: null argument");
  fv::Nccl* n = fv::nccl();
  if (!n->handle) return fv::fail(FV_ERR_COMM, n->why);
  fv::NcclId id;
  const int rc = n->get_unique_id(&id);
  if (rc != 0) return fv::nccl_fail(n, "ncclGetUniqueId", rc);
  std::memcpy(id128, id.internal, 128);
  return FV_OK;
}

int fv_ctx_comm_init(fv_ctx* ctx, const uint8_t* id128, int nranks, int rank) {
  if (!ctx || !id128 || nranks < 1 || rank < 0 || rank >= nranks) return fv::fail(FV_ERR_ARG, "fv_ctx_comm_init: bad argument");
  fv::CtxGuard g(ctx);
  if (ctx->comm) return fv::fail(FV_ERR_ARG, "fv_ctx_comm_init: the context already belongs to a group");
  if (nranks == 1) {
    ctx->comm_rank = 0;
    ctx->comm_size = 1;
    return FV_OK;
  }
  fv::Nccl* n = fv::nccl();
  if (!n->handle) return fv::fail(FV_ERR_COMM, n->why);
  fv::NcclId id;
  std::memcpy(id.internal, id128, 128);
  void* comm = nullptr;
  const int rc = n->comm_init_rank(&comm, nranks, id, rank);  // collective: returns when every rank has called it
  if (rc != 0) return fv::nccl_fail(n, "ncclCommInitRank", rc);
  ctx->comm = comm;
  ctx->comm_rank = rank;
  ctx->comm_size = nranks;
  return FV_OK;
}

int fv_ctx_comm_rank(const fv_ctx* ctx) { return ctx ? ctx->comm_rank : -1; }
int fv_ctx_comm_size(const fv_ctx* ctx) { return ctx ? ctx->comm_size : 0; }

}  // extern "C"
