// NCCL communicator for the tensor-/expert-parallel engine.  NCCL is bound at run time (dlopen of libnccl.so.2), so
// the library has no link-time dependency on it and shares whatever NCCL the process has already loaded.
// One process per GPU; the unique id travels between ranks outside this library (a file, a TCP store, MPI, or
// torch.distributed's broadcast of 128 bytes).
//
// The reference project has no collective communication (HTTP only).
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <mutex>
#include <new>

#include "common.h"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) return;
#define EB_SYM(field, name) *(void**)(&a.field) = dlsym(a.handle, name)
    EB_SYM(GetUniqueId, "ncclGetUniqueId");
    EB_SYM(CommInitRank, "ncclCommInitRank");
    EB_SYM(CommDestroy, "ncclCommDestroy");
    EB_SYM(CommAbort, "ncclCommAbort");
    EB_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    EB_SYM(AllReduce, "ncclAllReduce");
    EB_SYM(AllGather, "ncclAllGather");
    EB_SYM(ReduceScatter, "ncclReduceScatter");
    EB_SYM(GroupStart, "ncclGroupStart");
    EB_SYM(GroupEnd, "ncclGroupEnd");
    EB_SYM(GetErrorString, "ncclGetErrorString");
#undef EB_SYM
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.CommAbort && a.CommGetAsyncError && a.AllReduce &&
           a.AllGather && a.ReduceScatter && a.GroupStart && a.GroupEnd && a.GetErrorString;
  });
  return a;
}

}  // namespace

struct eb_comm {
  ncclComm_t comm = nullptr;
  int rank = 0, size = 1;
};

#define EB_NCCL(expr)                                                                                   \
  do {                                                                                                  \
    ncclResult_t _r = (expr);                                                                           \
    if (_r != ncclSuccess) return eb::fail(1000 + (int32_t)_r, "%s: %s", #expr, api().GetErrorString(_r)); \
  } while (0)

extern "C" {

int32_t eb_comm_unique_id(void* h_id128) {
  EB_REQUIRE(h_id128, EB_ERR_ARG, "eb_comm_unique_id: null");
  EB_REQUIRE(api().ok, EB_ERR_NODEVICE, "eb_comm_unique_id: libnccl.so.2 could not be loaded");
  static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id is 128 bytes");
  ncclUniqueId id;
  EB_NCCL(api().GetUniqueId(&id));
  memcpy(h_id128, &id, sizeof(id));
  return EB_OK;
}

int32_t eb_comm_create(const void* h_id128, int32_t rank, int32_t size, eb_comm** out) {
  EB_REQUIRE(h_id128 && out, EB_ERR_ARG, "eb_comm_create: null");
  EB_REQUIRE(size >= 1 && rank >= 0 && rank < size, EB_ERR_ARG, "eb_comm_create: rank %d of %d", rank, size);
  EB_REQUIRE(api().ok, EB_ERR_NODEVICE, "eb_comm_create: libnccl.so.2 could not be loaded");
  eb_comm* c = new (std::nothrow) eb_comm;
  EB_REQUIRE(c, EB_ERR_NOMEM, "eb_comm_create: host allocation failed");
  c->rank = rank;
  c->size = size;
  ncclUniqueId id;
  memcpy(&id, h_id128, sizeof(id));
  ncclResult_t r = api().CommInitRank(&c->comm, size, id, rank);
  if (r != ncclSuccess) {
    delete c;
    return eb::fail(1000 + (int32_t)r, "ncclCommInitRank: %s", api().GetErrorString(r));
  }
  *out = c;
  return EB_OK;
}

int32_t eb_comm_destroy(eb_comm* c) {
  if (!c) return EB_OK;
  if (c->comm) api().CommDestroy(c->comm);
  delete c;
  return EB_OK;
}

int32_t eb_comm_info(const eb_comm* c, int32_t* rank, int32_t* size) {
  EB_REQUIRE(c, EB_ERR_ARG, "eb_comm_info: null");
  if (rank) *rank = c->rank;
  if (size) *size = c->size;
  return EB_OK;
}

int32_t eb_comm_allreduce_f32(eb_comm* c, void* d_buf, int64_t count, void* stream) {
  EB_REQUIRE(c && d_buf && count >= 0, EB_ERR_ARG, "eb_comm_allreduce_f32: bad argument");
  if (count == 0 || c->size == 1) return EB_OK;
  EB_NCCL(api().AllReduce(d_buf, d_buf, (size_t)count, ncclFloat32, ncclSum, c->comm, eb::as_stream(stream)));
  return EB_OK;
}

// In-place all-gather of up to three buffers in one NCCL group: rank r's bytes[i] bytes already sit at offset
// r * bytes[i] of buffer i; on return every rank holds all `size` slices of every buffer.
int32_t eb_comm_allgather(eb_comm* c, int32_t n_bufs, void* const* d_bufs, const int64_t* bytes_per_rank, void* stream) {
  EB_REQUIRE(c && d_bufs && bytes_per_rank && n_bufs >= 1 && n_bufs <= 3, EB_ERR_ARG, "eb_comm_allgather: bad argument");
  for (int i = 0; i < n_bufs; ++i)
    EB_REQUIRE(d_bufs[i] && bytes_per_rank[i] >= 0, EB_ERR_ARG, "eb_comm_allgather: buffer %d", i);
  if (c->size == 1) return EB_OK;
  EB_NCCL(api().GroupStart());
  ncclResult_t r = ncclSuccess;
  for (int i = 0; i < n_bufs && r == ncclSuccess; ++i)
    if (bytes_per_rank[i] > 0)
      r = api().AllGather((const char*)d_bufs[i] + (size_t)c->rank * bytes_per_rank[i], d_bufs[i], (size_t)bytes_per_rank[i],
                          ncclInt8, c->comm, eb::as_stream(stream));
  ncclResult_t re = api().GroupEnd();
  EB_NCCL(r);
  EB_NCCL(re);
  return EB_OK;
}

// In-place reduce-scatter (fp32 sum): every rank contributes size * count_per_rank floats at d_buf; rank r's sum of
// slice r lands at d_buf + r * count_per_rank (the other slices of d_buf are left undefined).
int32_t eb_comm_reduce_scatter_f32(eb_comm* c, void* d_buf, int64_t count_per_rank, void* stream) {
  EB_REQUIRE(c && d_buf && count_per_rank >= 0, EB_ERR_ARG, "eb_comm_reduce_scatter_f32: bad argument");
  if (count_per_rank == 0 || c->size == 1) return EB_OK;
  EB_NCCL(api().ReduceScatter(d_buf, (float*)d_buf + (size_t)c->rank * count_per_rank, (size_t)count_per_rank, ncclFloat32, ncclSum,
                              c->comm, eb::as_stream(stream)));
  return EB_OK;
}

// The same on bf16 elements (half the bytes on the wire; the sum is rounded to bf16 on the way).
int32_t eb_comm_reduce_scatter_bf16(eb_comm* c, void* d_buf, int64_t count_per_rank, void* stream) {
  EB_REQUIRE(c && d_buf && count_per_rank >= 0, EB_ERR_ARG, "eb_comm_reduce_scatter_bf16: bad argument");
  if (count_per_rank == 0 || c->size == 1) return EB_OK;
  EB_NCCL(api().ReduceScatter(d_buf, (uint16_t*)d_buf + (size_t)c->rank * count_per_rank, (size_t)count_per_rank, ncclBfloat16,
                              ncclSum, c->comm, eb::as_stream(stream)));
  return EB_OK;
}

// Asynchronous error of the communicator (0 = healthy).  A host that sees a non-zero value, or whose step does not
// return within its own deadline, calls eb_comm_abort and rebuilds the communicator.
int32_t eb_comm_async_error(eb_comm* c, int32_t* err) {
  EB_REQUIRE(c && err, EB_ERR_ARG, "eb_comm_async_error: null");
  ncclResult_t e = ncclSuccess;
  EB_NCCL(api().CommGetAsyncError(c->comm, &e));
  *err = (int32_t)e;
  return EB_OK;
}

int32_t eb_comm_abort(eb_comm* c) {
  EB_REQUIRE(c, EB_ERR_ARG, "eb_comm_abort: null");
  if (c->comm) {
    api().CommAbort(c->comm);
    c->comm = nullptr;
  }
  return EB_OK;
}

}  // extern "C"
