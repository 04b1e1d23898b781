// NCCL context: used ONLY to bootstrap ChunkTensors (unique id, handle
// exchange, barriers) -- never on the per-batch path.
// Replaces reference src/nccl_context.{h,cc}.  Differences: errors are returned
// instead of abort()ing (NCCL_CALL, src/dgs_headers.h:11-20); the exchange
// buffers are small device scratch instead of cudaHostRegister'ed stack
// variables (src/chunk_tensor.cc:84-89,116-130); a private non-blocking stream
// replaces the legacy default stream (src/nccl_context.cc:32).
//
// NCCL is bound at run time (dlopen of libnccl.so.2 on first use) rather than
// at link time: a process that already holds an NCCL -- PyTorch ships its own
// -- keeps using that one copy, and loading this library never drags a second,
// possibly older NCCL into the process ahead of it.
#include "comm.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "../kernels/common.cuh"

namespace dgs {
namespace {
struct Comm {
  ncclComm_t comm = nullptr;
  cudaStream_t stream = nullptr;
  float* barrier_buf = nullptr;
  int rank = 0;
  int size = 1;
  int device = -1;
  bool ready = false;
} g;

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommUserRank)(const ncclComm_t, int*) = nullptr;
  ncclResult_t (*CommCount)(const ncclComm_t, int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
} nccl;

int load_nccl() {
  if (nccl.ok) return DGS_OK;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  DGS_REQUIRE(h != nullptr, DGS_ERR_NCCL, "cannot load libnccl.so.2: %s", dlerror());
#define DGS_SYM(field, name)                                                  \
  nccl.field = reinterpret_cast<decltype(nccl.field)>(dlsym(h, name));        \
  DGS_REQUIRE(nccl.field != nullptr, DGS_ERR_NCCL, "libnccl has no symbol %s", name)
  DGS_SYM(GetUniqueId, "ncclGetUniqueId");
  DGS_SYM(CommInitRank, "ncclCommInitRank");
  DGS_SYM(CommUserRank, "ncclCommUserRank");
  DGS_SYM(CommCount, "ncclCommCount");
  DGS_SYM(CommDestroy, "ncclCommDestroy");
  DGS_SYM(Broadcast, "ncclBroadcast");
  DGS_SYM(AllGather, "ncclAllGather");
  DGS_SYM(AllReduce, "ncclAllReduce");
  DGS_SYM(GetErrorString, "ncclGetErrorString");
#undef DGS_SYM
  nccl.ok = true;
  return DGS_OK;
}

int nccl_fail(ncclResult_t r, const char* what, const char* file, int line) {
  set_error("%s:%d: %s failed: %s", file, line, what, nccl.GetErrorString ? nccl.GetErrorString(r) : "?");
  return DGS_ERR_NCCL;
}
#define DGS_NCCL_TRY(call)                                              \
  do {                                                                  \
    ncclResult_t r__ = (call);                                          \
    if (r__ != ncclSuccess) return nccl_fail(r__, #call, __FILE__, __LINE__); \
  } while (0)
}  // namespace

int comm_broadcast_bytes(void* buf, size_t nbytes, int root) {
  if (!g.ready || g.size == 1 || nbytes == 0) return DGS_OK;
  void* d = nullptr;
  DGS_CUDA_TRY(cudaMalloc(&d, nbytes));
  DGS_CUDA_TRY(cudaMemcpyAsync(d, buf, nbytes, cudaMemcpyHostToDevice, g.stream));
  DGS_NCCL_TRY(nccl.Broadcast(d, d, nbytes, ncclChar, root, g.comm, g.stream));
  DGS_CUDA_TRY(cudaMemcpyAsync(buf, d, nbytes, cudaMemcpyDeviceToHost, g.stream));
  DGS_CUDA_TRY(cudaStreamSynchronize(g.stream));
  DGS_CUDA_TRY(cudaFree(d));
  return DGS_OK;
}

int comm_allgather_bytes(const void* send, void* recv, size_t nbytes) {
  if (!g.ready || g.size == 1) {
    std::memcpy(recv, send, nbytes);
    return DGS_OK;
  }
  char* d = nullptr;
  DGS_CUDA_TRY(cudaMalloc(&d, nbytes * (g.size + 1)));
  DGS_CUDA_TRY(cudaMemcpyAsync(d, send, nbytes, cudaMemcpyHostToDevice, g.stream));
  DGS_NCCL_TRY(nccl.AllGather(d, d + nbytes, nbytes, ncclChar, g.comm, g.stream));
  DGS_CUDA_TRY(cudaMemcpyAsync(recv, d + nbytes, nbytes * g.size, cudaMemcpyDeviceToHost, g.stream));
  DGS_CUDA_TRY(cudaStreamSynchronize(g.stream));
  DGS_CUDA_TRY(cudaFree(d));
  return DGS_OK;
}
}  // namespace dgs

using namespace dgs;

extern "C" int dgs_comm_get_unique_id(int64_t* id16) {
  DGS_REQUIRE(id16 != nullptr, DGS_ERR_INVALID, "dgs_comm_get_unique_id: null output");
  static_assert(sizeof(ncclUniqueId) == 16 * sizeof(int64_t), "unique id is 128 bytes");
  int rc = load_nccl();
  if (rc != DGS_OK) return rc;
  ncclUniqueId id;
  DGS_NCCL_TRY(nccl.GetUniqueId(&id));
  std::memcpy(id16, &id, sizeof(id));
  return DGS_OK;
}

extern "C" int dgs_comm_init(int64_t nranks, const int64_t* id16, int64_t rank) {
  DGS_REQUIRE(!g.ready, DGS_ERR_INVALID, "dgs_comm_init: communicator already set");
  DGS_REQUIRE(id16 != nullptr && nranks >= 1 && nranks <= DGS_MAX_PARTS && rank >= 0 && rank < nranks,
              DGS_ERR_INVALID, "dgs_comm_init: nranks=%lld rank=%lld (at most %d ranks)",
              (long long)nranks, (long long)rank, DGS_MAX_PARTS);
  int rc = load_nccl();
  if (rc != DGS_OK) return rc;
  ncclUniqueId id;
  std::memcpy(&id, id16, sizeof(id));
  DGS_CUDA_TRY(cudaGetDevice(&g.device));
  DGS_NCCL_TRY(nccl.CommInitRank(&g.comm, static_cast<int>(nranks), id, static_cast<int>(rank)));
  DGS_NCCL_TRY(nccl.CommUserRank(g.comm, &g.rank));
  DGS_NCCL_TRY(nccl.CommCount(g.comm, &g.size));
  DGS_CUDA_TRY(cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking));
  DGS_CUDA_TRY(cudaMalloc(&g.barrier_buf, sizeof(float)));
  DGS_CUDA_TRY(cudaMemset(g.barrier_buf, 0, sizeof(float)));
  g.ready = true;
  return DGS_OK;
}

extern "C" int dgs_comm_barrier(void) {
  if (!g.ready || g.size == 1) return DGS_OK;
  DGS_NCCL_TRY(nccl.AllReduce(g.barrier_buf, g.barrier_buf, 1, ncclFloat, ncclSum, g.comm, g.stream));
  DGS_CUDA_TRY(cudaStreamSynchronize(g.stream));
  return DGS_OK;
}

extern "C" int dgs_comm_rank(void) { return g.ready ? g.rank : 0; }
extern "C" int dgs_comm_size(void) { return g.ready ? g.size : 1; }

extern "C" int dgs_comm_destroy(void) {
  if (!g.ready) return DGS_OK;
  g.ready = false;
  cudaFree(g.barrier_buf);
  cudaStreamDestroy(g.stream);
  nccl.CommDestroy(g.comm);
  g = Comm();
  return DGS_OK;
}
