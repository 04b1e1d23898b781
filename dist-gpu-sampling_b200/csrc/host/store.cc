// HMGStore: the memory behind one ChunkTensor.
//
// Replaces ChunkTensor's constructor, LoadFromTensor, the two view getters and
// _Free (reference src/chunk_tensor.cc:37-263) and the cudaMalloc bookkeeping
// of src/cuda_context.h:11-38.
//
// Same placement: the first `threshold` elements are split into equal,
// contiguous per-GPU chunks (cudaMalloc, peers mapped with cudaIpc handles that
// are exchanged through the bootstrap communicator); the rest is a pinned
// shared host tail every rank maps (SysV segment + cudaHostRegister).
//
// Different:
//   * kernels get a by-value dgs_chunk_desc instead of a pointer to a
//     device-resident accessor struct, so nothing is allocated for it;
//   * all ranks first compare their (shape, element size, capacity): a
//     mismatch returns DGS_ERR_MISMATCH on every rank instead of mapping
//     inconsistent chunks;
//   * the SysV segment is created with IPC_PRIVATE (no key collisions) and
//     marked for removal as soon as every rank has attached, so a crashed rank
//     cannot leak it; a single-rank store uses anonymous memory;
//   * LoadFromTensor never passes a negative size when a trailing chunk is
//     empty (total=5, world=4 in the reference: src/chunk_tensor.cc:189-190);
//   * failures are returned as codes, nothing exits the process.
#include <sys/ipc.h>
#include <sys/mman.h>
#include <sys/shm.h>

#include <atomic>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <new>

#include "../kernels/common.cuh"
#include "comm.h"

struct dgs_store {
  int64_t shape[2] = {0, 0};
  int32_t ndim = 0;
  int32_t esz = 0;
  int64_t elem_stride = 1;
  int64_t total = 0, each = 0, threshold = 0, host_elems = 0;
  int32_t world = 1, rank = 0;
  void* dev[DGS_MAX_PARTS] = {nullptr};
  void* host = nullptr;         // host address of the tail
  void* host_dev = nullptr;     // device-visible address of the tail
  bool host_registered = false;
  size_t host_reg_piece = 0;    // 0: one registration for the whole tail, else registered in pieces of this size
  bool host_is_shm = false;
  size_t host_bytes = 0;
  size_t local_bytes = 0;
  bool peers_open = false;
};

namespace dgs {
namespace {
std::atomic<int64_t> g_allocated{0};

// Chunks are allocated in whole 2 MB units.  A peer that opens the cudaIpc
// handle of an allocation whose size is not a multiple of 2 MB ends up with a
// small-page mapping: measured on B200, random 8-byte reads over a 12.8e9-byte
// peer chunk ran at 75 M/s, over a 13 GiB chunk at 6.4 G/s.  The bookkeeping
// (dgs_alloc_current_bytes) keeps counting the bytes that were asked for.
constexpr size_t kChunkGranularity = size_t(2) << 20;

int tracked_malloc(void** p, size_t bytes) {
  *p = nullptr;
  if (bytes == 0) return DGS_OK;
  const size_t padded = (bytes + kChunkGranularity - 1) / kChunkGranularity * kChunkGranularity;
  DGS_CUDA_TRY(cudaMalloc(p, padded));
  g_allocated += static_cast<int64_t>(bytes);
  return DGS_OK;
}
void tracked_free(void* p, size_t bytes) {
  if (p == nullptr) return;
  cudaFree(p);
  g_allocated -= static_cast<int64_t>(bytes);
}

// Host-side failure injection for the tests of the collective error path: with
// DGS_TEST_REFUSE_HOST_REGISTER=<rank> in the environment that rank treats the pinning of the host tail
// as refused by the OS.  Nothing on the GPU is touched; read at every call so a test can set and clear it.
bool host_register_refused(int rank) {
  const char* e = std::getenv("DGS_TEST_REFUSE_HOST_REGISTER");
  return e != nullptr && e[0] != '\0' && std::atoi(e) == rank;
}

struct Meta {
  int64_t total, cap, shape0, shape1;
  int32_t esz, ndim;
};

// Release everything this rank holds; no collectives (used on error paths and
// by destroy after its barriers).
void release_local(dgs_store* s) {
  if (s->host != nullptr) {
    if (s->host_registered) {
      if (s->host_reg_piece == 0) {
        cudaHostUnregister(s->host);
      } else {
        for (size_t off = 0; off < s->host_bytes; off += s->host_reg_piece)
          cudaHostUnregister(static_cast<char*>(s->host) + off);
      }
    }
    if (s->host_is_shm) shmdt(s->host);
    else munmap(s->host, s->host_bytes);
    s->host = nullptr;
  }
  if (s->peers_open)
    for (int i = 0; i < s->world; ++i)
      if (i != s->rank && s->dev[i] != nullptr) cudaIpcCloseMemHandle(s->dev[i]);
  s->peers_open = false;
}
}  // namespace
}  // namespace dgs

using namespace dgs;

extern "C" int dgs_placement(int64_t total, int32_t esz, int64_t cap_bytes, int32_t world,
                             int64_t* each, int64_t* threshold, int64_t* host_elems) {
  DGS_REQUIRE(total >= 0 && esz > 0 && cap_bytes >= 0 && world >= 1, DGS_ERR_INVALID,
              "dgs_placement: total=%lld esz=%d capacity=%lld world=%d", (long long)total, esz,
              (long long)cap_bytes, world);
  int64_t e = cap_bytes / esz;
  int64_t t = e * world;
  if (t > total) {
    t = total;
    e = (total + world - 1) / world;
  }
  if (each) *each = e;
  if (threshold) *threshold = t;
  if (host_elems) *host_elems = total - t;
  return DGS_OK;
}

extern "C" int64_t dgs_alloc_current_bytes(void) { return g_allocated.load(); }

extern "C" int dgs_store_create(const int64_t* shape, int32_t ndim, int32_t esz,
                                int64_t capacity_per_gpu_bytes, dgs_store** out) {
  DGS_REQUIRE(out != nullptr && shape != nullptr, DGS_ERR_INVALID, "dgs_store_create: null argument");
  *out = nullptr;
  DGS_REQUIRE(ndim == 1 || ndim == 2, DGS_ERR_INVALID, "ChunkTensor needs 1 or 2 dims, got %d", ndim);
  DGS_REQUIRE(capacity_per_gpu_bytes >= 0, DGS_ERR_INVALID, "capacity_per_gpu must be >= 0");
  DGS_REQUIRE(esz_log2(esz) >= 0, DGS_ERR_UNSUPPORTED, "element size %d is not supported", esz);
  for (int i = 0; i < ndim; ++i)
    DGS_REQUIRE(shape[i] >= 0, DGS_ERR_INVALID, "negative dimension %lld", (long long)shape[i]);

  dgs_store* s = new (std::nothrow) dgs_store();
  DGS_REQUIRE(s != nullptr, DGS_ERR_INVALID, "out of host memory");
  s->ndim = ndim;
  s->esz = esz;
  s->world = dgs_comm_size();
  s->rank = dgs_comm_rank();
  s->total = 1;
  for (int i = 0; i < ndim; ++i) {
    s->shape[i] = shape[i];
    s->total *= shape[i];
  }
  s->elem_stride = ndim == 2 ? shape[1] : 1;  // strides_[0], src/chunk_tensor.cc:46-52
  dgs_placement(s->total, esz, capacity_per_gpu_bytes, s->world, &s->each, &s->threshold, &s->host_elems);

  int rc = DGS_OK;
  // ---- every rank must describe the same tensor ----
  if (s->world > 1) {
    Meta mine{s->total, capacity_per_gpu_bytes, s->shape[0], s->shape[1], esz, ndim};
    Meta all[DGS_MAX_PARTS];
    rc = comm_allgather_bytes(&mine, all, sizeof(Meta));
    if (rc == DGS_OK)
      for (int i = 0; i < s->world; ++i)
        if (std::memcmp(&all[i], &mine, sizeof(Meta)) != 0) {
          set_error("ChunkTensor metadata differs between rank %d and rank %d", s->rank, i);
          rc = DGS_ERR_MISMATCH;
          break;
        }
    // make the verdict collective: one rank's mismatch fails every rank
    int32_t verdicts[DGS_MAX_PARTS];
    int32_t v = rc;
    int rc2 = comm_allgather_bytes(&v, verdicts, sizeof(v));
    if (rc == DGS_OK && rc2 != DGS_OK) rc = rc2;
    if (rc == DGS_OK)
      for (int i = 0; i < s->world; ++i)
        if (verdicts[i] != DGS_OK) {
          set_error("ChunkTensor creation rejected on rank %d (code %d)", i, verdicts[i]);
          rc = verdicts[i];
          break;
        }
    if (rc != DGS_OK) {
      delete s;
      return rc;
    }
  }

  // ---- host tail ----
  if (s->host_elems > 0) {
    s->host_bytes = static_cast<size_t>(s->host_elems) * esz;
    if (s->world == 1) {
      void* p = mmap(nullptr, s->host_bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
      if (p == MAP_FAILED) {
        set_error("host tail: mmap of %zu bytes failed: %s", s->host_bytes, std::strerror(errno));
        rc = DGS_ERR_SHM;
      } else {
        s->host = p;
      }
    } else {
      int shmid = -1;
      if (s->rank == 0) {
        shmid = shmget(IPC_PRIVATE, s->host_bytes, IPC_CREAT | IPC_EXCL | 0600);
        if (shmid < 0) set_error("host tail: shmget of %zu bytes failed: %s", s->host_bytes, std::strerror(errno));
      }
      rc = comm_broadcast_bytes(&shmid, sizeof(shmid), 0);
      if (rc == DGS_OK && shmid < 0) {
        if (s->rank != 0) set_error("host tail: rank 0 could not create the shared segment");
        rc = DGS_ERR_SHM;
      }
      if (rc == DGS_OK) {
        void* p = shmat(shmid, nullptr, 0);
        if (p == reinterpret_cast<void*>(-1)) {
          set_error("host tail: shmat failed: %s", std::strerror(errno));
          rc = DGS_ERR_SHM;
        } else {
          s->host = p;
          s->host_is_shm = true;
        }
        // all ranks have tried to attach: mark the segment for removal now, it
        // lives on until the last detach
        int brc = dgs_comm_barrier();
        if (s->rank == 0) shmctl(shmid, IPC_RMID, nullptr);
        if (rc == DGS_OK) rc = brc;
      }
    }
    if (rc == DGS_OK) {
      const bool refused = host_register_refused(s->rank);  // injected: as if pinning had failed for good
      cudaError_t e = refused ? cudaErrorMemoryAllocation
                              : cudaHostRegister(s->host, s->host_bytes, cudaHostRegisterDefault);
      if (e != cudaSuccess && !refused) {
        // Seen on a 2-GPU run: pinning a 6.7 GB shared segment in one call failed with
        // cudaErrorOperatingSystem while several ranks were pinning the same pages.  Registering the
        // tail in 1 GiB pieces asks the OS for far less at a time; with UVA the pieces form one
        // device-visible range at the host address.
        cudaGetLastError();
        int uva_same_ptr = 0, dev_id = 0;
        cudaGetDevice(&dev_id);
        cudaDeviceGetAttribute(&uva_same_ptr, cudaDevAttrCanUseHostPointerForRegisteredMem, dev_id);
        const size_t piece = size_t(1) << 30;
        size_t done = 0;
        if (uva_same_ptr) {
          e = cudaSuccess;
          for (; done < s->host_bytes && e == cudaSuccess; done += piece) {
            const size_t len = s->host_bytes - done < piece ? s->host_bytes - done : piece;
            e = cudaHostRegister(static_cast<char*>(s->host) + done, len, cudaHostRegisterDefault);
          }
          if (e == cudaSuccess) {
            s->host_reg_piece = piece;
          } else {
            for (size_t off = 0; off + piece < done; off += piece) cudaHostUnregister(static_cast<char*>(s->host) + off);
          }
        }
      }
      if (e != cudaSuccess) {
        rc = cuda_fail(e, "cudaHostRegister(host tail)", __FILE__, __LINE__);
      } else if (s->host_reg_piece != 0) {
        s->host_registered = true;
        s->host_dev = s->host;
      } else {
        s->host_registered = true;
        e = cudaHostGetDevicePointer(&s->host_dev, s->host, 0);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaHostGetDevicePointer", __FILE__, __LINE__);
      }
    }
  }

  // ---- device chunk + peer mappings ----
  // (entered by every rank even after a local failure, so that the collective
  // handle exchange below never leaves a peer waiting)
  if (s->each > 0) {
    s->local_bytes = static_cast<size_t>(s->each) * esz;
    if (rc == DGS_OK) rc = tracked_malloc(&s->dev[s->rank], s->local_bytes);
    if (rc == DGS_OK) {
      // same fill as the reference (src/chunk_tensor.cc:108)
      cudaError_t e = cudaMemset(s->dev[s->rank], 0xFF, s->local_bytes);
      // the fill runs on the legacy default stream, the exchanges below on the communicator's own
      // non-blocking stream: finish the fill here, so that nothing a peer writes into this chunk once the
      // constructor has returned on its side (a root's LoadFromTensor, an in-place fill) can be overtaken by it
      if (e == cudaSuccess) e = cudaDeviceSynchronize();
      if (e != cudaSuccess) rc = cuda_fail(e, "cudaMemset(chunk)", __FILE__, __LINE__);
    }
    if (s->world > 1) {
      // exchange handles even after a local failure so that no rank is left waiting
      struct Msg {
        cudaIpcMemHandle_t h;
        int32_t ok;
      } mine, all[DGS_MAX_PARTS];
      std::memset(&mine, 0, sizeof(mine));
      mine.ok = 0;
      if (rc == DGS_OK) {
        cudaError_t e = cudaIpcGetMemHandle(&mine.h, s->dev[s->rank]);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaIpcGetMemHandle", __FILE__, __LINE__);
        else mine.ok = 1;
      }
      int rc2 = comm_allgather_bytes(&mine, all, sizeof(Msg));
      if (rc == DGS_OK) rc = rc2;
      if (rc == DGS_OK)
        for (int i = 0; i < s->world; ++i)
          if (!all[i].ok) {
            set_error("rank %d could not allocate or export its chunk", i);
            rc = DGS_ERR_CUDA;
          }
      if (rc == DGS_OK) {
        s->peers_open = true;
        for (int i = 0; i < s->world && rc == DGS_OK; ++i) {
          if (i == s->rank) continue;
          cudaError_t e = cudaIpcOpenMemHandle(&s->dev[i], all[i].h, cudaIpcMemLazyEnablePeerAccess);
          if (e != cudaSuccess) {
            s->dev[i] = nullptr;
            rc = cuda_fail(e, "cudaIpcOpenMemHandle", __FILE__, __LINE__);
          }
        }
      }
    }
  }
  if (s->world > 1) {
    // The outcome is collective: a rank that failed in any stage above (pinning the host tail, allocating
    // or exporting its chunk, opening a peer's) fails the constructor on every rank.  Without this an
    // all-host tensor -- no handle exchange, so no `ok` flags -- could be alive on some ranks and not on
    // others, and the survivors' next collective would wait for ever.  Doubles as the closing barrier.
    int32_t verdicts[DGS_MAX_PARTS];
    const int32_t v = rc;
    const int rc2 = comm_allgather_bytes(&v, verdicts, sizeof(v));
    if (rc == DGS_OK) rc = rc2;
    if (rc == DGS_OK)
      for (int i = 0; i < s->world; ++i)
        if (verdicts[i] != DGS_OK) {
          set_error("ChunkTensor creation failed on rank %d (code %d)", i, verdicts[i]);
          rc = verdicts[i];
          break;
        }
  }
  if (rc != DGS_OK) {
    release_local(s);
    tracked_free(s->dev[s->rank], s->local_bytes);
    delete s;
    return rc;
  }
  *out = s;
  return DGS_OK;
}

extern "C" int dgs_store_destroy(dgs_store* s) {
  if (s == nullptr) return DGS_OK;
  // order of the reference (src/chunk_tensor.cc:235-263): drop the mappings,
  // wait for every rank, then free the chunk peers may still have mapped
  release_local(s);
  int rc = DGS_OK;
  if (s->world > 1) rc = dgs_comm_barrier();
  tracked_free(s->dev[s->rank], s->local_bytes);
  if (s->world > 1) {
    int brc = dgs_comm_barrier();
    if (rc == DGS_OK) rc = brc;
  }
  delete s;
  return rc;
}

extern "C" int dgs_store_desc(const dgs_store* s, dgs_chunk_desc* out) {
  DGS_REQUIRE(s != nullptr && out != nullptr, DGS_ERR_INVALID, "dgs_store_desc: null argument");
  std::memset(out, 0, sizeof(*out));
  out->total = s->total;
  out->threshold = s->threshold;
  out->each = s->each;
  out->num_parts = s->world;
  out->local_rank = s->rank;
  out->esz = s->esz;
  out->host = s->host_dev;
  for (int i = 0; i < s->world; ++i) out->dev[i] = s->dev[i];
  return DGS_OK;
}

extern "C" int64_t dgs_store_elem_stride(const dgs_store* s) { return s ? s->elem_stride : 0; }

extern "C" int dgs_store_load(dgs_store* s, const void* host_data, int64_t n_elems) {
  DGS_REQUIRE(s != nullptr, DGS_ERR_INVALID, "dgs_store_load: null store");
  DGS_REQUIRE(n_elems == s->total, DGS_ERR_INVALID, "dgs_store_load: tensor has %lld elements, store %lld",
              (long long)n_elems, (long long)s->total);
  if (s->total == 0) return DGS_OK;
  DGS_REQUIRE(host_data != nullptr, DGS_ERR_INVALID, "dgs_store_load: null data");
  const char* src = static_cast<const char*>(host_data);
  for (int i = 0; i < s->world; ++i) {
    const int64_t lo = static_cast<int64_t>(i) * s->each;
    int64_t cnt = s->total - lo;
    if (cnt > s->each) cnt = s->each;
    if (cnt <= 0) break;
    DGS_REQUIRE(s->dev[i] != nullptr, DGS_ERR_INVALID, "dgs_store_load: chunk %d is not mapped", i);
    DGS_CUDA_TRY(cudaMemcpy(s->dev[i], src + lo * s->esz, static_cast<size_t>(cnt) * s->esz,
                            cudaMemcpyHostToDevice));
  }
  if (s->host_elems > 0)
    std::memcpy(s->host, src + s->each * s->world * s->esz, static_cast<size_t>(s->host_elems) * s->esz);
  DGS_CUDA_TRY(cudaDeviceSynchronize());
  return DGS_OK;
}

extern "C" int dgs_store_host_view(const dgs_store* s, void** ptr, int64_t* n_elems) {
  DGS_REQUIRE(s != nullptr && ptr != nullptr && n_elems != nullptr, DGS_ERR_INVALID,
              "dgs_store_host_view: null argument");
  *ptr = s->host_elems > 0 ? s->host : nullptr;
  *n_elems = s->host_elems > 0 ? s->host_elems : 0;
  return DGS_OK;
}

extern "C" int dgs_store_local_view(const dgs_store* s, void** ptr, int64_t* n_elems) {
  DGS_REQUIRE(s != nullptr && ptr != nullptr && n_elems != nullptr, DGS_ERR_INVALID,
              "dgs_store_local_view: null argument");
  *ptr = s->each > 0 ? s->dev[s->rank] : nullptr;
  *n_elems = s->each > 0 ? s->each : 0;
  return DGS_OK;
}
